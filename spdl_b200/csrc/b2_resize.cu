// Fused colour conversion -> bilinear resize -> crop / letterbox -> scale/bias over a ragged batch.
//
// Semantics (the CPU restatement in the test oracle is the definition):
//   gx = crop_x + ox;  sx = max(fma(scale_x, gx + 0.5, -0.5), 0);  x0 = int(sx);
//   x1 = min(x0 + 1, src_w - 1);  wx1 = sx - x0;  wx0 = 1 - wx1      (same for y)
//   every tap is converted to 8-bit RGB exactly as the dense kernel does, then
//   top = fma(wx1, t01, wx0*t00); bot = fma(wx1, t11, wx0*t10); val = fma(wy1, bot, wy0*top)
//   an output pixel whose (gx, gy) lies outside [0, resized_w) x [0, resized_h) takes the pad
//   colour instead (only when the descriptor gives a resized size);
//   u8 output: floor(val + 0.5) clamped to 0..255; float outputs: fma(val, scale, bias).
//
// One CTA produces 4 output rows of one image (2 when the staged rows of 4 would leave few CTAs
// per SM).
//   Stage:   for each output row the CTA needs two luma rows and one or two chroma rows (two
//            planes for I420).  Warp 0 works out the distinct row spans (rows shared between
//            neighbouring output rows are fetched once), and each lane hands its span to the
//            bulk-copy engine (cp.async.bulk global -> shared, completion on one mbarrier).  The
//            spans are widened to 16-byte boundaries; global traffic is whole 16-byte segments
//            of touched rows and nothing else.
//   Table:   while the copies are in flight the CTA builds one entry per output column (tap
//            offsets and weight): the horizontal taps are the same for every row of the image.
//   Compute: a lane converts groups of four consecutive output columns.  When a row's groups fill
//            whole warps, a warp owns one output row (or half of one) and its lanes walk the row's
//            groups 32 apart, with everything that depends on the row only -- the staged row
//            addresses, the vertical weights, the destination row -- in registers; otherwise the
//            CTA's lanes take the (row, group) items of the tile in turn, so that only the tile's
//            last warp has idle lanes.  Per pixel a lane reads its column's table entry, converts
//            the four taps (the two source rows of a tap column ride in the two lanes of the packed
//            fp32 instructions) and blends; a group goes out as vector stores when it lies inside
//            the image and the destination is 16-byte aligned, element by element otherwise, so
//            no destination pointer, stride or width has an alignment requirement.
//            RGB sources (no colour conversion): a lane converts single pixels, neighbouring lanes
//            neighbouring columns, whose taps lie a few bytes apart in the staged rows (far fewer
//            shared-memory wavefronts per tap load); elements are stored one by one.
#include <cuda_fp16.h>

#include <atomic>
#include <type_traits>

#include "b2_common.cuh"

namespace b2 {
namespace {

struct ResizeParams {
  const uint8_t* base;
  const b2_image_desc* descs;
  int out_w, out_h;
  ColorMat mat;
  void* dst;
  long long image_stride, group_stride;  // elements
  long long chan_off[3];                 // element offset of colour channel R, G, B in an image
  int row_stride, px_stride;             // elements between output rows / pixels of one channel
  int frames_per_group;                  // > 1: image i sits at (i / T) * group + (i % T) * image
  int first_image;                       // index of blockIdx.y == 0 in the caller's table
  float ch_scale[3], ch_bias[3];         // per colour channel; scale carries the 2^24 of kTapScale
  float ch_pad[3];                       // pad colour per channel, scaled by 2^-24 like the taps
  int span_cap;                          // bytes reserved per staged row span (multiple of 16)
  int span_cap2;                         // I420: bytes reserved per staged row of the half-width
                                         // planes (span_cap covers the first plane only)
  int vec_store;                         // 1: whole groups of four pixels may use vector stores
  int rows;                              // output rows per tile: 4, or 2 for wide sources
  int tiles;                             // tiles a CTA converts, one after the other
  int flat;                              // 1: lanes take the (row, group) items of a tile in turn
  unsigned groups_recip;                 // 2^32 / groups + 1: item / groups by multiply-high
  const int* luma_map;                   // optional: where source row r of the first plane is
  const int* chroma_map;                 // ... and of the half-height planes (row-sparse sources)
  int* status;                           // optional device word for B2_STATUS_* bits
  unsigned wait_limit;                   // polls of a bounded wait
  int debug_flags;
  int prefetch;                          // 1: ask for the next tile's rows in L2 one tile ahead
};

constexpr int kRows = 4;  // output rows per CTA, at most

// One staged row span as the staging warp locates it.
struct SpanLoc {
  const uint8_t* src;  // 16-byte aligned start in global memory
  long long key;       // (plane, source row): equal keys are fetched once
  int bytes, head;     // bytes to copy (a multiple of 16); offset of the span's first byte in them
  float wy1;           // weight of the lower tap row
  int active;
};
constexpr int kResizeThreads = 128;
constexpr int kResizeWarps = kResizeThreads / 32;
// 128-thread CTAs, 8 resident per SM (32 warps, no spills): measured best; larger CTAs or
// tighter register caps (more warps, spills) were slower.
constexpr int kResizeMinBlocks = 8;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

struct Axis {
  int i0, i1;
  float w1;
};
// g: output coordinate in the resized grid, already as float.  No conversion instructions:
// floor() is an add of 2^23 with round-toward-zero (0 <= s < 2^22 for every coordinate inside
// the grid; whatever a nonsensical descriptor produces is clamped into [0, n_in - 1]).
__device__ __forceinline__ Axis axis_of(float scale, float g, int n_in) {
  const float s = fmaxf(__fmaf_rn(scale, __fadd_rn(g, 0.5f), -0.5f), 0.0f);
  const float t = __fadd_rz(s, kTwo23);
  int a = (int)(__float_as_uint(t) & 0x7FFFFFu);
  float fa = __fsub_rn(t, kTwo23);
  if (a > n_in - 1) {  // cannot happen for in-grid coordinates; keeps every access in bounds
    a = n_in - 1;
    fa = (float)a;
  }
  Axis r;
  r.i0 = a;
  r.i1 = min(a + 1, n_in - 1);
  r.w1 = __fsub_rn(s, fa);
  return r;
}

__device__ __forceinline__ float biased(uint32_t b) { return __uint_as_float(0x4B000000u | b); }

// Two clamped 8-bit values in 16-bit lanes -> two floats, scaled by 2^-24: a halfword n (0..255)
// read as an fp16 bit pattern is the subnormal n * 2^-24, and fp16 -> fp32 conversion is exact.
// The blend below is linear, so it runs on the scaled values (scaling by a power of two commutes
// with every rounding) and the factor 2^24 is folded into the final multiply.
constexpr float kTapScale = 16777216.0f;  // 2^24
__device__ __forceinline__ float2 halves_to_float2(uint32_t lanes) {
  return __half22float2(*reinterpret_cast<const __half2*>(&lanes));
}
// {row0, row1} channel values after the truncating clamp (see clamp2_bits), scaled by 2^-24.
__device__ __forceinline__ float2 clamp_to_float2(float2 bits) {
  return halves_to_float2(clamp2_bits(bits.x, bits.y));
}
__device__ __forceinline__ float2 x2_mul(float2 a, float2 b) {
  unsigned long long d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(pack2(a)), "l"(pack2(b)));
  return unpack2(d);
}

// Waits for the phase of an mbarrier with the given parity: at most `limit` polls, sleeping a few
// hundred nanoseconds between them (a sleeping warp takes no issue slots from its neighbours).
__device__ __forceinline__ bool bounded_wait(uint32_t bar_addr, uint32_t parity, unsigned limit) {
  for (unsigned spin = 0; spin < limit; ++spin) {
    uint32_t done;
    asm volatile(
        "{ .reg .pred P; mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2; "
        "selp.u32 %0, 1, 0, P; }"
        : "=r"(done)
        : "r"(bar_addr), "r"(parity)
        : "memory");
    if (done) return true;
    __nanosleep(spin < 64 ? 100 : 2000);
  }
  return false;
}

// ---- shared-memory loads by 32-bit shared address (no generic-pointer arithmetic) ---------------
__device__ __forceinline__ uint32_t lds_u8(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint4 lds_v4(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(a));
  return v;
}

// What warp 0 works out for each output row of a tile while it stages the rows: shared addresses
// of the staged source rows (first plane's rows y0/y1, then the second and third planes'), the
// vertical weights, and whether the row lies inside the image at all.
struct __align__(16) RowInfo {
  uint32_t row[6];
  float wy0, wy1;
};

// One tap column of one output pixel: two source rows in the two lanes -> clamped 8-bit R, G, B
// (scaled by 2^-24, see kTapScale).
template <int FMT, int ARITH, bool UV16, class M>
__device__ __forceinline__ void convert_taps(const M& m, const RowInfo& in, uint32_t sx,
                                             uint32_t ci, float2 (&t)[3]) {
  constexpr bool kYuv = FMT == B2_SRC_NV12 || FMT == B2_SRC_I420;
  if constexpr (!kYuv) {
    // already RGB: the taps are the bytes themselves (two rows into 16-bit lanes)
    if constexpr (FMT == B2_SRC_RGB_PLANAR) {
      t[0] = halves_to_float2(__byte_perm(lds_u8(in.row[0] + sx), lds_u8(in.row[1] + sx), 0x5410u));
      t[1] = halves_to_float2(__byte_perm(lds_u8(in.row[2] + ci), lds_u8(in.row[3] + ci), 0x5410u));
      t[2] = halves_to_float2(__byte_perm(lds_u8(in.row[4] + ci), lds_u8(in.row[5] + ci), 0x5410u));
    } else {
#pragma unroll
      for (int ch = 0; ch < 3; ++ch)
        t[ch] = halves_to_float2(
            __byte_perm(lds_u8(in.row[0] + sx + ch), lds_u8(in.row[1] + sx + ch), 0x5410u));
    }
  } else {
    float2 bu, bv;
    if constexpr (FMT == B2_SRC_NV12) {
      uint32_t p0, p1;  // {U, V} of row 0 / row 1
      if constexpr (UV16) {
        p0 = lds_u16(in.row[2] + ci);
        p1 = lds_u16(in.row[3] + ci);
      } else {
        p0 = lds_u8(in.row[2] + ci) | (lds_u8(in.row[2] + ci + 1) << 8);
        p1 = lds_u8(in.row[3] + ci) | (lds_u8(in.row[3] + ci + 1) << 8);
      }
      bu = make_float2(biased_byte(p0, 0), biased_byte(p1, 0));
      bv = make_float2(biased_byte(p0, 1), biased_byte(p1, 1));
    } else {
      bu = make_float2(biased(lds_u8(in.row[2] + ci)), biased(lds_u8(in.row[3] + ci)));
      bv = make_float2(biased(lds_u8(in.row[4] + ci)), biased(lds_u8(in.row[5] + ci)));
    }
    const Chroma2 ch = chroma2_of<ARITH>(m, bu, bv);
    float2 cr, cg, cb;
    pixel2_bits<ARITH>(m, make_float2(biased(lds_u8(in.row[0] + sx)), biased(lds_u8(in.row[1] + sx))),
                       ch, cr, cg, cb);
    t[0] = clamp_to_float2(cr);
    t[1] = clamp_to_float2(cg);
    t[2] = clamp_to_float2(cb);
  }
}

// Rounding / scale+bias of one blended value (scaled by 2^-24), channel c.
// u8: floor(val + 0.5) as a subnormal bit pattern (val >= 0), ready for pack4_sat.
template <int DTYPE>
__device__ __forceinline__ float finish(const ResizeParams& p, float v, int c) {
  if constexpr (DTYPE == B2_U8) return __fmul_rz(__fmaf_rn(v, kTapScale, 0.5f), __uint_as_float(1u));
  else return __fmaf_rn(v, p.ch_scale[c], p.ch_bias[c]);
}
template <int DTYPE, typename T>
__device__ __forceinline__ void store_elem(T* q, float f) {
  if constexpr (DTYPE == B2_U8) *q = (uint8_t)pack4_sat(f, 0.0f, 0.0f, 0.0f);
  else if constexpr (DTYPE == B2_F32) *q = f;
  else *q = __float2bfloat16_rn(f);
}
__device__ __forceinline__ uint32_t bf16x2_bits(float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}

// The four-pixel group g of one output row.  drow: the row in the destination; val[k][c]: pixel
// k, colour channel c.
template <int FMT, int LAYOUT, int DTYPE, int ARITH, bool UV16, typename T>
__device__ __forceinline__ void convert_group(const ResizeParams& p, const MatPairs<ARITH>& m,
                                              const RowInfo& in, uint32_t xoffs, uint32_t xw,
                                              T* drow, int g, int groups, int cin0, int cin1) {
  {
    const int ox0 = 4 * g;
    const uint4 w4 = lds_v4(xw + 16u * (uint32_t)g);
    const float w1s[4] = {__uint_as_float(w4.x), __uint_as_float(w4.y), __uint_as_float(w4.z),
                          __uint_as_float(w4.w)};
    float val[4][3];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      // entries are stored so that neighbouring lanes read neighbouring entries
      const uint4 e = lds_v4(xoffs + 16u * (uint32_t)(k * groups + g));
      const float2 wx1 = dup2(w1s[k]), wx0 = dup2(__fsub_rn(1.0f, w1s[k]));
      float2 t0[3], t1[3];  // [channel] of tap column x0 / x1, lanes = {row y0, row y1}
      convert_taps<FMT, ARITH, UV16>(m, in, e.x, e.z, t0);
      convert_taps<FMT, ARITH, UV16>(m, in, e.y, e.w, t1);
#pragma unroll
      for (int c = 0; c < 3; ++c) {
        // {top, bot} = fma(wx1, t?1, wx0 * t?0) for both rows at once
        const float2 tb = x2_fma(wx1, t1[c], x2_mul(wx0, t0[c]));
        val[k][c] = finish<DTYPE>(p, __fmaf_rn(in.wy1, tb.y, __fmul_rn(in.wy0, tb.x)), c);
      }
    }
    if (p.vec_store && ox0 >= cin0 && ox0 + 4 <= cin1) {
      // four whole pixels inside the image, 16-byte aligned destination: vector stores
      if constexpr (LAYOUT == B2_NCHW) {
#pragma unroll
        for (int c = 0; c < 3; ++c) {
          T* q = drow + p.chan_off[c] + ox0;
          if constexpr (DTYPE == B2_U8)
            *reinterpret_cast<uint32_t*>(q) = pack4_sat(val[0][c], val[1][c], val[2][c], val[3][c]);
          else if constexpr (DTYPE == B2_F32)
            *reinterpret_cast<float4*>(q) = make_float4(val[0][c], val[1][c], val[2][c], val[3][c]);
          else
            *reinterpret_cast<uint2*>(q) = make_uint2(bf16x2_bits(val[0][c], val[1][c]),
                                                      bf16x2_bits(val[2][c], val[3][c]));
        }
      } else {
        if (p.chan_off[0] != 0) {  // BGR: blue goes first
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float tmp = val[k][0];
            val[k][0] = val[k][2];
            val[k][2] = tmp;
          }
        }
        T* q = drow + 3 * ox0;
        if constexpr (DTYPE == B2_U8) {
          uint32_t* o = reinterpret_cast<uint32_t*>(q);
          o[0] = pack4_sat(val[0][0], val[0][1], val[0][2], val[1][0]);
          o[1] = pack4_sat(val[1][1], val[1][2], val[2][0], val[2][1]);
          o[2] = pack4_sat(val[2][2], val[3][0], val[3][1], val[3][2]);
        } else if constexpr (DTYPE == B2_F32) {
          float4* o = reinterpret_cast<float4*>(q);
          o[0] = make_float4(val[0][0], val[0][1], val[0][2], val[1][0]);
          o[1] = make_float4(val[1][1], val[1][2], val[2][0], val[2][1]);
          o[2] = make_float4(val[2][2], val[3][0], val[3][1], val[3][2]);
        } else {
          uint2* o = reinterpret_cast<uint2*>(q);
          o[0] = make_uint2(bf16x2_bits(val[0][0], val[0][1]), bf16x2_bits(val[0][2], val[1][0]));
          o[1] = make_uint2(bf16x2_bits(val[1][1], val[1][2]), bf16x2_bits(val[2][0], val[2][1]));
          o[2] = make_uint2(bf16x2_bits(val[2][2], val[3][0]), bf16x2_bits(val[3][1], val[3][2]));
        }
      }
      return;
    }
    // the ragged end of a row, padding columns, or a destination that is not 16-byte aligned
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int ox = ox0 + k;
      if (ox >= p.out_w) break;
      const bool inside = ox >= cin0 && ox < cin1;
#pragma unroll
      for (int c = 0; c < 3; ++c)
        store_elem<DTYPE>(drow + p.chan_off[c] + (long long)ox * p.px_stride,
                          inside ? val[k][c] : finish<DTYPE>(p, p.ch_pad[c], c));
    }
  }
}

// One output pixel (float outputs: their elements are stored one by one, so neighbouring lanes can
// take neighbouring pixels, whose taps lie a few bytes apart in the staged rows: one or two
// shared-memory wavefronts per tap load instead of one per 128 bytes of a span that is four times
// as long).  The column table is indexed by the column here.  q[c]: where the lane's column 0 of
// this pass goes for colour channel c; K: the pixel is column 32 * K further on (a compile-time
// offset).  PAD: columns outside [cin0, cin1) exist and take the pad colour.
template <int FMT, int LAYOUT, int DTYPE, int ARITH, bool UV16, bool PAD, int K, typename T>
__device__ __forceinline__ void convert_pixel(const ResizeParams& p, const MatPairs<ARITH>& m,
                                              const RowInfo& in, uint32_t xoffs, uint32_t xw,
                                              T* const (&q)[3], int ox, int cin0, int cin1) {
  constexpr int kStep = 32 * K * (LAYOUT == B2_NCHW ? 1 : 3);  // elements
  const uint4 e = lds_v4(xoffs + 16u * (uint32_t)ox);
  const float w1 = __uint_as_float(lds_u32(xw + 4u * (uint32_t)ox));
  const float2 wx1 = dup2(w1), wx0 = dup2(__fsub_rn(1.0f, w1));
  float2 t0[3], t1[3];  // [channel] of tap column x0 / x1, lanes = {row y0, row y1}
  convert_taps<FMT, ARITH, UV16>(m, in, e.x, e.z, t0);
  convert_taps<FMT, ARITH, UV16>(m, in, e.y, e.w, t1);
  const bool inside = !PAD || (ox >= cin0 && ox < cin1);
#pragma unroll
  for (int c = 0; c < 3; ++c) {
    const float2 tb = x2_fma(wx1, t1[c], x2_mul(wx0, t0[c]));
    float v = finish<DTYPE>(p, __fmaf_rn(in.wy1, tb.y, __fmul_rn(in.wy0, tb.x)), c);
    if constexpr (PAD) v = inside ? v : finish<DTYPE>(p, p.ch_pad[c], c);
    store_elem<DTYPE>(q[c] + kStep, v);
  }
}

template <int FMT, int LAYOUT, int DTYPE, int ARITH>
__global__ void __launch_bounds__(kResizeThreads, kResizeMinBlocks) resize_kernel(const ResizeParams p) {
  using T = typename OutT<DTYPE>::type;
  constexpr bool kYuv = FMT == B2_SRC_NV12 || FMT == B2_SRC_I420;
  constexpr int kPlanes = FMT == B2_SRC_NV12 ? 4 : (FMT == B2_SRC_RGB_INTERLEAVED ? 2 : 6);
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ b2_image_desc sd;
  __shared__ RowInfo s_rows[kRows];
  __shared__ int s_odd_chroma;  // a staged interleaved-chroma row of this tile has an odd address
  __shared__ SpanLoc s_next[32];  // the next tile's spans, per lane of the staging warp
  // bar[0]: the staged rows.  bar[1]: nothing ever arrives on it (B2_DEBUG_EXPIRE_WAIT).
  __shared__ __align__(8) unsigned long long bar[2];

  const int n = blockIdx.y;
  const int tid = threadIdx.x;
  if (tid < 16)
    reinterpret_cast<uint32_t*>(&sd)[tid] =
        __ldg(reinterpret_cast<const uint32_t*>(p.descs + n) + tid);
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar[0])));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar[1])));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const b2_image_desc d = sd;
  auto report = [&](int bit) {
    if (tid == 0 && p.status != nullptr) atomicOr(p.status, bit);
  };
  if (d.src_w < 1 || d.src_h < 1 || !(d.scale_x > 0.0f) || !(d.scale_y > 0.0f)) {
    report(B2_STATUS_BAD_GEOMETRY);
    return;
  }

  // Output columns / rows that map into the image; the rest is letterbox padding.
  int cin0 = 0, cin1 = p.out_w, rin0 = 0, rin1 = p.out_h;
  if (d.resized_w > 0) {
    cin0 = max(0, -d.crop_x);
    cin1 = min(p.out_w, d.resized_w - d.crop_x);
  }
  if (d.resized_h > 0) {
    rin0 = max(0, -d.crop_y);
    rin1 = min(p.out_h, d.resized_h - d.crop_y);
  }
  if (cin0 >= cin1) cin0 = cin1 = rin0 = rin1 = 0;  // nothing maps into the image: all padding
  // Source coordinates must stay where floor() by mantissa is exact (below 2^22), which also
  // makes the taps grow with the output coordinate; anything else (a scale of 1e9, an infinity)
  // is a nonsensical descriptor.
  {
    const float sx_max = __fmaf_rn(d.scale_x, (float)(d.crop_x + max(cin1, 1)) + 0.5f, -0.5f);
    const float sy_max = __fmaf_rn(d.scale_y, (float)(d.crop_y + max(rin1, 1)) + 0.5f, -0.5f);
    if (!(sx_max < 4194304.0f) || !(sy_max < 4194304.0f)) {
      report(B2_STATUS_BAD_GEOMETRY);
      return;
    }
  }

  // Horizontal extent of source pixels touched by this image's output columns.
  int xlo = 0, xhi = 1;
  if (cin0 < cin1) {
    const Axis ax_first = axis_of(d.scale_x, (float)(d.crop_x + cin0), d.src_w);
    const Axis ax_last = axis_of(d.scale_x, (float)(d.crop_x + cin1 - 1), d.src_w);
    xlo = ax_first.i0;
    xhi = ax_last.i1 + 1;  // source columns [xlo, xhi)
    if (xhi <= xlo) {      // taps that do not grow with the column: a nonsensical descriptor
      report(B2_STATUS_BAD_GEOMETRY);
      return;
    }
  }
  // byte range of the first plane's rows, and of the other planes' rows
  const int blo = FMT == B2_SRC_RGB_INTERLEAVED ? 3 * xlo : xlo;
  const int bhi = FMT == B2_SRC_RGB_INTERLEAVED ? 3 * xhi : xhi;
  const int cxlo = FMT == B2_SRC_NV12 ? (xlo & ~1) : (FMT == B2_SRC_I420 ? (xlo >> 1) : xlo);
  const int cxhi = FMT == B2_SRC_NV12   ? (((xhi - 1) & ~1) + 2)
                   : FMT == B2_SRC_I420 ? (((xhi - 1) >> 1) + 1)
                                        : xhi;
  // A descriptor wider than the caller's max_src_w would overrun the staging rows: such an image
  // is skipped (its output is left untouched) rather than allowed to write out of bounds.
  // I420's second and third plane have rows half as wide, and slots half as large
  constexpr bool kHalfSlots = FMT == B2_SRC_I420;
  constexpr bool kLocateAhead = FMT != B2_SRC_RGB_INTERLEAVED;
  // a lane converts single pixels (convert_pixel) instead of groups of four
  constexpr bool kLanePixels = FMT == B2_SRC_RGB_INTERLEAVED || FMT == B2_SRC_RGB_PLANAR;
  if (bhi - blo + 15 > p.span_cap ||
      cxhi - cxlo + 15 > (kHalfSlots ? p.span_cap2 : p.span_cap)) {
    report(B2_STATUS_IMAGE_TOO_WIDE);
    return;
  }

  // Column table, one entry per output column (the horizontal taps are the same for every row of
  // the image): byte offsets of the two tap columns in a staged first-plane row (x, y) and in a
  // staged second/third-plane row (z, w), and the weight of the second tap.  Columns are handled
  // in groups of four by one lane; entry k of group g sits at [k * groups + g] so that the lanes
  // of a warp read neighbouring entries, and the four weights of a group form one vector.
  const int groups = (p.out_w + 3) >> 2;
  const uint32_t sbase = smem_u32(smem);
  const uint32_t xoffs =
      sbase + (uint32_t)(kHalfSlots ? p.rows * (2 * p.span_cap + (kPlanes - 2) * p.span_cap2)
                                    : p.rows * kPlanes * p.span_cap);
  const uint32_t xw = xoffs + 64u * (uint32_t)groups;
  const int warp = tid >> 5, lane = tid & 31;
  const int r = warp % p.rows;  // p.rows is 2 or 4: the output row of a tile this warp converts
  const int g0 = lane + 32 * (warp / p.rows);
  const int gstep = 32 * (kResizeWarps / p.rows);
  long long img = (long long)p.first_image + n;
  if (p.frames_per_group > 1) {
    const long long grp = img / p.frames_per_group;
    img = grp * p.group_stride + (img - grp * p.frames_per_group) * p.image_stride;
  } else {
    img *= p.image_stride;
  }
  T* const dimg = static_cast<T*>(p.dst) + img;
  const MatPairs<ARITH> m(p.mat);  // the coefficients as register pairs, built once

  // Where the staged span of plane slot pl (0/1: first plane, 2/3: second, 4/5: third; odd slots
  // hold the lower tap row) starts for source row yrow: the 16-byte aligned address to copy from,
  // the bytes to copy (a multiple of 16) and how far into them the span begins (head).  key
  // identifies (plane, row) for finding spans that several output rows share.  With row maps the
  // caller stored only the touched rows, back to back; a row the map does not cover is a hole:
  // the span then stays inside the buffer (row 0) and the caller reports it.
  auto span_start = [&](int yrow, int pl, long long& key, bool& hole, int& bytes,
                        int& head) -> const uint8_t* {
    const uint8_t* row;
    int lo, n;
    if (pl < 2) {
      key = yrow;
      int at = p.luma_map != nullptr ? __ldg(p.luma_map + yrow) : yrow;
      hole = at < 0;
      row = p.base + d.y_off + (size_t)max(at, 0) * d.y_pitch;
      lo = blo;
      n = bhi - blo;
    } else {
      const int plane = pl < 4 ? 1 : 2;
      const int prow = kYuv ? yrow >> 1 : yrow;  // chroma planes are half height
      key = ((long long)plane << 32) | (uint32_t)prow;
      const int* map = kYuv ? p.chroma_map : p.luma_map;
      int at = map != nullptr ? __ldg(map + prow) : prow;
      hole = at < 0;
      row = p.base + (plane == 1 ? d.u_off : d.v_off) + (size_t)max(at, 0) * d.uv_pitch;
      lo = cxlo;
      n = cxhi - cxlo;
    }
    head = (int)((uintptr_t)(row + lo) & 15);
    bytes = (n + head + 15) & ~15;
    return row + lo - head;
  };

  // A CTA converts p.tiles consecutive tiles of p.rows output rows, one after the other through
  // the same staging buffer: what depends on the image only (descriptor, geometry, the column
  // table) is then worked out once for all of them.
  for (int tile = 0; tile < p.tiles; ++tile) {
    const int oy0 = (blockIdx.x * p.tiles + tile) * p.rows;
    if (oy0 >= p.out_h) break;
    const int rows_here = min(p.rows, p.out_h - oy0);
    if (tile > 0) __syncthreads();  // every warp is done with the rows of the previous tile
    bool arrived = true;
    if (tid < 32) {
      const int sr = lane / kPlanes, pl = lane - sr * kPlanes;
      // Locating a span (tap rows, row maps, addresses) is the long part of staging, and the
      // other warps wait for it.  For the planar formats (16-24 spans per tile) the spans of tile
      // t + 1 are therefore located while the copies of tile t are in flight and kept in shared
      // memory (one entry per lane, read back by the lane that wrote it), so that a tile's
      // copies start as soon as its buffer is free: 1.5 % faster.  Interleaved RGB (two long
      // spans per output row) gains nothing from that but 4.5 % from having the next tile's rows
      // fetched into L2 early, which in turn costs the planar formats' four-row tiles 2-3 %.
      auto locate = [&](int oy) {
        SpanLoc L;
        L.src = nullptr;
        L.key = -1 - lane;  // unique for idle lanes
        L.bytes = L.head = 0;
        L.wy1 = 0.0f;
        L.active = lane < p.rows * kPlanes && oy >= rin0 && oy < rin1;
        if (L.active) {
          const Axis ay = axis_of(d.scale_y, (float)(d.crop_y + oy), d.src_h);
          L.wy1 = ay.w1;
          bool hole;
          L.src = span_start((pl & 1) ? ay.i1 : ay.i0, pl, L.key, hole, L.bytes, L.head);
          if (hole && p.status != nullptr) atomicOr(p.status, B2_STATUS_BAD_GEOMETRY);
        }
        return L;
      };
      const SpanLoc cur = tile == 0 || !kLocateAhead ? locate(oy0 + sr) : s_next[lane];
      const bool active = cur.active;
      const long long key = cur.key;
      const uint8_t* const src = cur.src;  // 16-byte aligned start of the span in global memory
      const int bytes = cur.bytes, head = cur.head;
      if (active && pl == 0) {
        s_rows[sr].wy0 = __fsub_rn(1.0f, cur.wy1);
        s_rows[sr].wy1 = cur.wy1;
      }
      // the first lane holding a given (plane, source row) fetches it; the others alias its slot
      const unsigned same = __match_any_sync(0xffffffffu, key);
      const int owner = __ffs(same) - 1;
      const bool fetch = active && owner == lane;
      // every lane owns a slot; with half-size slots the first-plane slots come first
      uint32_t slot, owner_slot;
      if constexpr (kHalfSlots) {
        slot = sbase + (uint32_t)(pl < 2 ? (2 * sr + pl) * p.span_cap
                                         : 2 * p.rows * p.span_cap +
                                               ((kPlanes - 2) * sr + pl - 2) * p.span_cap2);
        owner_slot = __shfl_sync(0xffffffffu, slot, owner);
      } else {
        slot = sbase + (uint32_t)(lane * p.span_cap);
        owner_slot = sbase + (uint32_t)(owner * p.span_cap);
      }
      if (active) s_rows[sr].row[pl] = owner_slot + (uint32_t)head;
      if constexpr (FMT == B2_SRC_NV12) {
        const bool odd = __any_sync(0xffffffffu, active && pl >= 2 && (head & 1));
        if (lane == 0) s_odd_chroma = odd;
      }
      const unsigned total = __reduce_add_sync(0xffffffffu, fetch ? (unsigned)bytes : 0u);
      if (tile > 0)  // order the other warps' reads of the buffer before the engine's writes
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      if (lane == 0)
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(
                         smem_u32(&bar[0])),
                     "r"(total)
                     : "memory");
      __syncwarp();
      if (fetch)
        // The source must allow reads of every aligned 16-byte segment that holds at least one
        // byte of a touched row (true of any allocation that starts and ends on such boundaries).
        asm volatile(
            "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
                "r"(slot),
            "l"(src), "r"(bytes), "r"(smem_u32(&bar[0]))
            : "memory");
      if ((kLocateAhead || p.prefetch) && tile + 1 < p.tiles && oy0 + p.rows < p.out_h) {
        const SpanLoc nxt = locate(oy0 + p.rows + sr);
        if constexpr (kLocateAhead) s_next[lane] = nxt;
        // ... and, where a tile is short next to the latency of its copies, asked for in L2
        if (p.prefetch && nxt.active)
          asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(nxt.src), "r"(nxt.bytes)
                       : "memory");
      }
    }
    if (tile == 0) {
      // the column table, while the first copies are in flight
      for (int ox = tid; ox < 4 * groups; ox += kResizeThreads) {
        const int oxc = min(max(ox, cin0), max(cin1 - 1, cin0));  // padding repeats an edge column
        const Axis ax = axis_of(d.scale_x, (float)(d.crop_x + oxc), d.src_w);
        // inside [xlo, xhi) by construction; the clamp keeps a nonsensical descriptor in the rows
        const int i0 = min(max(ax.i0, xlo), xhi - 1), i1 = min(max(ax.i1, xlo), xhi - 1);
        const int m3 = FMT == B2_SRC_RGB_INTERLEAVED ? 3 : 1;
        const uint32_t x0 = (uint32_t)(m3 * (i0 - xlo)), x1 = (uint32_t)(m3 * (i1 - xlo));
        uint32_t c0, c1;
        if constexpr (FMT == B2_SRC_NV12) {
          c0 = (uint32_t)((i0 & ~1) - cxlo);
          c1 = (uint32_t)((i1 & ~1) - cxlo);
        } else if constexpr (FMT == B2_SRC_I420) {
          c0 = (uint32_t)((i0 >> 1) - cxlo);
          c1 = (uint32_t)((i1 >> 1) - cxlo);
        } else {
          c0 = x0;
          c1 = x1;
        }
        const int grp = ox >> 2, k = ox & 3;
        reinterpret_cast<uint4*>(smem + (xoffs - sbase))[kLanePixels ? ox : k * groups + grp] =
            make_uint4(x0, x1, c0, c1);
        reinterpret_cast<float*>(smem + (xw - sbase))[ox] = ax.w1;
      }
    }
    // Warp 0 waits for the rows (the other warps wait at the barrier, which costs no issue
    // slots); the barrier publishes the rows, s_rows and the column table to everybody and makes
    // the outcome one decision for the whole CTA.
    if (tid < 32) arrived = bounded_wait(smem_u32(&bar[0]), (uint32_t)(tile & 1), p.wait_limit);
    if (!__syncthreads_and(arrived)) {
      // The rows did not arrive in time: report, give the copies that may still be in flight one
      // more bounded wait (shared memory must not be released under them), and leave.
      report(B2_STATUS_WAIT_EXPIRED);
      bounded_wait(smem_u32(&bar[0]), (uint32_t)(tile & 1), p.wait_limit);
      return;
    }
    if (p.debug_flags & B2_DEBUG_EXPIRE_WAIT) {
      if (!__syncthreads_and(bounded_wait(smem_u32(&bar[1]), 0u, 4u))) {
        report(B2_STATUS_WAIT_EXPIRED);
        return;
      }
    }

    // ---- compute ---------------------------------------------------------------------------------
    // interleaved chroma pairs can be fetched with one 16-bit load when the staged rows kept an
    // even address (they do whenever the source plane and pitch are even)
    const bool uv16 = FMT == B2_SRC_NV12 && !s_odd_chroma;
    if constexpr (kLanePixels) {
      // a warp (or two) per output row, its lanes on 32 consecutive columns per pass
      if (r >= rows_here) continue;
      const int oy = oy0 + r;
      T* const drow = dimg + (long long)oy * p.row_stride;
      const int nsub = kResizeWarps / p.rows;  // warps that share the row take blocks of 128
      if (oy < rin0 || oy >= rin1) {           // a row of padding
        for (int ox = g0; ox < p.out_w; ox += 32 * nsub)
#pragma unroll
          for (int c = 0; c < 3; ++c)
            store_elem<DTYPE>(drow + p.chan_off[c] + (long long)ox * p.px_stride,
                              finish<DTYPE>(p, p.ch_pad[c], c));
        continue;
      }
      const RowInfo in = s_rows[r];
      constexpr int kPx = LAYOUT == B2_NCHW ? 1 : 3;  // elements between pixels of a channel
      auto row_pixels = [&](auto pairs16, auto pad) {
        constexpr bool U16 = decltype(pairs16)::value, PAD = decltype(pad)::value;
        // columns lane, lane + 32, lane + 64, lane + 96 of a block: four independent pixels
        const int first = lane + 128 * (warp / p.rows);
        T* q[3];
#pragma unroll
        for (int c = 0; c < 3; ++c) q[c] = drow + p.chan_off[c] + (long long)first * kPx;
        for (int ox = first; ox < p.out_w; ox += 128 * nsub) {
          convert_pixel<FMT, LAYOUT, DTYPE, ARITH, U16, PAD, 0>(p, m, in, xoffs, xw, q, ox, cin0,
                                                                cin1);
          if (ox + 32 < p.out_w)
            convert_pixel<FMT, LAYOUT, DTYPE, ARITH, U16, PAD, 1>(p, m, in, xoffs, xw, q, ox + 32,
                                                                  cin0, cin1);
          if (ox + 64 < p.out_w)
            convert_pixel<FMT, LAYOUT, DTYPE, ARITH, U16, PAD, 2>(p, m, in, xoffs, xw, q, ox + 64,
                                                                  cin0, cin1);
          if (ox + 96 < p.out_w)
            convert_pixel<FMT, LAYOUT, DTYPE, ARITH, U16, PAD, 3>(p, m, in, xoffs, xw, q, ox + 96,
                                                                  cin0, cin1);
#pragma unroll
          for (int c = 0; c < 3; ++c) q[c] += 128 * nsub * kPx;
        }
      };
      const bool pad = cin0 > 0 || cin1 < p.out_w;
      if (uv16) {
        if (pad) row_pixels(std::true_type{}, std::true_type{});
        else row_pixels(std::true_type{}, std::false_type{});
      } else {
        if (pad) row_pixels(std::false_type{}, std::true_type{});
        else row_pixels(std::false_type{}, std::false_type{});
      }
      continue;
    }
    if (p.flat) {
      // The row's groups do not fill whole warps: the CTA's lanes take the (row, group) items of
      // the tile in turn instead, so that only the tile's last warp has idle lanes.
      const int items = rows_here * groups;
      for (int item = tid; item < items; item += kResizeThreads) {
        const int ir = (int)__umulhi((unsigned)item, p.groups_recip);
        const int g = item - ir * groups;
        const int oy = oy0 + ir;
        T* const drow = dimg + (long long)oy * p.row_stride;
        if (oy < rin0 || oy >= rin1) {  // a row of padding
          for (int ox = 4 * g; ox < min(4 * g + 4, p.out_w); ++ox)
#pragma unroll
            for (int c = 0; c < 3; ++c)
              store_elem<DTYPE>(drow + p.chan_off[c] + (long long)ox * p.px_stride,
                                finish<DTYPE>(p, p.ch_pad[c], c));
          continue;
        }
        const RowInfo in = s_rows[ir];
        if (uv16)
          convert_group<FMT, LAYOUT, DTYPE, ARITH, true>(p, m, in, xoffs, xw, drow, g, groups, cin0,
                                                         cin1);
        else
          convert_group<FMT, LAYOUT, DTYPE, ARITH, false>(p, m, in, xoffs, xw, drow, g, groups,
                                                          cin0, cin1);
      }
      continue;
    }
    // a warp per output row (two warps when a tile has two rows)
    if (r >= rows_here) continue;
    const int oy = oy0 + r;
    T* const drow = dimg + (long long)oy * p.row_stride;
    if (oy < rin0 || oy >= rin1) {  // a row of padding
      for (int ox = g0; ox < p.out_w; ox += gstep)
#pragma unroll
        for (int c = 0; c < 3; ++c)
          store_elem<DTYPE>(drow + p.chan_off[c] + (long long)ox * p.px_stride,
                            finish<DTYPE>(p, p.ch_pad[c], c));
      continue;
    }
    const RowInfo in = s_rows[r];
    if (uv16) {
      for (int g = g0; g < groups; g += gstep)
        convert_group<FMT, LAYOUT, DTYPE, ARITH, true>(p, m, in, xoffs, xw, drow, g, groups, cin0,
                                                       cin1);
    } else {
      for (int g = g0; g < groups; g += gstep)
        convert_group<FMT, LAYOUT, DTYPE, ARITH, false>(p, m, in, xoffs, xw, drow, g, groups, cin0,
                                                        cin1);
    }
  }
}

// cudaFuncSetAttribute is needed once per kernel and device; remembering that it has been done
// keeps it off the launch path (a bit per device index; a cache, not state a caller can observe).
template <typename K>
int allow_big_smem(K kern, int device, std::atomic<unsigned long long>& done) {
  const bool tracked = device >= 0 && device < 64;
  if (tracked && (done.load(std::memory_order_acquire) >> device & 1ull)) return B2_OK;
  B2_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024),
          "raising the shared-memory limit of the resize kernel failed");
  if (tracked) done.fetch_or(1ull << device, std::memory_order_release);
  return B2_OK;
}

template <int FMT, int LAYOUT, int DTYPE, int ARITH>
int launch_t(const b2_resize_args& a, const ResizeParams& p, size_t smem, cudaStream_t stream) {
  auto kern = resize_kernel<FMT, LAYOUT, DTYPE, ARITH>;
  static std::atomic<unsigned long long> big_smem_done{0};
  if (smem > 48 * 1024) {
    const int rc = allow_big_smem(kern, a.device, big_smem_done);
    if (rc != B2_OK) return rc;
  }
  const int row_blocks = (a.out_h + p.rows * p.tiles - 1) / (p.rows * p.tiles);
  for (int n0 = 0; n0 < a.num_images; n0 += 65535) {
    const int nn = a.num_images - n0 < 65535 ? a.num_images - n0 : 65535;
    ResizeParams q = p;
    q.descs = p.descs + n0;
    q.first_image = n0;
    kern<<<dim3(row_blocks, nn), kResizeThreads, smem, stream>>>(q);
    B2_CUDA(cudaPeekAtLastError(), "launch of the resize kernel failed");
  }
  return B2_OK;
}

template <int FMT, int LAYOUT, int ARITH>
int launch_fla(const b2_resize_args& a, const ResizeParams& p, size_t smem, cudaStream_t s) {
  switch (a.dtype) {
    case B2_U8: return launch_t<FMT, LAYOUT, B2_U8, ARITH>(a, p, smem, s);
    case B2_F32: return launch_t<FMT, LAYOUT, B2_F32, ARITH>(a, p, smem, s);
    default: return launch_t<FMT, LAYOUT, B2_BF16, ARITH>(a, p, smem, s);
  }
}
template <int FMT, int ARITH>
int launch_fa(const b2_resize_args& a, const ResizeParams& p, size_t smem, cudaStream_t s) {
  return a.layout == B2_NCHW ? launch_fla<FMT, B2_NCHW, ARITH>(a, p, smem, s)
                             : launch_fla<FMT, B2_NHWC, ARITH>(a, p, smem, s);
}

}  // namespace

int launch_resize(const b2_resize_args& a, cudaStream_t stream) {
  if (a.num_images == 0 || a.out_w == 0 || a.out_h == 0) return B2_OK;
  ResizeParams p{};
  p.base = static_cast<const uint8_t*>(a.base);
  p.descs = a.descs;
  p.out_w = a.out_w;
  p.out_h = a.out_h;
  p.mat = color_matrix(a.matrix_coeff, a.full_range, a.arith);
  p.dst = a.dst;
  const long long plane = a.dst_plane_stride ? a.dst_plane_stride : (long long)a.out_w * a.out_h;
  p.image_stride = a.dst_image_stride ? a.dst_image_stride : 3LL * a.out_w * a.out_h;
  p.group_stride = a.dst_group_stride;
  p.frames_per_group = a.frames_per_group;
  p.row_stride = a.layout == B2_NCHW ? a.out_w : 3 * a.out_w;
  p.px_stride = a.layout == B2_NCHW ? 1 : 3;
  for (int c = 0; c < 3; ++c) {
    const int slot = a.order == B2_BGR ? 2 - c : c;  // where colour channel c goes
    p.chan_off[c] = a.layout == B2_NCHW ? slot * plane : slot;
    p.ch_scale[c] = a.scale[slot] * 16777216.0f;  // the kernel blends taps scaled by 2^-24 (exact)
    p.ch_bias[c] = a.bias[slot];
    p.ch_pad[c] = a.pad_value[c] * (1.0f / 16777216.0f);
  }
  // Vector stores need every group of four pixels 16-byte aligned in the destination.
  const int esz = a.dtype == B2_U8 ? 1 : (a.dtype == B2_F32 ? 4 : 2);
  auto aligned16 = [&](long long elements) { return (elements * esz) % 16 == 0; };
  p.vec_store = a.out_w % 4 == 0 && (uintptr_t)a.dst % 16 == 0 && aligned16(p.image_stride) &&
                aligned16(p.group_stride) && aligned16(p.row_stride) &&
                (a.layout != B2_NCHW || aligned16(plane));
  p.luma_map = a.luma_row_map;
  p.chroma_map = a.chroma_row_map;
  p.status = a.status;
  p.wait_limit = 1u << 19;  // about a second of sleeping polls
  p.debug_flags = a.debug_flags;
  // A staged span holds at most max_src_w + 1 bytes (interleaved chroma rows of an odd width)
  // plus up to 15 bytes of alignment head, rounded up to whole 16-byte segments.
  const long long row_bytes =
      a.src_format == B2_SRC_RGB_INTERLEAVED ? 3LL * a.max_src_w : (long long)a.max_src_w;
  const long long span = ((row_bytes + 2 + 15 + 15) / 16) * 16;
  // the rows of I420's second and third plane are half as wide
  const long long span2 =
      a.src_format == B2_SRC_I420 ? (((a.max_src_w + 1LL) / 2 + 2 + 15 + 15) / 16) * 16 : span;
  const int planes = a.src_format == B2_SRC_NV12 ? 4 : (a.src_format == B2_SRC_RGB_INTERLEAVED ? 2 : 6);
  const size_t per_row = (size_t)(2 * span + (planes - 2) * span2);  // staging per output row
  // per column 16 bytes of offsets + 4 bytes of weight, for whole groups of four columns
  const size_t table = (size_t)((a.out_w + 3) / 4) * 80;
  // Four output rows per CTA amortise the per-CTA work best; wide sources (4K rows) take two,
  // which halves the staging buffer and lets more CTAs share an SM.
  p.rows = (size_t)kRows * per_row + table > 40 * 1024 ? 2 : kRows;
  const size_t smem = (size_t)p.rows * per_row + table;
  if (span >= 65536 || smem > 200 * 1024)
    return fail(B2_ERR_LIMIT,
                "max_src_w %d and out_w %d need %zu bytes of staging; the limit is %d bytes",
                a.max_src_w, a.out_w, smem, 200 * 1024);
  p.span_cap = (int)span;
  p.span_cap2 = (int)span2;
  p.prefetch = a.src_format == B2_SRC_RGB_INTERLEAVED || p.rows == 2;
  // Tiles per CTA: enough to spread the per-image work of a CTA over many rows, few enough to
  // leave every SM several CTAs' worth of an image batch (148 SMs x 8 resident CTAs).
  p.tiles = 8;
  while (p.tiles > 1 && (long long)a.num_images * ((a.out_h + p.rows * p.tiles - 1) /
                                                    (p.rows * p.tiles)) < 4 * 148 * 8)
    p.tiles >>= 1;
  // Items in turn when that takes fewer warp passes over a tile than a warp (or two) per row.
  // The reciprocal is exact for every item of a tile when groups >= 2 (for a single group it does
  // not fit 32 bits, and a warp per row is as good).
  const int groups = (a.out_w + 3) / 4, lanes_per_row = 32 * (kResizeWarps / p.rows);
  const int passes_flat = (p.rows * groups + 31) / 32;
  const int passes_rows = kResizeWarps * ((groups + lanes_per_row - 1) / lanes_per_row);
  p.flat = groups >= 2 && passes_flat < passes_rows;
  p.groups_recip = groups >= 2 ? (unsigned)((1ull << 32) / (unsigned)groups + 1) : 0u;
  const bool sws = a.arith == B2_ARITH_SWSCALE;
  switch (a.src_format) {
    case B2_SRC_NV12:
      return sws ? launch_fa<B2_SRC_NV12, B2_ARITH_SWSCALE>(a, p, smem, stream)
                 : launch_fa<B2_SRC_NV12, B2_ARITH_REFERENCE>(a, p, smem, stream);
    case B2_SRC_I420:
      return sws ? launch_fa<B2_SRC_I420, B2_ARITH_SWSCALE>(a, p, smem, stream)
                 : launch_fa<B2_SRC_I420, B2_ARITH_REFERENCE>(a, p, smem, stream);
    case B2_SRC_RGB_PLANAR:
      return launch_fa<B2_SRC_RGB_PLANAR, B2_ARITH_REFERENCE>(a, p, smem, stream);
    default:
      return launch_fa<B2_SRC_RGB_INTERLEAVED, B2_ARITH_REFERENCE>(a, p, smem, stream);
  }
}

}  // namespace b2

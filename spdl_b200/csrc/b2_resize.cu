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
//   Compute: a warp owns one output row (or half of one), a lane walks the row's columns 32
//            apart.  Everything that depends on the row only -- the staged row addresses, the
//            vertical weights, the destination row -- is computed once per warp and lives in
//            registers; per pixel a lane reads its column's table entry, converts the four taps
//            (the two source rows of a tap column ride in the two lanes of the packed fp32
//            instructions), blends and stores one element per channel, consecutive lanes to
//            consecutive addresses.  Stores are element-wise, so no destination pointer, stride
//            or width has an alignment requirement.
#include <cuda_fp16.h>

#include <atomic>

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
  int rows;                              // output rows per CTA: 4, or 2 for wide sources
  int* status;                           // optional device word for B2_STATUS_* bits
  unsigned wait_limit;                   // polls of about a microsecond each
  int debug_flags;
};

constexpr int kRows = 4;  // output rows per CTA, at most
constexpr int kResizeThreads = 128;
constexpr int kResizeWarps = kResizeThreads / 32;
// 128-thread CTAs, 8 resident per SM (32 warps, no spills): measured best; larger CTAs or
// tighter register caps (more warps, spills) were slower.
constexpr int kResizeMinBlocks = 8;
constexpr int kMaxSpans = kRows * 6;

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

// Waits for phase 0 of an mbarrier, at most `limit` polls of about a microsecond each.
__device__ __forceinline__ bool bounded_wait(uint32_t bar_addr, unsigned limit) {
  uint32_t done = 0;
  for (unsigned spin = 0; spin < limit && !done; ++spin)
    asm volatile(
        "{ .reg .pred P; mbarrier.try_wait.parity.shared::cta.b64 P, [%1], 0, %2; "
        "selp.u32 %0, 1, 0, P; }"
        : "=r"(done)
        : "r"(bar_addr), "r"(1000u)
        : "memory");
  return done != 0;
}

template <int FMT, int DTYPE, int ARITH>
__global__ void __launch_bounds__(kResizeThreads, kResizeMinBlocks) resize_kernel(const ResizeParams p) {
  using T = typename OutT<DTYPE>::type;
  constexpr bool kYuv = FMT == B2_SRC_NV12 || FMT == B2_SRC_I420;
  constexpr int kPlanes = FMT == B2_SRC_NV12 ? 4 : (FMT == B2_SRC_RGB_INTERLEAVED ? 2 : 6);
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ b2_image_desc sd;
  __shared__ int s_off[kMaxSpans];
  // bar[0]: the staged rows.  bar[1]: nothing ever arrives on it (B2_DEBUG_EXPIRE_WAIT).
  __shared__ __align__(8) unsigned long long bar[2];

  const int n = blockIdx.y;
  const int oy0 = blockIdx.x * p.rows;
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
  const bool any_cols = cin0 < cin1;

  // Horizontal extent of source pixels touched by this image's output columns.
  int xlo = 0, xhi = 1;
  if (any_cols) {
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
  if (bhi - blo + 15 > p.span_cap || cxhi - cxlo + 15 > p.span_cap) {
    report(B2_STATUS_IMAGE_TOO_WIDE);
    return;
  }

  const int rows_here = min(p.rows, p.out_h - oy0);
  if (tid < 32) {
    const int lane = tid;
    const int nspans = rows_here * kPlanes;
    const int r = lane / kPlanes, pl = lane - r * kPlanes;
    const int oy = oy0 + r;
    const bool active = lane < nspans && any_cols && oy >= rin0 && oy < rin1;
    long long key = -1 - lane;  // unique for idle lanes
    const uint8_t* src = nullptr;
    int lo = 0, bytes = 0, head = 0;
    if (active) {
      const Axis ay = axis_of(d.scale_y, (float)(d.crop_y + oy), d.src_h);
      const int yrow = (pl & 1) ? ay.i1 : ay.i0;
      if (pl < 2) {
        key = yrow;
        src = p.base + d.y_off + (size_t)yrow * d.y_pitch;
        lo = blo;
        bytes = bhi - blo;
      } else {
        const int plane = pl < 4 ? 1 : 2;          // second / third plane
        const int prow = kYuv ? yrow >> 1 : yrow;  // chroma planes are half height
        key = ((long long)plane << 32) | (uint32_t)prow;
        src = p.base + (plane == 1 ? d.u_off : d.v_off) + (size_t)prow * d.uv_pitch;
        lo = cxlo;
        bytes = cxhi - cxlo;
      }
      head = (int)((uintptr_t)(src + lo) & 15);
      bytes = (bytes + head + 15) & ~15;
    }
    // the first lane holding a given (plane, source row) fetches it; the others alias its slot
    const unsigned same = __match_any_sync(0xffffffffu, key);
    const int owner = __ffs(same) - 1;
    const bool fetch = active && owner == lane;
    if (lane < kMaxSpans) s_off[lane] = active ? owner * p.span_cap + head : 0;
    const unsigned total = __reduce_add_sync(0xffffffffu, fetch ? (unsigned)bytes : 0u);
    if (lane == 0)
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&bar[0])),
                   "r"(total)
                   : "memory");
    __syncwarp();
    if (fetch)
      // The source must allow reads of every aligned 16-byte segment that holds at least one
      // byte of a touched row (true of any allocation that starts and ends on such boundaries).
      asm volatile(
          "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
              smem_u32(smem + (size_t)lane * p.span_cap)),
          "l"(src + lo - head), "r"(bytes), "r"(smem_u32(&bar[0]))
          : "memory");
  }
  // While the copies are in flight: one table entry per output column (the horizontal taps are
  // the same for every row of the image): byte offsets of the two tap columns in a staged
  // first-plane row (x, y) and in a staged second/third-plane row (z, w), and the weight of the
  // second tap (negative: a padding column).
  uint4* const xoffs = reinterpret_cast<uint4*>(smem + (size_t)p.rows * kPlanes * p.span_cap);
  float* const xw = reinterpret_cast<float*>(xoffs + p.out_w);
  for (int ox = tid; ox < p.out_w; ox += kResizeThreads) {
    if (ox < cin0 || ox >= cin1) {
      xoffs[ox] = make_uint4(0u, 0u, 0u, 0u);
      xw[ox] = -1.0f;
      continue;
    }
    const Axis ax = axis_of(d.scale_x, (float)(d.crop_x + ox), d.src_w);
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
    xoffs[ox] = make_uint4(x0, x1, c0, c1);
    xw[ox] = fmaxf(ax.w1, 0.0f);
  }
  __syncthreads();  // s_off and the column table are visible
  if (!bounded_wait(smem_u32(&bar[0]), p.wait_limit)) {
    // The rows did not arrive in time: report, give the copies that may still be in flight one
    // more bounded wait (shared memory must not be released under them), and leave the tile.
    report(B2_STATUS_WAIT_EXPIRED);
    bounded_wait(smem_u32(&bar[0]), p.wait_limit);
    return;
  }
  if (p.debug_flags & B2_DEBUG_EXPIRE_WAIT) {
    if (!bounded_wait(smem_u32(&bar[1]), 4u)) {
      report(B2_STATUS_WAIT_EXPIRED);
      return;
    }
  }

  // ---- compute: a warp per output row ------------------------------------------------------------
  const int warp = tid >> 5, lane = tid & 31;
  const int r = warp % p.rows;             // p.rows is 2 or 4
  const int col0 = lane + 32 * (warp / p.rows);
  const int cstep = 32 * (kResizeWarps / p.rows);
  if (r >= rows_here) return;
  const int oy = oy0 + r;
  const ColorMat m = p.mat;
  long long img = (long long)p.first_image + n;
  if (p.frames_per_group > 1) {
    const long long g = img / p.frames_per_group;
    img = g * p.group_stride + (img - g * p.frames_per_group) * p.image_stride;
  } else {
    img *= p.image_stride;
  }
  T* const drow = static_cast<T*>(p.dst) + img + (long long)oy * p.row_stride;
  T* const d0 = drow + p.chan_off[0];
  T* const d1 = drow + p.chan_off[1];
  T* const d2 = drow + p.chan_off[2];
  auto store = [&](int ox, float v0, float v1, float v2) {  // blended values (scaled by 2^-24)
    const long long o = (long long)ox * p.px_stride;
    if constexpr (DTYPE == B2_U8) {
      // floor(val + 0.5) as a subnormal bit pattern (val >= 0), then a saturating pack
      const float unit = __uint_as_float(1u);
      const uint32_t w = pack4_sat(__fmul_rz(__fmaf_rn(v0, kTapScale, 0.5f), unit),
                                   __fmul_rz(__fmaf_rn(v1, kTapScale, 0.5f), unit),
                                   __fmul_rz(__fmaf_rn(v2, kTapScale, 0.5f), unit), 0.0f);
      d0[o] = (uint8_t)w;
      d1[o] = (uint8_t)(w >> 8);
      d2[o] = (uint8_t)(w >> 16);
    } else {
      const float f0 = __fmaf_rn(v0, p.ch_scale[0], p.ch_bias[0]);
      const float f1 = __fmaf_rn(v1, p.ch_scale[1], p.ch_bias[1]);
      const float f2 = __fmaf_rn(v2, p.ch_scale[2], p.ch_bias[2]);
      if constexpr (DTYPE == B2_F32) {
        d0[o] = f0;
        d1[o] = f1;
        d2[o] = f2;
      } else {
        d0[o] = __float2bfloat16_rn(f0);
        d1[o] = __float2bfloat16_rn(f1);
        d2[o] = __float2bfloat16_rn(f2);
      }
    }
  };
  if (!any_cols || oy < rin0 || oy >= rin1) {  // a row of padding
    for (int ox = col0; ox < p.out_w; ox += cstep) store(ox, p.ch_pad[0], p.ch_pad[1], p.ch_pad[2]);
    return;
  }

  const Axis ay = axis_of(d.scale_y, (float)(d.crop_y + oy), d.src_h);
  const float2 wy = make_float2(__fsub_rn(1.0f, ay.w1), ay.w1);  // {wy0, wy1}
  const int* so = s_off + r * kPlanes;
  const unsigned char* y0p = smem + so[0];
  const unsigned char* y1p = smem + so[1];
  const unsigned char* u0p = kPlanes > 2 ? smem + so[2] : nullptr;
  const unsigned char* u1p = kPlanes > 2 ? smem + so[3] : nullptr;
  const unsigned char* v0p = kPlanes > 4 ? smem + so[4] : nullptr;
  const unsigned char* v1p = kPlanes > 4 ? smem + so[5] : nullptr;
  // interleaved chroma pairs can be fetched with one 16-bit load when the staged rows kept an
  // even address (they do whenever the source plane and pitch are even)
  const bool uv16 = FMT == B2_SRC_NV12 && ((so[2] | so[3]) & 1) == 0;
  (void)u0p; (void)u1p; (void)v0p; (void)v1p; (void)uv16;

  for (int ox = col0; ox < p.out_w; ox += cstep) {
    const float w1 = xw[ox];
    if (w1 < 0.0f) {  // a padding column
      store(ox, p.ch_pad[0], p.ch_pad[1], p.ch_pad[2]);
      continue;
    }
    const uint4 e = xoffs[ox];
    const float2 wx1 = dup2(w1), wx0 = dup2(__fsub_rn(1.0f, w1));
    float2 t[2][3];  // [column x0/x1][channel], lanes = {row y0, row y1}, clamped 0..255
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const uint32_t sx = c ? e.y : e.x;
      const uint32_t ci = c ? e.w : e.z;
      if constexpr (!kYuv) {
        // already RGB: the taps are the bytes themselves (two rows into 16-bit lanes)
        if constexpr (FMT == B2_SRC_RGB_PLANAR) {
          t[c][0] = halves_to_float2(__byte_perm(y0p[sx], y1p[sx], 0x5410u));
          t[c][1] = halves_to_float2(__byte_perm(u0p[ci], u1p[ci], 0x5410u));
          t[c][2] = halves_to_float2(__byte_perm(v0p[ci], v1p[ci], 0x5410u));
        } else {
#pragma unroll
          for (int ch = 0; ch < 3; ++ch)
            t[c][ch] = halves_to_float2(__byte_perm(y0p[sx + ch], y1p[sx + ch], 0x5410u));
        }
      } else {
        float2 bu, bv;
        if constexpr (FMT == B2_SRC_NV12) {
          uint32_t p0, p1;  // {U, V} of row 0 / row 1
          if (uv16) {
            p0 = *reinterpret_cast<const uint16_t*>(u0p + ci);
            p1 = *reinterpret_cast<const uint16_t*>(u1p + ci);
          } else {
            p0 = u0p[ci] | ((uint32_t)u0p[ci + 1] << 8);
            p1 = u1p[ci] | ((uint32_t)u1p[ci + 1] << 8);
          }
          bu = make_float2(biased_byte(p0, 0), biased_byte(p1, 0));
          bv = make_float2(biased_byte(p0, 1), biased_byte(p1, 1));
        } else {
          bu = make_float2(biased(u0p[ci]), biased(u1p[ci]));
          bv = make_float2(biased(v0p[ci]), biased(v1p[ci]));
        }
        const Chroma2 ch = chroma2_of<ARITH>(m, bu, bv);
        float2 cr, cg, cb;
        pixel2_bits<ARITH>(m, make_float2(biased(y0p[sx]), biased(y1p[sx])), ch, cr, cg, cb);
        t[c][0] = clamp_to_float2(cr);
        t[c][1] = clamp_to_float2(cg);
        t[c][2] = clamp_to_float2(cb);
      }
    }
    float val[3];
#pragma unroll
    for (int c = 0; c < 3; ++c) {
      // {top, bot} = fma(wx1, t?1, wx0 * t?0) for both rows at once
      const float2 tb = x2_fma(wx1, t[1][c], x2_mul(wx0, t[0][c]));
      val[c] = __fmaf_rn(wy.y, tb.y, __fmul_rn(wy.x, tb.x));
    }
    store(ox, val[0], val[1], val[2]);
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

template <int FMT, int DTYPE, int ARITH>
int launch_t(const b2_resize_args& a, const ResizeParams& p, size_t smem, cudaStream_t stream) {
  auto kern = resize_kernel<FMT, DTYPE, ARITH>;
  static std::atomic<unsigned long long> big_smem_done{0};
  if (smem > 48 * 1024) {
    const int rc = allow_big_smem(kern, a.device, big_smem_done);
    if (rc != B2_OK) return rc;
  }
  const int row_blocks = (a.out_h + p.rows - 1) / p.rows;
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

template <int FMT, int ARITH>
int launch_fa(const b2_resize_args& a, const ResizeParams& p, size_t smem, cudaStream_t s) {
  switch (a.dtype) {
    case B2_U8: return launch_t<FMT, B2_U8, ARITH>(a, p, smem, s);
    case B2_F32: return launch_t<FMT, B2_F32, ARITH>(a, p, smem, s);
    default: return launch_t<FMT, B2_BF16, ARITH>(a, p, smem, s);
  }
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
  p.status = a.status;
  p.wait_limit = 1u << 20;
  p.debug_flags = a.debug_flags;
  // A staged span holds at most max_src_w + 1 bytes (interleaved chroma rows of an odd width)
  // plus up to 15 bytes of alignment head, rounded up to whole 16-byte segments.
  const long long row_bytes =
      a.src_format == B2_SRC_RGB_INTERLEAVED ? 3LL * a.max_src_w : (long long)a.max_src_w;
  const long long span = ((row_bytes + 2 + 15 + 15) / 16) * 16;
  const int planes = a.src_format == B2_SRC_NV12 ? 4 : (a.src_format == B2_SRC_RGB_INTERLEAVED ? 2 : 6);
  const size_t table = (size_t)a.out_w * 20;  // 16 bytes of offsets + 4 bytes of weight per column
  // Four output rows per CTA amortise the per-CTA work best; wide sources (4K rows) take two,
  // which halves the staging buffer and lets more CTAs share an SM.
  p.rows = (size_t)kRows * planes * span + table > 40 * 1024 ? 2 : kRows;
  const size_t smem = (size_t)p.rows * planes * span + table;
  if (span >= 65536 || smem > 200 * 1024)
    return fail(B2_ERR_LIMIT,
                "max_src_w %d and out_w %d need %zu bytes of staging; the limit is %d bytes",
                a.max_src_w, a.out_w, smem, 200 * 1024);
  p.span_cap = (int)span;
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

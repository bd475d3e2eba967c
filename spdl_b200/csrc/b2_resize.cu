// Fused colour conversion -> bilinear resize -> crop -> scale/bias over a ragged batch.
//
// Semantics (the CPU restatement in the test oracle is the definition):
//   gx = crop_x + ox;  sx = max(fma(scale_x, gx + 0.5, -0.5), 0);  x0 = int(sx);
//   x1 = min(x0 + 1, src_w - 1);  wx1 = sx - x0;  wx0 = 1 - wx1      (same for y)
//   every tap is converted to 8-bit RGB exactly as the dense kernel does, then
//   top = fma(wx1, t01, wx0*t00); bot = fma(wx1, t11, wx0*t10); val = fma(wy1, bot, wy0*top)
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
//   Compute: each thread owns four consecutive output pixels of one row.  The two source rows of
//            a tap column ride in the two lanes of the packed fp32 instructions, so one
//            instruction stream converts both rows of a column and the horizontal blend of both
//            rows; 16-byte (fp32), 8-byte (bf16) or 4-byte (u8) stores per channel.
#include <cuda_fp16.h>

#include "b2_common.cuh"

namespace b2 {
namespace {

struct ResizeParams {
  const uint8_t* base;
  const b2_image_desc* descs;
  int out_w, out_h;
  ColorMat mat;
  void* dst;
  long long dst_image_stride;
  ScaleBias sb;
  int span_cap;   // bytes reserved per staged row span (multiple of 16)
  int vec_store;  // 1: out_w % 4 == 0 and the destination is 16-byte aligned
  int rows;       // output rows per CTA: kRows, or 2 for wide sources
};

constexpr int kRows = 4;  // output rows per CTA, at most
constexpr int kResizeThreads = 128;
// 128-thread CTAs, 8 resident per SM (32 warps, 63 registers, no spills): measured best; larger
// CTAs or tighter register caps (more warps, spills) were slower.
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
// floor() is an add of 2^23 with round-toward-zero (0 <= s < 2^22 here).
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

template <int FMT, int LAYOUT, int DTYPE, bool BGR>
__global__ void __launch_bounds__(kResizeThreads, kResizeMinBlocks) resize_kernel(const ResizeParams p) {
  using T = typename OutT<DTYPE>::type;
  constexpr bool kYuv = FMT == B2_SRC_NV12 || FMT == B2_SRC_I420;
  constexpr int kPlanes = FMT == B2_SRC_NV12 ? 4 : (FMT == B2_SRC_RGB_INTERLEAVED ? 2 : 6);
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ b2_image_desc sd;
  __shared__ int s_off[kMaxSpans];
  __shared__ __align__(8) unsigned long long bar;

  const int n = blockIdx.y;
  const int oy0 = blockIdx.x * p.rows;
  const int tid = threadIdx.x;
  if (tid < 16)
    reinterpret_cast<uint32_t*>(&sd)[tid] =
        __ldg(reinterpret_cast<const uint32_t*>(p.descs + n) + tid);
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const b2_image_desc d = sd;
  if (d.src_w < 1 || d.src_h < 1) return;

  // Horizontal extent of source pixels touched by this image's output columns.
  const Axis ax_first = axis_of(d.scale_x, (float)d.crop_x, d.src_w);
  const Axis ax_last = axis_of(d.scale_x, (float)(d.crop_x + p.out_w - 1), d.src_w);
  const int xlo = ax_first.i0, xhi = ax_last.i1 + 1;  // source columns [xlo, xhi)
  // byte range of the first plane's rows, and of the other planes' rows
  const int blo = FMT == B2_SRC_RGB_INTERLEAVED ? 3 * xlo : xlo;
  const int bhi = FMT == B2_SRC_RGB_INTERLEAVED ? 3 * xhi : xhi;
  const int cxlo = FMT == B2_SRC_NV12 ? (xlo & ~1) : (FMT == B2_SRC_I420 ? (xlo >> 1) : xlo);
  const int cxhi = FMT == B2_SRC_NV12   ? (((xhi - 1) & ~1) + 2)
                   : FMT == B2_SRC_I420 ? (((xhi - 1) >> 1) + 1)
                                        : xhi;
  // A descriptor wider than the caller's max_src_w would overrun the staging rows: such an image
  // is skipped (its output is left untouched) rather than allowed to write out of bounds.
  if (bhi - blo + 15 > p.span_cap || cxhi - cxlo + 15 > p.span_cap) return;

  const int rows_here = min(p.rows, p.out_h - oy0);
  if (tid < 32) {
    const int lane = tid;
    const int nspans = rows_here * kPlanes;
    const bool active = lane < nspans;
    const int r = lane / kPlanes, pl = lane - r * kPlanes;
    long long key = -1 - lane;  // unique for idle lanes
    const uint8_t* src = nullptr;
    int lo = 0, bytes = 0, head = 0;
    if (active) {
      const Axis ay = axis_of(d.scale_y, (float)(d.crop_y + oy0 + r), d.src_h);
      const int yrow = (pl & 1) ? ay.i1 : ay.i0;
      if (pl < 2) {
        key = yrow;
        src = p.base + d.y_off + (size_t)yrow * d.y_pitch;
        lo = blo;
        bytes = bhi - blo;
      } else {
        const int plane = pl < 4 ? 1 : 2;       // second / third plane
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
    if (active) s_off[lane] = owner * p.span_cap + head;
    const unsigned total = __reduce_add_sync(0xffffffffu, fetch ? (unsigned)bytes : 0u);
    if (lane == 0)
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&bar)),
                   "r"(total)
                   : "memory");
    __syncwarp();
    if (fetch)
      // An aligned 16-byte segment that holds at least one valid byte lies inside the allocation
      // (allocations start and end on coarser boundaries), so widening never leaves it.
      asm volatile(
          "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
              smem_u32(smem + (size_t)lane * p.span_cap)),
          "l"(src + lo - head), "r"(bytes), "r"(smem_u32(&bar))
          : "memory");
  }
  // While the copies are in flight: one table entry per output column (the horizontal taps are
  // the same for every row of the image).  {x0 | x1 << 16, c0 | c1 << 16, wx1, -}: byte offsets
  // of the two tap columns in a staged first-plane row and in a staged second/third-plane row.
  uint4* xtab = reinterpret_cast<uint4*>(smem + (size_t)p.rows * kPlanes * p.span_cap);
  const int tab_groups = (p.out_w + 3) >> 2;
  for (int ox = tid; ox < p.out_w; ox += kResizeThreads) {
    const Axis ax = axis_of(d.scale_x, (float)(d.crop_x + ox), d.src_w);
    const int m3 = FMT == B2_SRC_RGB_INTERLEAVED ? 3 : 1;
    const uint32_t x0 = (uint32_t)(m3 * (ax.i0 - xlo)), x1 = (uint32_t)(m3 * (ax.i1 - xlo));
    uint32_t c0, c1;
    if constexpr (FMT == B2_SRC_NV12) {
      c0 = (uint32_t)((ax.i0 & ~1) - cxlo);
      c1 = (uint32_t)((ax.i1 & ~1) - cxlo);
    } else if constexpr (FMT == B2_SRC_I420) {
      c0 = (uint32_t)((ax.i0 >> 1) - cxlo);
      c1 = (uint32_t)((ax.i1 >> 1) - cxlo);
    } else {
      c0 = x0;
      c1 = x1;
    }
    // stored so that the four-pixel groups of neighbouring threads read neighbouring entries
    xtab[(ox & 3) * tab_groups + (ox >> 2)] =
        make_uint4(x0 | (x1 << 16), c0 | (c1 << 16), __float_as_uint(ax.w1), 0u);
  }
  __syncthreads();  // s_off and xtab are visible
  {
    // Wait for the copies, with a limit: a wait that runs out abandons the tile.
    uint32_t done = 0;
    for (int spin = 0; spin < (1 << 20) && !done; ++spin)
      asm volatile(
          "{ .reg .pred P; mbarrier.try_wait.parity.shared::cta.b64 P, [%1], 0; "
          "selp.u32 %0, 1, 0, P; }"
          : "=r"(done)
          : "r"(smem_u32(&bar))
          : "memory");
    if (!done) return;
  }

  const ColorMat m = p.mat;
  T* dst = static_cast<T*>(p.dst) + (long long)n * p.dst_image_stride;
  const int groups = (p.out_w + 3) >> 2;
  const int total = rows_here * groups;
  for (int gi = tid; gi < total; gi += kResizeThreads) {
    const int r = gi / groups, ox0 = (gi - r * groups) * 4;
    const int oy = oy0 + r;
    const Axis ay = axis_of(d.scale_y, (float)(d.crop_y + oy), d.src_h);
    const float wy1 = ay.w1, wy0 = __fsub_rn(1.0f, wy1);
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
    float val[4][3];  // [pixel][output slot]
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      // pixels past the row end repeat the last column; they are never stored
      const int oxk = min(ox0 + k, p.out_w - 1);
      const uint4 e = xtab[(oxk & 3) * tab_groups + (oxk >> 2)];
      const float w1 = __uint_as_float(e.z);
      const float2 wx1 = dup2(w1), wx0 = dup2(__fsub_rn(1.0f, w1));
      float2 t[2][3];  // [column x0/x1][channel], lanes = {row y0, row y1}, clamped 0..255
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int sx = c ? (int)(e.x >> 16) : (int)(e.x & 0xFFFFu);
        const int ci = c ? (int)(e.y >> 16) : (int)(e.y & 0xFFFFu);
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
          continue;
        }
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
        const Chroma2 ch = chroma2_of(m, bu, bv);
        float2 cr, cg, cb;
        pixel2_bits(m, make_float2(biased(y0p[sx]), biased(y1p[sx])), ch, cr, cg, cb);
        t[c][0] = clamp_to_float2(cr);
        t[c][1] = clamp_to_float2(cg);
        t[c][2] = clamp_to_float2(cb);
      }
#pragma unroll
      for (int s = 0; s < 3; ++s) {
        const int c = BGR ? 2 - s : s;
        // {top, bot} = fma(wx1, t?1, wx0 * t?0) for both rows at once
        const float2 tb = x2_fma(wx1, t[1][c], x2_mul(wx0, t[0][c]));
        val[k][s] = __fmaf_rn(wy1, tb.y, __fmul_rn(wy0, tb.x));
      }
    }

    // ---- finish and store four pixels -------------------------------------------------------
    const bool full4 = p.vec_store && ox0 + 4 <= p.out_w;
    if constexpr (DTYPE == B2_U8) {
      // floor(val + 0.5) as a subnormal bit pattern (val >= 0): see pack4_sat
      float q[4][3];
#pragma unroll
      for (int k = 0; k < 4; ++k)
#pragma unroll
        for (int s = 0; s < 3; ++s)
          q[k][s] = __fmul_rz(__fmaf_rn(val[k][s], kTapScale, 0.5f), __uint_as_float(1u));
      if (full4) {
        if constexpr (LAYOUT == B2_NCHW) {
#pragma unroll
          for (int s = 0; s < 3; ++s)
            *reinterpret_cast<uint32_t*>(dst + ((long long)s * p.out_h + oy) * p.out_w + ox0) =
                pack4_sat(q[0][s], q[1][s], q[2][s], q[3][s]);
        } else {
          uint32_t* o = reinterpret_cast<uint32_t*>(dst + ((long long)oy * p.out_w + ox0) * 3);
          o[0] = pack4_sat(q[0][0], q[0][1], q[0][2], q[1][0]);
          o[1] = pack4_sat(q[1][1], q[1][2], q[2][0], q[2][1]);
          o[2] = pack4_sat(q[2][2], q[3][0], q[3][1], q[3][2]);
        }
        continue;
      }
#pragma unroll
      for (int k = 0; k < 4; ++k)
#pragma unroll
        for (int s = 0; s < 3; ++s)
          val[k][s] = (float)(pack4_sat(q[k][s], q[k][s], q[k][s], q[k][s]) & 0xFFu);
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k)
#pragma unroll
        for (int s = 0; s < 3; ++s) val[k][s] = __fmaf_rn(val[k][s], p.sb.s[s], p.sb.b[s]);
      if (full4) {
        if constexpr (DTYPE == B2_F32) {
          if constexpr (LAYOUT == B2_NCHW) {
#pragma unroll
            for (int s = 0; s < 3; ++s)
              *reinterpret_cast<float4*>(dst + ((long long)s * p.out_h + oy) * p.out_w + ox0) =
                  make_float4(val[0][s], val[1][s], val[2][s], val[3][s]);
          } else {
            float4* o = reinterpret_cast<float4*>(dst + ((long long)oy * p.out_w + ox0) * 3);
            o[0] = make_float4(val[0][0], val[0][1], val[0][2], val[1][0]);
            o[1] = make_float4(val[1][1], val[1][2], val[2][0], val[2][1]);
            o[2] = make_float4(val[2][2], val[3][0], val[3][1], val[3][2]);
          }
        } else {
          auto b2w = [](float a, float b) {
            __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
            return *reinterpret_cast<uint32_t*>(&t);
          };
          if constexpr (LAYOUT == B2_NCHW) {
#pragma unroll
            for (int s = 0; s < 3; ++s)
              *reinterpret_cast<uint2*>(dst + ((long long)s * p.out_h + oy) * p.out_w + ox0) =
                  make_uint2(b2w(val[0][s], val[1][s]), b2w(val[2][s], val[3][s]));
          } else {
            uint2* o = reinterpret_cast<uint2*>(dst + ((long long)oy * p.out_w + ox0) * 3);
            o[0] = make_uint2(b2w(val[0][0], val[0][1]), b2w(val[0][2], val[1][0]));
            o[1] = make_uint2(b2w(val[1][1], val[1][2]), b2w(val[2][0], val[2][1]));
            o[2] = make_uint2(b2w(val[2][2], val[3][0]), b2w(val[3][1], val[3][2]));
          }
        }
        continue;
      }
    }
    // ragged end of a row, or a destination that is not 16-byte aligned: element stores
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (ox0 + k >= p.out_w) break;
#pragma unroll
      for (int s = 0; s < 3; ++s) {
        const long long idx = LAYOUT == B2_NCHW
                                  ? ((long long)s * p.out_h + oy) * p.out_w + ox0 + k
                                  : ((long long)oy * p.out_w + ox0 + k) * 3 + s;
        if constexpr (DTYPE == B2_U8) dst[idx] = (uint8_t)(int)val[k][s];
        else if constexpr (DTYPE == B2_F32) dst[idx] = val[k][s];
        else dst[idx] = __float2bfloat16_rn(val[k][s]);
      }
    }
  }
}

template <int FMT, int LAYOUT, int DTYPE, bool BGR>
int launch_t(const b2_resize_args& a, const ResizeParams& p, size_t smem, cudaStream_t stream) {
  auto kern = resize_kernel<FMT, LAYOUT, DTYPE, BGR>;
  if (smem > 48 * 1024)
    B2_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
            "raising the shared-memory limit of the resize kernel failed");
  const int row_blocks = (a.out_h + p.rows - 1) / p.rows;
  for (int n0 = 0; n0 < a.num_images; n0 += 65535) {
    const int nn = a.num_images - n0 < 65535 ? a.num_images - n0 : 65535;
    ResizeParams q = p;
    q.descs = p.descs + n0;
    const size_t esz = DTYPE == B2_U8 ? 1 : (DTYPE == B2_F32 ? 4 : 2);
    q.dst = static_cast<char*>(p.dst) + (size_t)n0 * p.dst_image_stride * esz;
    kern<<<dim3(row_blocks, nn), kResizeThreads, smem, stream>>>(q);
    B2_CUDA(cudaPeekAtLastError(), "launch of the resize kernel failed");
  }
  return B2_OK;
}

template <int FMT, int LAYOUT>
int launch_fl(const b2_resize_args& a, const ResizeParams& p, size_t smem, cudaStream_t s) {
  const bool bgr = a.order == B2_BGR;
  switch (a.dtype) {
    case B2_U8:
      return bgr ? launch_t<FMT, LAYOUT, B2_U8, true>(a, p, smem, s)
                 : launch_t<FMT, LAYOUT, B2_U8, false>(a, p, smem, s);
    case B2_F32:
      return bgr ? launch_t<FMT, LAYOUT, B2_F32, true>(a, p, smem, s)
                 : launch_t<FMT, LAYOUT, B2_F32, false>(a, p, smem, s);
    default:
      return bgr ? launch_t<FMT, LAYOUT, B2_BF16, true>(a, p, smem, s)
                 : launch_t<FMT, LAYOUT, B2_BF16, false>(a, p, smem, s);
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
  p.mat = color_matrix(a.matrix_coeff, a.full_range);
  p.dst = a.dst;
  p.dst_image_stride = a.dst_image_stride ? a.dst_image_stride : 3LL * a.out_w * a.out_h;
  for (int i = 0; i < 3; ++i) {
    p.sb.s[i] = a.scale[i] * 16777216.0f;  // the kernel blends taps scaled by 2^-24 (exact)
    p.sb.b[i] = a.bias[i];
  }
  const int esz = a.dtype == B2_U8 ? 1 : (a.dtype == B2_F32 ? 4 : 2);
  p.vec_store = a.out_w % 4 == 0 && (uintptr_t)a.dst % 16 == 0 &&
                (p.dst_image_stride * esz) % 16 == 0;
  // A staged span holds at most max_src_w + 1 bytes (interleaved chroma rows of an odd width)
  // plus up to 15 bytes of alignment head, rounded up to whole 16-byte segments.
  const int row_bytes = a.src_format == B2_SRC_RGB_INTERLEAVED ? 3 * a.max_src_w : a.max_src_w;
  p.span_cap = ((row_bytes + 2 + 15 + 15) / 16) * 16;
  const int planes = a.src_format == B2_SRC_NV12 ? 4 : (a.src_format == B2_SRC_RGB_INTERLEAVED ? 2 : 6);
  const size_t table = (size_t)((a.out_w + 3) / 4) * 64;
  // Four output rows per CTA amortise the per-CTA work best; wide sources (4K rows) take two,
  // which halves the staging buffer and lets more CTAs share an SM.
  p.rows = (size_t)kRows * planes * p.span_cap + table > 40 * 1024 ? 2 : kRows;
  const size_t smem = (size_t)p.rows * planes * p.span_cap + table;
  if (p.span_cap >= 65536 || smem > 200 * 1024)
    return fail(B2_ERR_LIMIT, "max_src_w %d needs %zu bytes of staging; the limit is %d bytes",
                a.max_src_w, smem, 200 * 1024);
  switch (a.src_format) {
    case B2_SRC_NV12:
      return a.layout == B2_NCHW ? launch_fl<B2_SRC_NV12, B2_NCHW>(a, p, smem, stream)
                                 : launch_fl<B2_SRC_NV12, B2_NHWC>(a, p, smem, stream);
    case B2_SRC_I420:
      return a.layout == B2_NCHW ? launch_fl<B2_SRC_I420, B2_NCHW>(a, p, smem, stream)
                                 : launch_fl<B2_SRC_I420, B2_NHWC>(a, p, smem, stream);
    case B2_SRC_RGB_PLANAR:
      return a.layout == B2_NCHW ? launch_fl<B2_SRC_RGB_PLANAR, B2_NCHW>(a, p, smem, stream)
                                 : launch_fl<B2_SRC_RGB_PLANAR, B2_NHWC>(a, p, smem, stream);
    default:
      return a.layout == B2_NCHW ? launch_fl<B2_SRC_RGB_INTERLEAVED, B2_NCHW>(a, p, smem, stream)
                                 : launch_fl<B2_SRC_RGB_INTERLEAVED, B2_NHWC>(a, p, smem, stream);
  }
}

}  // namespace b2

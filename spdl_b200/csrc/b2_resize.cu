// Fused colour conversion -> bilinear resize -> crop -> scale/bias over a ragged batch.
//
// Semantics (the CPU restatement in the test oracle is the definition):
//   gx = crop_x + ox;  sx = max(fma(scale_x, gx + 0.5, -0.5), 0);  x0 = int(sx);
//   x1 = min(x0 + 1, src_w - 1);  wx1 = sx - x0;  wx0 = 1 - wx1      (same for y)
//   every tap is converted to 8-bit RGB exactly as the dense kernel does, then
//   top = fma(wx1, t01, wx0*t00); bot = fma(wx1, t11, wx0*t10); val = fma(wy1, bot, wy0*top)
//   u8 output: floor(val + 0.5) clamped to 0..255; float outputs: fma(val, scale, bias).
//
// One CTA produces kRows output rows of one image.  For each output row it needs two luma rows
// and one or two chroma rows; the CTA copies exactly the spans of those rows that its outputs
// touch into shared memory with 16-byte coalesced loads, then every thread interpolates one
// output pixel at a time from shared memory.  Global traffic is therefore whole 16-byte
// segments of the touched rows and nothing else.
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
  int span_cap;  // bytes reserved per staged row
};

constexpr int kRows = 4;        // output rows per CTA
constexpr int kResizeThreads = 256;

struct Axis {
  int i0, i1;
  float w1;
};
__device__ __forceinline__ Axis axis_of(float scale, int g, int n_in) {
  float s = fmaxf(__fmaf_rn(scale, (float)g + 0.5f, -0.5f), 0.0f);
  int a = (int)s;
  a = min(a, n_in - 1);
  Axis r;
  r.i0 = a;
  r.i1 = min(a + 1, n_in - 1);
  r.w1 = __fsub_rn(s, (float)a);
  return r;
}

// Copy bytes [lo, hi) of a source row into shared memory at s[0 .. hi-lo).  The global range is
// widened to 16-byte boundaries when the row pointer allows it; `shift` tells the caller where
// byte `lo` landed.
__device__ __forceinline__ int stage_span(const uint8_t* row, int lo, int hi, unsigned char* s,
                                          int tid, int nthreads) {
  const uintptr_t a = (uintptr_t)(row + lo);
  const int head = (int)(a & 15);
  const uint8_t* g = row + lo - head;  // 16-byte aligned
  const int total = hi - lo + head;
  const int nvec = (total + 15) >> 4;
  // Rows start 16-byte aligned relative to the allocation in every layout this library
  // produces; reading up to 15 bytes past `hi` could leave the allocation, so the last
  // partial vector is fetched bytewise.
  const int full = total >> 4;
  for (int i = tid; i < full; i += nthreads)
    reinterpret_cast<uint4*>(s)[i] = __ldg(reinterpret_cast<const uint4*>(g) + i);
  if (full < nvec) {
    const int rem = total - (full << 4);
    for (int i = tid; i < rem; i += nthreads) s[(full << 4) + i] = __ldg(g + (full << 4) + i);
  }
  return head;
}

template <int FMT, int LAYOUT, int DTYPE, bool BGR>
__global__ void __launch_bounds__(kResizeThreads) resize_kernel(const ResizeParams p) {
  using T = typename OutT<DTYPE>::type;
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ b2_image_desc sd;
  __shared__ int s_head[kRows][6];

  const int n = blockIdx.y;
  const int oy0 = blockIdx.x * kRows;
  const int tid = threadIdx.x;
  if (tid < 16) reinterpret_cast<uint32_t*>(&sd)[tid] =
      __ldg(reinterpret_cast<const uint32_t*>(p.descs + n) + tid);
  __syncthreads();
  const b2_image_desc d = sd;

  // Horizontal extent of source pixels touched by this image's output columns.
  const Axis ax_first = axis_of(d.scale_x, d.crop_x, d.src_w);
  const Axis ax_last = axis_of(d.scale_x, d.crop_x + p.out_w - 1, d.src_w);
  const int xlo = ax_first.i0, xhi = ax_last.i1 + 1;  // [xlo, xhi)
  const int cxlo = FMT == B2_SRC_NV12 ? (xlo & ~1) : (xlo >> 1);
  const int cxhi = FMT == B2_SRC_NV12 ? (((xhi - 1) & ~1) + 2) : (((xhi - 1) >> 1) + 1);

  // A descriptor wider than the caller's max_src_w would overrun the staging rows: such an image
  // is skipped (its output is left untouched) rather than allowed to write out of bounds.
  if (xhi - xlo + 15 > p.span_cap || cxhi - cxlo + 15 > p.span_cap || d.src_w < 1 || d.src_h < 1)
    return;

  // Shared layout per output row: [y0 | y1 | c0a | c1a | (I420: c0b | c1b)], span_cap bytes each.
  constexpr int kPlanes = FMT == B2_SRC_NV12 ? 4 : 6;
  const int rows_here = min(kRows, p.out_h - oy0);
  for (int r = 0; r < rows_here; ++r) {
    const Axis ay = axis_of(d.scale_y, d.crop_y + oy0 + r, d.src_h);
    unsigned char* sr = smem + (size_t)r * kPlanes * p.span_cap;
    const uint8_t* yb = p.base + d.y_off;
    int h;
    h = stage_span(yb + (size_t)ay.i0 * d.y_pitch, xlo, xhi, sr, tid, kResizeThreads);
    if (tid == 0) s_head[r][0] = h;
    h = stage_span(yb + (size_t)ay.i1 * d.y_pitch, xlo, xhi, sr + p.span_cap, tid, kResizeThreads);
    if (tid == 0) s_head[r][1] = h;
    const uint8_t* ub = p.base + d.u_off;
    h = stage_span(ub + (size_t)(ay.i0 >> 1) * d.uv_pitch, cxlo, cxhi, sr + 2 * p.span_cap, tid,
                   kResizeThreads);
    if (tid == 0) s_head[r][2] = h;
    h = stage_span(ub + (size_t)(ay.i1 >> 1) * d.uv_pitch, cxlo, cxhi, sr + 3 * p.span_cap, tid,
                   kResizeThreads);
    if (tid == 0) s_head[r][3] = h;
    if constexpr (FMT == B2_SRC_I420) {
      const uint8_t* vb = p.base + d.v_off;
      h = stage_span(vb + (size_t)(ay.i0 >> 1) * d.uv_pitch, cxlo, cxhi, sr + 4 * p.span_cap, tid,
                     kResizeThreads);
      if (tid == 0) s_head[r][4] = h;
      h = stage_span(vb + (size_t)(ay.i1 >> 1) * d.uv_pitch, cxlo, cxhi, sr + 5 * p.span_cap, tid,
                     kResizeThreads);
      if (tid == 0) s_head[r][5] = h;
    }
  }
  __syncthreads();

  const ColorMat m = p.mat;
  T* dst = static_cast<T*>(p.dst) + (long long)n * p.dst_image_stride;
  const int total = rows_here * p.out_w;
  for (int i = tid; i < total; i += kResizeThreads) {
    const int r = i / p.out_w, ox = i - r * p.out_w;
    const int oy = oy0 + r;
    const Axis ay = axis_of(d.scale_y, d.crop_y + oy, d.src_h);
    const Axis ax = axis_of(d.scale_x, d.crop_x + ox, d.src_w);
    const unsigned char* sr = smem + (size_t)r * kPlanes * p.span_cap;
    const float wx1 = ax.w1, wx0 = __fsub_rn(1.0f, wx1);
    const float wy1 = ay.w1, wy0 = __fsub_rn(1.0f, wy1);
    int tap[2][2][3];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const unsigned char* ys = sr + j * p.span_cap + s_head[r][j];
      const unsigned char* us = sr + (2 + j) * p.span_cap + s_head[r][2 + j];
      const unsigned char* vs =
          FMT == B2_SRC_I420 ? sr + (4 + j) * p.span_cap + s_head[r][4 + j] : nullptr;
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int sx = k ? ax.i1 : ax.i0;
        const int Y = ys[sx - xlo];
        int cu, cv;
        if constexpr (FMT == B2_SRC_NV12) {
          cu = us[(sx & ~1) - cxlo];
          cv = us[(sx & ~1) - cxlo + 1];
        } else {
          cu = us[(sx >> 1) - cxlo];
          cv = vs[(sx >> 1) - cxlo];
        }
        pixel_u8(m, Y, cu, cv, tap[j][k][0], tap[j][k][1], tap[j][k][2]);
      }
    }
#pragma unroll
    for (int s = 0; s < 3; ++s) {
      const int c = BGR ? 2 - s : s;
      const float top = __fmaf_rn(wx1, (float)tap[0][1][c], __fmul_rn(wx0, (float)tap[0][0][c]));
      const float bot = __fmaf_rn(wx1, (float)tap[1][1][c], __fmul_rn(wx0, (float)tap[1][0][c]));
      float val = __fmaf_rn(wy1, bot, __fmul_rn(wy0, top));
      if constexpr (DTYPE == B2_U8) val = fminf(fmaxf(floorf(__fadd_rn(val, 0.5f)), 0.0f), 255.0f);
      const long long idx = LAYOUT == B2_NCHW ? ((long long)s * p.out_h + oy) * p.out_w + ox
                                              : ((long long)oy * p.out_w + ox) * 3 + s;
      dst[idx] = finish<T>(val, p.sb.s[s], p.sb.b[s]);
    }
  }
}

template <int FMT, int LAYOUT, int DTYPE, bool BGR>
int launch_t(const b2_resize_args& a, const ResizeParams& p, size_t smem, cudaStream_t stream) {
  auto kern = resize_kernel<FMT, LAYOUT, DTYPE, BGR>;
  if (smem > 48 * 1024)
    B2_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
            "raising the shared-memory limit of the resize kernel failed");
  const int row_blocks = (a.out_h + kRows - 1) / kRows;
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
    p.sb.s[i] = a.scale[i];
    p.sb.b[i] = a.bias[i];
  }
  // A staged row holds at most max_src_w bytes (interleaved chroma rows are as wide as luma rows)
  // plus the 15 bytes of alignment head, rounded to 16.
  p.span_cap = ((a.max_src_w + 2 + 15 + 15) / 16) * 16;
  const int planes = a.src_format == B2_SRC_NV12 ? 4 : 6;
  const size_t smem = (size_t)kRows * planes * p.span_cap;
  if (smem > 200 * 1024)
    return fail(B2_ERR_LIMIT, "max_src_w %d needs %zu bytes of staging; the limit is %d bytes",
                a.max_src_w, smem, 200 * 1024);
  if (a.src_format == B2_SRC_NV12)
    return a.layout == B2_NCHW ? launch_fl<B2_SRC_NV12, B2_NCHW>(a, p, smem, stream)
                               : launch_fl<B2_SRC_NV12, B2_NHWC>(a, p, smem, stream);
  return a.layout == B2_NCHW ? launch_fl<B2_SRC_I420, B2_NCHW>(a, p, smem, stream)
                             : launch_fl<B2_SRC_I420, B2_NHWC>(a, p, smem, stream);
}

}  // namespace b2

// Dense colour conversion: every pixel of every frame, no resampling.
//
// Three kernel families.
//   dense_vec_kernel   the fast path.  One thread owns a 2-row x PX-pixel block (PX = 16 bytes
//                      of output per channel: 16 px for u8, 8 for bf16, 4 for fp32), so the two
//                      rows share one chroma load, every global load is one 4/8/16-byte vector
//                      and every global store is a 16-byte vector.  Planar output is stored
//                      straight from registers (a warp writes 512 contiguous bytes per
//                      instruction).  Interleaved output (48 bytes per thread per row) is staged
//                      in shared memory by the warp and leaves as one bulk asynchronous copy
//                      (cp.async.bulk shared->global) per row segment.
//   dense_rows_kernel  rows on arbitrary byte boundaries (a pointer, pitch or width that breaks
//                      the vector path's alignment): one CTA per row pair realigns the rows
//                      through shared memory and runs the same packed arithmetic from there.
//   dense_quad_kernel  the last resort: one thread per 2x2 quad with byte accesses (widths under
//                      16, rows too wide for shared memory).
//
// The kernels are HBM-bound: 1.5 bytes read and 3*sizeof(T) written per pixel.
#include "b2_common.cuh"

namespace b2 {
namespace {

struct DenseParams {
  const uint8_t* y;
  const uint8_t* u;
  const uint8_t* v;
  const void* const* y_table;
  const void* const* u_table;
  const void* const* v_table;
  long long y_frame_stride, uv_frame_stride;
  int y_pitch, uv_pitch;  // bytes between rows (the launcher rejects pitches beyond 2^31)
  int width, height;      // height here is the even part of the frame height
  ColorMat mat;
  void* dst;
  long long dst_plane_stride, dst_frame_stride;  // elements
  int dst_row_pitch;                              // elements
  ScaleBias sb;
};

// Load NB bytes into ceil(NB/4) words.  Streaming (read-once) cache hint.
template <int NB>
__device__ __forceinline__ void load_bytes(const uint8_t* p, uint32_t* w) {
  if constexpr (NB == 16) {
    uint4 t = __ldcs(reinterpret_cast<const uint4*>(p));
    w[0] = t.x; w[1] = t.y; w[2] = t.z; w[3] = t.w;
  } else if constexpr (NB == 8) {
    uint2 t = __ldcs(reinterpret_cast<const uint2*>(p));
    w[0] = t.x; w[1] = t.y;
  } else if constexpr (NB == 4) {
    w[0] = __ldcs(reinterpret_cast<const uint32_t*>(p));
  } else {
    w[0] = __ldcs(reinterpret_cast<const uint16_t*>(p));
  }
}
template <int NB>
__device__ __forceinline__ void load_bytes_any(const uint8_t* p, uint32_t* w, bool aligned) {
  if (aligned) {
    load_bytes<NB>(p, w);
  } else {
#pragma unroll
    for (int i = 0; i < (NB + 3) / 4; ++i) w[i] = 0;
#pragma unroll
    for (int i = 0; i < NB; ++i) w[i >> 2] |= (uint32_t)__ldcs(p + i) << (8 * (i & 3));
  }
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

constexpr int kDenseThreads = 128;
// 12 resident CTAs (48 warps) per SM: measured best (CTAs of 64 threads are no faster, of 32
// or 256 slower); caps the kernel at 40 registers per thread.
constexpr int kDenseMinBlocks = 12;

template <int FMT, int LAYOUT, int DTYPE, bool BGR, bool TABLE>
__global__ void __launch_bounds__(kDenseThreads, kDenseMinBlocks) dense_vec_kernel(const DenseParams p) {
  using T = typename OutT<DTYPE>::type;
  constexpr int PX = 16 / (int)sizeof(T);  // pixels per thread per row
  constexpr int NW = PX / 4;               // luma words per row
  constexpr int UVB = FMT == B2_SRC_NV12 ? PX : PX / 2;  // chroma bytes per plane row segment
  constexpr int UVW = (UVB + 3) / 4;

  const int cx = blockIdx.x * blockDim.x + threadIdx.x;
  const int rp = blockIdx.y * blockDim.y + threadIdx.y;
  const int n = blockIdx.z;
  const int x0 = cx * PX;
  const bool active = x0 < p.width && 2 * rp < p.height;

  uint32_t out[2][12];  // 48 bytes per row, already in destination order

  // Interleaved output is staged in shared memory per warp (2 rows x 32 lanes x 48 bytes).
  extern __shared__ __align__(128) unsigned char stage_raw[];
  const int lane = threadIdx.x & 31;
  unsigned char* ws =
      stage_raw + ((threadIdx.y * blockDim.x + threadIdx.x) >> 5) * (2 * 32 * 48) + lane * 48;
  // The 16-byte pieces of a row are stored as soon as they are complete, which keeps fewer
  // finished words alive in registers.
  constexpr bool kEarlyStage = LAYOUT == B2_NHWC;
  auto stage_piece = [&](int r, int i) {
    *reinterpret_cast<uint4*>(ws + r * 1536 + i * 16) =
        make_uint4(out[r][4 * i], out[r][4 * i + 1], out[r][4 * i + 2], out[r][4 * i + 3]);
  };

  if (active) {
    const uint8_t *yb, *ub, *vb = nullptr;
    bool aligned = true;
    if constexpr (TABLE) {
      yb = static_cast<const uint8_t*>(p.y_table[n]);
      ub = static_cast<const uint8_t*>(p.u_table[n]);
      if constexpr (FMT == B2_SRC_I420) vb = static_cast<const uint8_t*>(p.v_table[n]);
      aligned = (((uintptr_t)yb | (uintptr_t)ub | (uintptr_t)vb) & 15) == 0;
    } else {
      yb = p.y + (long long)n * p.y_frame_stride;
      ub = p.u + (long long)n * p.uv_frame_stride;
      if constexpr (FMT == B2_SRC_I420) vb = p.v + (long long)n * p.uv_frame_stride;
    }
    uint32_t yw[2][NW], uw[UVW], vw[UVW];
    const uint8_t* y0p = yb + (size_t)(2 * rp) * (unsigned)p.y_pitch + x0;
    const uint8_t* up = ub + (size_t)rp * (unsigned)p.uv_pitch + (FMT == B2_SRC_NV12 ? x0 : x0 / 2);
    if constexpr (TABLE) {
      load_bytes_any<PX>(y0p, yw[0], aligned);
      load_bytes_any<PX>(y0p + p.y_pitch, yw[1], aligned);
      load_bytes_any<UVB>(up, uw, aligned);
      if constexpr (FMT == B2_SRC_I420)
        load_bytes_any<UVB>(vb + (size_t)rp * (unsigned)p.uv_pitch + x0 / 2, vw, aligned);
    } else {
      load_bytes<PX>(y0p, yw[0]);
      load_bytes<PX>(y0p + p.y_pitch, yw[1]);
      load_bytes<UVB>(up, uw);
      if constexpr (FMT == B2_SRC_I420)
        load_bytes<UVB>(vb + (size_t)rp * (unsigned)p.uv_pitch + x0 / 2, vw);
    }
    (void)vw;

    const ColorMat m = p.mat;
#pragma unroll
    for (int j = 0; j < NW; ++j) {
      // chroma of the two 2x2 quads under luma word j: lane x = first quad, lane y = second
      Chroma2 c;
      if constexpr (FMT == B2_SRC_NV12) {
        c = chroma2_of(m, make_float2(biased_byte(uw[j], 0), biased_byte(uw[j], 2)),
                       make_float2(biased_byte(uw[j], 1), biased_byte(uw[j], 3)));
      } else {
        const int w = j >> 1, b = (j & 1) * 2;
        c = chroma2_of(m, make_float2(biased_byte(uw[w], b), biased_byte(uw[w], b + 1)),
                       make_float2(biased_byte(vw[w], b), biased_byte(vw[w], b + 1)));
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        // ch[slot][pixel]: channel value + 1.5*2^23, truncated (floor in the low mantissa bits)
        float ch[3][4];
#pragma unroll
        for (int k = 0; k < 2; ++k) {  // pixels k and k+2 share one packed instruction stream
          float2 cr, cg, cb;
          pixel2_bits(m, make_float2(biased_byte(yw[r][j], k), biased_byte(yw[r][j], k + 2)), c, cr,
                      cg, cb);
          ch[BGR ? 2 : 0][k] = cr.x; ch[BGR ? 2 : 0][k + 2] = cr.y;
          ch[1][k] = cg.x;           ch[1][k + 2] = cg.y;
          ch[BGR ? 0 : 2][k] = cb.x; ch[BGR ? 0 : 2][k + 2] = cb.y;
        }
        if constexpr (DTYPE == B2_U8) {
          if constexpr (LAYOUT == B2_NCHW) {
#pragma unroll
            for (int s = 0; s < 3; ++s)
              out[r][4 * s + j] = bytes4(clamp2_bits(ch[s][0], ch[s][1]), clamp2_bits(ch[s][2], ch[s][3]));
          } else {
            out[r][3 * j + 0] = bytes4(clamp2_bits(ch[0][0], ch[1][0]), clamp2_bits(ch[2][0], ch[0][1]));
            out[r][3 * j + 1] = bytes4(clamp2_bits(ch[1][1], ch[2][1]), clamp2_bits(ch[0][2], ch[1][2]));
            out[r][3 * j + 2] = bytes4(clamp2_bits(ch[2][2], ch[0][3]), clamp2_bits(ch[1][3], ch[2][3]));
            if (j >= 1) stage_piece(r, j - 1);  // piece i needs the luma words up to i + 1
          }
        } else {
          float f[3][4];
#pragma unroll
          for (int s = 0; s < 3; ++s) {
            const uint32_t q01 = clamp2_bits(ch[s][0], ch[s][1]), q23 = clamp2_bits(ch[s][2], ch[s][3]);
            // exact 0..255 floats of two pixels, then value * scale + bias, two lanes at a time
            const float2 sc = dup2(p.sb.s[s]), bi = dup2(p.sb.b[s]), off = dup2(-kTwo23);
            const float2 a = x2_fma(x2_add(make_float2(biased_byte(q01, 0), biased_byte(q01, 2)), off),
                                    sc, bi);
            const float2 b = x2_fma(x2_add(make_float2(biased_byte(q23, 0), biased_byte(q23, 2)), off),
                                    sc, bi);
            f[s][0] = a.x; f[s][1] = a.y; f[s][2] = b.x; f[s][3] = b.y;
          }
          if constexpr (DTYPE == B2_F32) {  // NW == 1
#pragma unroll
            for (int s = 0; s < 3; ++s)
#pragma unroll
              for (int k = 0; k < 4; ++k)
                out[r][LAYOUT == B2_NCHW ? 4 * s + k : 3 * k + s] = __float_as_uint(f[s][k]);
            if constexpr (kEarlyStage) {
#pragma unroll
              for (int i = 0; i < 3; ++i) stage_piece(r, i);
            }
          } else {  // bf16, NW == 2: 8 pixels, two per word
            if constexpr (LAYOUT == B2_NCHW) {
#pragma unroll
              for (int s = 0; s < 3; ++s)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                  __nv_bfloat162 t = __floats2bfloat162_rn(f[s][2 * h], f[s][2 * h + 1]);
                  out[r][4 * s + 2 * j + h] = *reinterpret_cast<uint32_t*>(&t);
                }
            } else {
              // 12 values of this luma word in memory order: p0(s0 s1 s2) p1(...) ...
#pragma unroll
              for (int w = 0; w < 6; ++w) {
                const int e0 = 2 * w, e1 = 2 * w + 1;
                __nv_bfloat162 t = __floats2bfloat162_rn(f[e0 % 3][e0 / 3], f[e1 % 3][e1 / 3]);
                out[r][6 * j + w] = *reinterpret_cast<uint32_t*>(&t);
              }
              if (j == 0) {
                stage_piece(r, 0);
              } else {
                stage_piece(r, 1);
                stage_piece(r, 2);
              }
            }
          }
        }
      }
    }
  }

  T* dst = static_cast<T*>(p.dst) + (long long)n * p.dst_frame_stride;
  if constexpr (LAYOUT == B2_NCHW) {
    if (active) {
#pragma unroll
      for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int s = 0; s < 3; ++s) {
          T* q = dst + s * p.dst_plane_stride + (long long)(2 * rp + r) * p.dst_row_pitch + x0;
          __stcs(reinterpret_cast<uint4*>(q),
                 make_uint4(out[r][4 * s], out[r][4 * s + 1], out[r][4 * s + 2], out[r][4 * s + 3]));
        }
    }
  } else {
    // Interleaved: the warp's 32 x 48 bytes per row are contiguous in the destination.  Stage
    // them in shared memory and hand each row segment to the bulk-copy engine.
    // make the generic-proxy writes visible to the async proxy, then let lane 0 issue the copies
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (lane == 0 && 2 * rp < p.height) {
      const int wx0 = (cx - lane) * PX;  // first pixel of the warp's segment (lane 0's cx)
      int px_in_seg = p.width - wx0;
      if (px_in_seg > 32 * PX) px_in_seg = 32 * PX;
      if (px_in_seg > 0) {
        const uint32_t bytes = (uint32_t)px_in_seg * 3u * (uint32_t)sizeof(T);
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          T* q = dst + (long long)(2 * rp + r) * p.dst_row_pitch + (long long)wx0 * 3;
          asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(q),
                       "r"(smem_addr(ws + r * 1536)), "r"(bytes)  // lane 0: ws is the segment start
                       : "memory");
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        // the staging buffer must outlive the engine's reads of it
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      }
    }
  }
}

// One thread's block of 2 rows x PX pixels: luma words yw, chroma words uw (and vw for I420) in,
// 48 bytes per row out, already in destination order (interleaved: linear; planar: 16 bytes per
// output slot).  The same arithmetic as the vector kernel's inner loop.
template <int FMT, int LAYOUT, int DTYPE, bool BGR, int NW, int UVW>
__device__ __forceinline__ void convert_chunk(const ColorMat& m, const ScaleBias& sb,
                                              const uint32_t (&yw)[2][NW],
                                              const uint32_t (&uw)[UVW],
                                              const uint32_t (&vw)[UVW], uint32_t (&out)[2][12]) {
#pragma unroll
  for (int j = 0; j < NW; ++j) {
    Chroma2 c;
    if constexpr (FMT == B2_SRC_NV12) {
      c = chroma2_of(m, make_float2(biased_byte(uw[j], 0), biased_byte(uw[j], 2)),
                     make_float2(biased_byte(uw[j], 1), biased_byte(uw[j], 3)));
    } else {
      const int w = j >> 1, b = (j & 1) * 2;
      c = chroma2_of(m, make_float2(biased_byte(uw[w], b), biased_byte(uw[w], b + 1)),
                     make_float2(biased_byte(vw[w], b), biased_byte(vw[w], b + 1)));
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float ch[3][4];
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        float2 cr, cg, cb;
        pixel2_bits(m, make_float2(biased_byte(yw[r][j], k), biased_byte(yw[r][j], k + 2)), c, cr,
                    cg, cb);
        ch[BGR ? 2 : 0][k] = cr.x; ch[BGR ? 2 : 0][k + 2] = cr.y;
        ch[1][k] = cg.x;           ch[1][k + 2] = cg.y;
        ch[BGR ? 0 : 2][k] = cb.x; ch[BGR ? 0 : 2][k + 2] = cb.y;
      }
      if constexpr (DTYPE == B2_U8) {
        if constexpr (LAYOUT == B2_NCHW) {
#pragma unroll
          for (int s = 0; s < 3; ++s)
            out[r][4 * s + j] =
                bytes4(clamp2_bits(ch[s][0], ch[s][1]), clamp2_bits(ch[s][2], ch[s][3]));
        } else {
          out[r][3 * j + 0] = bytes4(clamp2_bits(ch[0][0], ch[1][0]), clamp2_bits(ch[2][0], ch[0][1]));
          out[r][3 * j + 1] = bytes4(clamp2_bits(ch[1][1], ch[2][1]), clamp2_bits(ch[0][2], ch[1][2]));
          out[r][3 * j + 2] = bytes4(clamp2_bits(ch[2][2], ch[0][3]), clamp2_bits(ch[1][3], ch[2][3]));
        }
      } else {
        float f[3][4];
#pragma unroll
        for (int s = 0; s < 3; ++s) {
          const uint32_t q01 = clamp2_bits(ch[s][0], ch[s][1]), q23 = clamp2_bits(ch[s][2], ch[s][3]);
          const float2 sc = dup2(sb.s[s]), bi = dup2(sb.b[s]), off = dup2(-kTwo23);
          const float2 a = x2_fma(
              x2_add(make_float2(biased_byte(q01, 0), biased_byte(q01, 2)), off), sc, bi);
          const float2 b = x2_fma(
              x2_add(make_float2(biased_byte(q23, 0), biased_byte(q23, 2)), off), sc, bi);
          f[s][0] = a.x; f[s][1] = a.y; f[s][2] = b.x; f[s][3] = b.y;
        }
        if constexpr (DTYPE == B2_F32) {
#pragma unroll
          for (int s = 0; s < 3; ++s)
#pragma unroll
            for (int k = 0; k < 4; ++k)
              out[r][LAYOUT == B2_NCHW ? 4 * s + k : 3 * k + s] = __float_as_uint(f[s][k]);
        } else if constexpr (LAYOUT == B2_NCHW) {
#pragma unroll
          for (int s = 0; s < 3; ++s)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              __nv_bfloat162 t = __floats2bfloat162_rn(f[s][2 * h], f[s][2 * h + 1]);
              out[r][4 * s + 2 * j + h] = *reinterpret_cast<uint32_t*>(&t);
            }
        } else {
#pragma unroll
          for (int w = 0; w < 6; ++w) {
            const int e0 = 2 * w, e1 = 2 * w + 1;
            __nv_bfloat162 t = __floats2bfloat162_rn(f[e0 % 3][e0 / 3], f[e1 % 3][e1 / 3]);
            out[r][6 * j + w] = *reinterpret_cast<uint32_t*>(&t);
          }
        }
      }
    }
  }
}

// ---- rows path: any alignment, vector arithmetic ------------------------------------------------
// Packed batches whose width is not a multiple of 16 (854x480 video, odd crops) have rows that
// start on arbitrary byte boundaries, which rules out the vector kernel's direct 16-byte
// accesses.  Here one CTA owns a row pair of one frame: it copies the source rows into shared
// memory with aligned 16-byte global loads, shifting bytes into place with funnel shifts, runs
// the same packed arithmetic out of shared memory, assembles the output rows in shared memory
// and writes them with aligned 16-byte global stores (plus a few byte stores at the ragged ends).

// smem[0..n) = g[0..n) for any alignment of g.  Reads whole aligned 16-byte segments (each holds
// at least one valid byte, so it lies inside the allocation); writes whole 16-byte vectors, i.e.
// up to 15 bytes of padding past n.
__device__ __forceinline__ void rows_load(unsigned char* s, const uint8_t* g, int n, int tid,
                                          int nthreads) {
  const int a = (int)((uintptr_t)g & 15);
  const uint4* gv = reinterpret_cast<const uint4*>(g - a);
  const int nsrc = (a + n + 15) >> 4, ndst = (n + 15) >> 4;
  const int ws = a >> 2, bs = (a & 3) * 8;
  for (int k = tid; k < ndst; k += nthreads) {
    const uint4 lo = __ldg(gv + k);
    const uint4 hi = k + 1 < nsrc ? __ldg(gv + k + 1) : make_uint4(0u, 0u, 0u, 0u);
    uint32_t w0, w1, w2, w3, w4;  // five consecutive source words starting at word `ws`
    switch (ws) {
      case 0: w0 = lo.x; w1 = lo.y; w2 = lo.z; w3 = lo.w; w4 = hi.x; break;
      case 1: w0 = lo.y; w1 = lo.z; w2 = lo.w; w3 = hi.x; w4 = hi.y; break;
      case 2: w0 = lo.z; w1 = lo.w; w2 = hi.x; w3 = hi.y; w4 = hi.z; break;
      default: w0 = lo.w; w1 = hi.x; w2 = hi.y; w3 = hi.z; w4 = hi.w; break;
    }
    reinterpret_cast<uint4*>(s)[k] =
        make_uint4(__funnelshift_r(w0, w1, bs), __funnelshift_r(w1, w2, bs),
                   __funnelshift_r(w2, w3, bs), __funnelshift_r(w3, w4, bs));
  }
}

// g[0..n) = smem[0..n) for any alignment of g; `s` is 16-byte aligned and readable up to
// n + 16 bytes.  Aligned 16-byte stores for the body, byte stores for the ragged head and tail.
__device__ __forceinline__ void rows_store(uint8_t* g, const unsigned char* s, int n, int tid,
                                           int nthreads) {
  int head = (int)((16 - ((uintptr_t)g & 15)) & 15);
  if (head > n) head = n;
  const int nvec = (n - head) >> 4;
  const int tail0 = head + (nvec << 4);
  for (int i = tid; i < head; i += nthreads) g[i] = s[i];
  for (int i = tail0 + tid; i < n; i += nthreads) g[i] = s[i];
  // two aligned 16-byte shared loads per vector (conflict-free), then the same word select and
  // byte shift as on the load side
  const uint4* sv = reinterpret_cast<const uint4*>(s);
  const int ws = head >> 2, bs = (head & 3) * 8;
  uint4* gv = reinterpret_cast<uint4*>(g + head);
  for (int k = tid; k < nvec; k += nthreads) {
    const uint4 lo = sv[k], hi = sv[k + 1];
    uint32_t w0, w1, w2, w3, w4;
    switch (ws) {
      case 0: w0 = lo.x; w1 = lo.y; w2 = lo.z; w3 = lo.w; w4 = hi.x; break;
      case 1: w0 = lo.y; w1 = lo.z; w2 = lo.w; w3 = hi.x; w4 = hi.y; break;
      case 2: w0 = lo.z; w1 = lo.w; w2 = hi.x; w3 = hi.y; w4 = hi.z; break;
      default: w0 = lo.w; w1 = hi.x; w2 = hi.y; w3 = hi.z; w4 = hi.w; break;
    }
    __stcs(gv + k, make_uint4(__funnelshift_r(w0, w1, bs), __funnelshift_r(w1, w2, bs),
                              __funnelshift_r(w2, w3, bs), __funnelshift_r(w3, w4, bs)));
  }
}

// One aligned shared load of NW 32-bit words.
template <int NW>
__device__ __forceinline__ void lds_words(const unsigned char* s, int index, uint32_t (&w)[NW]) {
  if constexpr (NW == 4) {
    const uint4 q = reinterpret_cast<const uint4*>(s)[index];
    w[0] = q.x; w[1] = q.y; w[2] = q.z; w[3] = q.w;
  } else if constexpr (NW == 2) {
    const uint2 q = reinterpret_cast<const uint2*>(s)[index];
    w[0] = q.x; w[1] = q.y;
  } else {
    w[0] = reinterpret_cast<const uint32_t*>(s)[index];
  }
}

constexpr int kRowsThreads = 128;

// Shared-memory plan of the rows kernel for a frame width, per row pair.
struct RowsPlan {
  int in_row;    // bytes reserved per staged source row
  int out_row;   // bytes reserved per assembled output row (NHWC) or plane row (NCHW)
  int total;
};
template <int LAYOUT, int DTYPE>
__host__ __device__ inline RowsPlan rows_plan(int width) {
  constexpr int esz = DTYPE == B2_U8 ? 1 : (DTYPE == B2_F32 ? 4 : 2);
  constexpr int px = 16 / esz;
  const int chunks = (width + px - 1) / px;
  RowsPlan r;
  r.in_row = ((width + 15) & ~15) + 32;
  r.out_row = LAYOUT == B2_NHWC ? chunks * 48 + 32 : chunks * 16 + 32;
  r.total = 4 * r.in_row + 2 * (LAYOUT == B2_NHWC ? 1 : 3) * r.out_row;
  return r;
}

template <int FMT, int LAYOUT, int DTYPE, bool BGR, bool TABLE>
__global__ void __launch_bounds__(kRowsThreads) dense_rows_kernel(const DenseParams p) {
  using T = typename OutT<DTYPE>::type;
  constexpr int PX = 16 / (int)sizeof(T);
  constexpr int NW = PX / 4;
  constexpr int UVB = FMT == B2_SRC_NV12 ? PX : PX / 2;
  constexpr int UVW = (UVB + 3) / 4;
  extern __shared__ __align__(128) unsigned char rows_smem[];
  const RowsPlan plan = rows_plan<LAYOUT, DTYPE>(p.width);
  unsigned char* sy0 = rows_smem;
  unsigned char* sy1 = sy0 + plan.in_row;
  unsigned char* su = sy1 + plan.in_row;
  unsigned char* sv = su + plan.in_row;
  unsigned char* so = sv + plan.in_row;  // [2][kOutRows][out_row]

  const int rp = blockIdx.x, n = blockIdx.y, tid = threadIdx.x;
  const int we = p.width & ~1;  // a trailing odd column is left untouched
  const uint8_t *yb, *ub, *vb = nullptr;
  if constexpr (TABLE) {
    yb = static_cast<const uint8_t*>(p.y_table[n]);
    ub = static_cast<const uint8_t*>(p.u_table[n]);
    if constexpr (FMT == B2_SRC_I420) vb = static_cast<const uint8_t*>(p.v_table[n]);
  } else {
    yb = p.y + (long long)n * p.y_frame_stride;
    ub = p.u + (long long)n * p.uv_frame_stride;
    if constexpr (FMT == B2_SRC_I420) vb = p.v + (long long)n * p.uv_frame_stride;
  }
  rows_load(sy0, yb + (size_t)(2 * rp) * (unsigned)p.y_pitch, we, tid, kRowsThreads);
  rows_load(sy1, yb + (size_t)(2 * rp + 1) * (unsigned)p.y_pitch, we, tid, kRowsThreads);
  rows_load(su, ub + (size_t)rp * (unsigned)p.uv_pitch, FMT == B2_SRC_NV12 ? we : we / 2, tid,
            kRowsThreads);
  if constexpr (FMT == B2_SRC_I420)
    rows_load(sv, vb + (size_t)rp * (unsigned)p.uv_pitch, we / 2, tid, kRowsThreads);
  __syncthreads();

  const ColorMat& m = p.mat;
  const int chunks = (we + PX - 1) / PX;
  for (int c = tid; c < chunks; c += kRowsThreads) {
    uint32_t yw[2][NW], uw[UVW], vw[UVW];
    lds_words<NW>(sy0, c, yw[0]);
    lds_words<NW>(sy1, c, yw[1]);
    if constexpr (UVB >= 4) {
      lds_words<UVW>(su, c, uw);
      if constexpr (FMT == B2_SRC_I420) lds_words<UVW>(sv, c, vw);
    } else {  // fp32 output from I420: two chroma bytes per plane and chunk
      uw[0] = reinterpret_cast<const uint16_t*>(su)[c];
      vw[0] = reinterpret_cast<const uint16_t*>(sv)[c];
    }
    (void)vw;
    uint32_t out[2][12];
    convert_chunk<FMT, LAYOUT, DTYPE, BGR>(m, p.sb, yw, uw, vw, out);
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        unsigned char* q = LAYOUT == B2_NHWC ? so + (size_t)r * plan.out_row + c * 48 + i * 16
                                             : so + (size_t)(r * 3 + i) * plan.out_row + c * 16;
        *reinterpret_cast<uint4*>(q) =
            make_uint4(out[r][4 * i], out[r][4 * i + 1], out[r][4 * i + 2], out[r][4 * i + 3]);
      }
  }
  __syncthreads();

  uint8_t* dst = reinterpret_cast<uint8_t*>(static_cast<T*>(p.dst) + (long long)n * p.dst_frame_stride);
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const long long row = 2 * rp + r;
    if constexpr (LAYOUT == B2_NHWC) {
      rows_store(dst + row * p.dst_row_pitch * (long long)sizeof(T), so + (size_t)r * plan.out_row,
                 we * 3 * (int)sizeof(T), tid, kRowsThreads);
    } else {
#pragma unroll
      for (int s = 0; s < 3; ++s)
        rows_store(dst + (s * p.dst_plane_stride + row * p.dst_row_pitch) * (long long)sizeof(T),
                   so + (size_t)(r * 3 + s) * plan.out_row, we * (int)sizeof(T), tid, kRowsThreads);
    }
  }
}

// Any-shape path: one thread per 2x2 quad (color_conversion.cu:98-137 has the same ownership).
template <int FMT, int LAYOUT, int DTYPE, bool BGR, bool TABLE>
__global__ void __launch_bounds__(256) dense_quad_kernel(const DenseParams p) {
  using T = typename OutT<DTYPE>::type;
  const int x = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  const int y = (blockIdx.y * blockDim.y + threadIdx.y) * 2;
  const int n = blockIdx.z;
  if (x + 1 >= p.width || y + 1 >= p.height) return;
  const uint8_t *yb, *ub, *vb = nullptr;
  if constexpr (TABLE) {
    yb = static_cast<const uint8_t*>(p.y_table[n]);
    ub = static_cast<const uint8_t*>(p.u_table[n]);
    if constexpr (FMT == B2_SRC_I420) vb = static_cast<const uint8_t*>(p.v_table[n]);
  } else {
    yb = p.y + (long long)n * p.y_frame_stride;
    ub = p.u + (long long)n * p.uv_frame_stride;
    if constexpr (FMT == B2_SRC_I420) vb = p.v + (long long)n * p.uv_frame_stride;
  }
  int cu, cv;
  if constexpr (FMT == B2_SRC_NV12) {
    const uint8_t* q = ub + (long long)(y >> 1) * p.uv_pitch + x;
    cu = q[0];
    cv = q[1];
  } else {
    cu = ub[(long long)(y >> 1) * p.uv_pitch + (x >> 1)];
    cv = vb[(long long)(y >> 1) * p.uv_pitch + (x >> 1)];
  }
  T* dst = static_cast<T*>(p.dst) + (long long)n * p.dst_frame_stride;
#pragma unroll
  for (int r = 0; r < 2; ++r)
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      int c[3];
      pixel_u8(p.mat, yb[(long long)(y + r) * p.y_pitch + x + k], cu, cv, c[BGR ? 2 : 0], c[1],
               c[BGR ? 0 : 2]);
#pragma unroll
      for (int s = 0; s < 3; ++s) {
        const long long idx =
            LAYOUT == B2_NCHW
                ? s * p.dst_plane_stride + (long long)(y + r) * p.dst_row_pitch + x + k
                : (long long)(y + r) * p.dst_row_pitch + (long long)(x + k) * 3 + s;
        dst[idx] = finish<T>((float)c[s], p.sb.s[s], p.sb.b[s]);
      }
    }
}

template <int FMT, int LAYOUT, int DTYPE, bool BGR, bool TABLE>
int launch_t(const DenseLaunch& L, const DenseParams& p, bool vec, cudaStream_t stream) {
  using T = typename OutT<DTYPE>::type;
  constexpr int PX = 16 / (int)sizeof(T);
  const int He = L.height & ~1;
  // gridDim.z is limited to 65535 frames per launch
  for (int n0 = 0; n0 < L.num_frames; n0 += 65535) {
    const int nn = L.num_frames - n0 < 65535 ? L.num_frames - n0 : 65535;
    DenseParams q = p;
    if (TABLE) {
      q.y_table = p.y_table + n0;
      q.u_table = p.u_table + n0;
      if (p.v_table) q.v_table = p.v_table + n0;
    } else {
      q.y = p.y + (long long)n0 * p.y_frame_stride;
      q.u = p.u + (long long)n0 * p.uv_frame_stride;
      if (p.v) q.v = p.v + (long long)n0 * p.uv_frame_stride;
    }
    q.dst = static_cast<T*>(p.dst) + (long long)n0 * p.dst_frame_stride;
    if (vec) {
      const int chunks = (L.width + PX - 1) / PX;
      int bx = ((chunks + 31) / 32) * 32;
      if (bx > kDenseThreads) bx = kDenseThreads;
      const int by = kDenseThreads / bx;
      dim3 block(bx, by), grid((chunks + bx - 1) / bx, (He / 2 + by - 1) / by, nn);
      const size_t smem = LAYOUT == B2_NHWC ? (size_t)(kDenseThreads / 32) * 2 * 32 * 48 : 0;
      dense_vec_kernel<FMT, LAYOUT, DTYPE, BGR, TABLE><<<grid, block, smem, stream>>>(q);
    } else if (rows_plan<LAYOUT, DTYPE>(L.width).total <= 200 * 1024 && L.width >= 16) {
      // unaligned rows: realign through shared memory, one CTA per row pair
      if (He < 2) continue;
      auto kern = dense_rows_kernel<FMT, LAYOUT, DTYPE, BGR, TABLE>;
      const int smem = rows_plan<LAYOUT, DTYPE>(L.width).total;
      if (smem > 48 * 1024)
        B2_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                "raising the shared-memory limit of the rows kernel failed");
      kern<<<dim3(He / 2, nn), kRowsThreads, smem, stream>>>(q);
    } else {
      dim3 block(32, 8), grid((L.width / 2 + 31) / 32, (He / 2 + 7) / 8, nn);
      if (grid.x == 0 || grid.y == 0) continue;
      dense_quad_kernel<FMT, LAYOUT, DTYPE, BGR, TABLE><<<grid, block, 0, stream>>>(q);
    }
    B2_CUDA(cudaPeekAtLastError(), "launch of the dense conversion kernel failed");
  }
  return B2_OK;
}

template <int FMT, int LAYOUT, int DTYPE>
int launch_fld(const DenseLaunch& L, const DenseParams& p, bool vec, cudaStream_t s) {
  const bool bgr = L.order == B2_BGR, table = L.y_table != nullptr;
  if (bgr) return table ? launch_t<FMT, LAYOUT, DTYPE, true, true>(L, p, vec, s)
                        : launch_t<FMT, LAYOUT, DTYPE, true, false>(L, p, vec, s);
  return table ? launch_t<FMT, LAYOUT, DTYPE, false, true>(L, p, vec, s)
               : launch_t<FMT, LAYOUT, DTYPE, false, false>(L, p, vec, s);
}
template <int FMT, int LAYOUT>
int launch_fl(const DenseLaunch& L, const DenseParams& p, bool vec, cudaStream_t s) {
  switch (L.dtype) {
    case B2_U8: return launch_fld<FMT, LAYOUT, B2_U8>(L, p, vec, s);
    case B2_F32: return launch_fld<FMT, LAYOUT, B2_F32>(L, p, vec, s);
    default: return launch_fld<FMT, LAYOUT, B2_BF16>(L, p, vec, s);
  }
}

inline bool mult(long long v, long long m) { return v % m == 0; }

}  // namespace

int launch_dense(const DenseLaunch& L, cudaStream_t stream) {
  if (L.num_frames == 0 || L.width < 2 || L.height < 2) return B2_OK;
  DenseParams p{};
  p.y = L.y; p.u = L.u; p.v = L.v;
  p.y_table = L.y_table; p.u_table = L.u_table; p.v_table = L.v_table;
  if (L.y_pitch > 0x7fffffffLL || L.uv_pitch > 0x7fffffffLL || L.dst_row_pitch > 0x7fffffffLL)
    return fail(B2_ERR_LIMIT, "row pitch beyond 2^31-1 bytes");
  p.y_pitch = (int)L.y_pitch; p.uv_pitch = (int)L.uv_pitch;
  p.y_frame_stride = L.y_frame_stride; p.uv_frame_stride = L.uv_frame_stride;
  p.width = L.width; p.height = L.height & ~1;
  p.mat = L.mat;
  p.dst = L.dst;
  p.dst_row_pitch = (int)L.dst_row_pitch;
  p.dst_plane_stride = L.dst_plane_stride;
  p.dst_frame_stride = L.dst_frame_stride;
  p.sb = L.sb;

  // Can every access of the vector path be a naturally aligned 4/8/16-byte vector?
  const int esz = L.dtype == B2_U8 ? 1 : (L.dtype == B2_F32 ? 4 : 2);
  const int px = 16 / esz;
  const int uvb = L.src_format == B2_SRC_NV12 ? px : px / 2;
  const bool table = L.y_table != nullptr;
  bool vec = mult(L.width, px) && mult(L.y_pitch, px) && mult(L.uv_pitch, uvb) &&
             mult((long long)(uintptr_t)L.dst, 16) && mult(L.dst_row_pitch * esz, 16) &&
             mult(L.dst_frame_stride * esz, 16);
  if (L.layout == B2_NCHW) vec = vec && mult(L.dst_plane_stride * esz, 16);
  if (!table) {
    vec = vec && mult((long long)(uintptr_t)L.y, px) && mult((long long)(uintptr_t)L.u, uvb) &&
          mult(L.y_frame_stride, px) && mult(L.uv_frame_stride, uvb);
    if (L.src_format == B2_SRC_I420) vec = vec && mult((long long)(uintptr_t)L.v, uvb);
  }
  if (L.src_format == B2_SRC_NV12)
    return L.layout == B2_NCHW ? launch_fl<B2_SRC_NV12, B2_NCHW>(L, p, vec, stream)
                               : launch_fl<B2_SRC_NV12, B2_NHWC>(L, p, vec, stream);
  return L.layout == B2_NCHW ? launch_fl<B2_SRC_I420, B2_NCHW>(L, p, vec, stream)
                             : launch_fl<B2_SRC_I420, B2_NHWC>(L, p, vec, stream);
}

}  // namespace b2

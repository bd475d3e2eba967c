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
//   dense_window_kernel rows that start on arbitrary (even) byte boundaries, e.g. packed frames
//                      whose width is not a multiple of 16: one row per thread, the chunk grid of
//                      each row slid so that the OUTPUT accesses stay 16-byte aligned, the input
//                      realigned with 4-byte loads and funnel shifts.
//   dense_shift_kernel the general case (odd addresses and pitches, any width): 4-byte accesses
//                      on both sides, output realigned through shared memory.
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
// w = row[x .. x+NB) for any alignment; bytes outside [0, limit) of the row are not needed and
// only aligned words that hold at least one byte of the row are read.
template <int NB>
__device__ __forceinline__ void load_window(const uint8_t* row, int x, int limit, uint32_t* w) {
  constexpr int NWD = (NB + 3) / 4;
  const uintptr_t addr = (uintptr_t)row + (intptr_t)x;  // x may be negative (before the row)
  const int a = (int)(addr & 3);
  const uint32_t* q = reinterpret_cast<const uint32_t*>(addr - a);
  const int t = x - a;  // row index of the first byte of q[0]
  uint32_t v[NWD + 1];
  if (t >= 0 && t + 4 * (NWD + 1) <= limit) {
#pragma unroll
    for (int i = 0; i <= NWD; ++i) v[i] = __ldg(q + i);
  } else {
#pragma unroll
    for (int i = 0; i <= NWD; ++i) {
      const int b = t + 4 * i;
      v[i] = (b + 3 >= 0 && b < limit) ? __ldg(q + i) : 0u;
    }
  }
#pragma unroll
  for (int i = 0; i < NWD; ++i) w[i] = __funnelshift_r(v[i], v[i + 1], a * 8);
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

constexpr int kDenseThreads = 128;
// 12 resident CTAs (48 warps) per SM: measured best (CTAs of 64 threads are no faster, of 32
// or 256 slower); caps the kernel at 40 registers per thread.
constexpr int kDenseMinBlocks = 12;

template <int FMT, int LAYOUT, int DTYPE, bool BGR, bool TABLE, int ARITH>
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
    const uint8_t* yrow = yb + (size_t)(2 * rp) * (unsigned)p.y_pitch;
    const uint8_t* urow = ub + (size_t)rp * (unsigned)p.uv_pitch;
    const uint8_t* vrow = FMT == B2_SRC_I420 ? vb + (size_t)rp * (unsigned)p.uv_pitch : nullptr;
    constexpr int CDIV = FMT == B2_SRC_NV12 ? 1 : 2;  // luma columns per chroma byte column
    if (TABLE && !aligned) {  // surfaces on odd addresses: realign word by word
      load_window<PX>(yrow, x0, p.width, yw[0]);
      load_window<PX>(yrow + p.y_pitch, x0, p.width, yw[1]);
      load_window<UVB>(urow, x0 / CDIV, p.width / CDIV, uw);
      if constexpr (FMT == B2_SRC_I420) load_window<UVB>(vrow, x0 / CDIV, p.width / CDIV, vw);
    } else {
      load_bytes<PX>(yrow + x0, yw[0]);
      load_bytes<PX>(yrow + x0 + p.y_pitch, yw[1]);
      load_bytes<UVB>(urow + x0 / CDIV, uw);
      if constexpr (FMT == B2_SRC_I420) load_bytes<UVB>(vrow + x0 / CDIV, vw);
    }
    (void)vw;

    const ColorMat m = p.mat;
#pragma unroll
    for (int j = 0; j < NW; ++j) {
      // chroma of the two 2x2 quads under luma word j: lane x = first quad, lane y = second
      Chroma2 c;
      if constexpr (FMT == B2_SRC_NV12) {
        c = chroma2_of<ARITH>(m, make_float2(biased_byte(uw[j], 0), biased_byte(uw[j], 2)),
                       make_float2(biased_byte(uw[j], 1), biased_byte(uw[j], 3)));
      } else {
        const int w = j >> 1, b = (j & 1) * 2;
        c = chroma2_of<ARITH>(m, make_float2(biased_byte(uw[w], b), biased_byte(uw[w], b + 1)),
                       make_float2(biased_byte(vw[w], b), biased_byte(vw[w], b + 1)));
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        // ch[slot][pixel]: the truncated channel value as a subnormal bit pattern (pixel2_ints)
        float ch[3][4];
#pragma unroll
        for (int k = 0; k < 2; ++k) {  // pixels k and k+2 share one packed instruction stream
          float2 cr, cg, cb;
          const float2 by = make_float2(biased_byte(yw[r][j], k), biased_byte(yw[r][j], k + 2));
          pixel2_ints<ARITH>(m, by, c, cr, cg, cb);
          ch[BGR ? 2 : 0][k] = cr.x; ch[BGR ? 2 : 0][k + 2] = cr.y;
          ch[1][k] = cg.x;           ch[1][k + 2] = cg.y;
          ch[BGR ? 0 : 2][k] = cb.x; ch[BGR ? 0 : 2][k + 2] = cb.y;
        }
        if constexpr (DTYPE == B2_U8) {
          if constexpr (LAYOUT == B2_NCHW) {
#pragma unroll
            for (int s = 0; s < 3; ++s)
              out[r][4 * s + j] = pack4_sat(ch[s][0], ch[s][1], ch[s][2], ch[s][3]);
          } else {
            out[r][3 * j + 0] = pack4_sat(ch[0][0], ch[1][0], ch[2][0], ch[0][1]);
            out[r][3 * j + 1] = pack4_sat(ch[1][1], ch[2][1], ch[0][2], ch[1][2]);
            out[r][3 * j + 2] = pack4_sat(ch[2][2], ch[0][3], ch[1][3], ch[2][3]);
            if (j >= 1) stage_piece(r, j - 1);  // piece i needs the luma words up to i + 1
          }
        } else {
          float f[3][4];
#pragma unroll
          for (int s = 0; s < 3; ++s) {
            const uint32_t q = pack4_sat(ch[s][0], ch[s][1], ch[s][2], ch[s][3]);
            // exact 0..255 floats of two pixels, then value * scale + bias, two lanes at a time
            const float2 sc = dup2(p.sb.s[s]), bi = dup2(p.sb.b[s]), off = dup2(-kTwo23);
            const float2 a = x2_fma(x2_add(make_float2(biased_byte(q, 0), biased_byte(q, 1)), off),
                                    sc, bi);
            const float2 b = x2_fma(x2_add(make_float2(biased_byte(q, 2), biased_byte(q, 3)), off),
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

// One thread's block of ROWS (1 or 2) rows x PX pixels under one chroma row: luma words yw,
// chroma words uw (and vw for I420) in, 48 bytes per row out, already in destination order (interleaved: linear; planar: 16 bytes per
// output slot).  The same arithmetic as the vector kernel's inner loop.
template <int FMT, int LAYOUT, int DTYPE, bool BGR, int ARITH, int NW, int UVW, int ROWS>
__device__ __forceinline__ void convert_chunk(const ColorMat& m, const ScaleBias& sb,
                                              const uint32_t (&yw)[ROWS][NW],
                                              const uint32_t (&uw)[UVW],
                                              const uint32_t (&vw)[UVW],
                                              uint32_t (&out)[ROWS][12]) {
#pragma unroll
  for (int j = 0; j < NW; ++j) {
    Chroma2 c;
    if constexpr (FMT == B2_SRC_NV12) {
      c = chroma2_of<ARITH>(m, make_float2(biased_byte(uw[j], 0), biased_byte(uw[j], 2)),
                     make_float2(biased_byte(uw[j], 1), biased_byte(uw[j], 3)));
    } else {
      const int w = j >> 1, b = (j & 1) * 2;
      c = chroma2_of<ARITH>(m, make_float2(biased_byte(uw[w], b), biased_byte(uw[w], b + 1)),
                     make_float2(biased_byte(vw[w], b), biased_byte(vw[w], b + 1)));
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      float ch[3][4];
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        float2 cr, cg, cb;
        const float2 by = make_float2(biased_byte(yw[r][j], k), biased_byte(yw[r][j], k + 2));
        pixel2_ints<ARITH>(m, by, c, cr, cg, cb);
        ch[BGR ? 2 : 0][k] = cr.x; ch[BGR ? 2 : 0][k + 2] = cr.y;
        ch[1][k] = cg.x;           ch[1][k + 2] = cg.y;
        ch[BGR ? 0 : 2][k] = cb.x; ch[BGR ? 0 : 2][k + 2] = cb.y;
      }
      if constexpr (DTYPE == B2_U8) {
        if constexpr (LAYOUT == B2_NCHW) {
#pragma unroll
          for (int s = 0; s < 3; ++s)
            out[r][4 * s + j] = pack4_sat(ch[s][0], ch[s][1], ch[s][2], ch[s][3]);
        } else {
          out[r][3 * j + 0] = pack4_sat(ch[0][0], ch[1][0], ch[2][0], ch[0][1]);
          out[r][3 * j + 1] = pack4_sat(ch[1][1], ch[2][1], ch[0][2], ch[1][2]);
          out[r][3 * j + 2] = pack4_sat(ch[2][2], ch[0][3], ch[1][3], ch[2][3]);
        }
      } else {
        float f[3][4];
#pragma unroll
        for (int s = 0; s < 3; ++s) {
          const uint32_t q = pack4_sat(ch[s][0], ch[s][1], ch[s][2], ch[s][3]);
          const float2 sc = dup2(sb.s[s]), bi = dup2(sb.b[s]), off = dup2(-kTwo23);
          const float2 a = x2_fma(
              x2_add(make_float2(biased_byte(q, 0), biased_byte(q, 1)), off), sc, bi);
          const float2 b = x2_fma(
              x2_add(make_float2(biased_byte(q, 2), biased_byte(q, 3)), off), sc, bi);
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

// ---- window path: rows on even byte boundaries -----------------------------------------------------
// Packed batches whose width is not a multiple of 16 (854x480 video, crops) have rows that start
// anywhere, which rules out the vector kernel's direct 16-byte accesses.  Here a thread owns PX
// pixels of ONE row, and the chunk grid of every row is slid left by d pixels, d chosen per row
// so that chunk boundaries fall on 16-byte boundaries of the DESTINATION row.  The output side is
// then that of the vector kernel (16-byte stores, bulk copies for interleaved output; only the
// first and last chunk of a row are ragged), and the alignment work moves to the source side,
// where it is cheap: the 4-byte words that cover the chunk, funnel-shifted.  d must be even so
// that a chunk starts on a chroma pair, which holds when the destination rows start on even
// element pairs; rows 2r and 2r+1 get different d, so each thread loads its own chroma.

constexpr int kWindowThreads = 128;

template <int FMT, int LAYOUT, int DTYPE, bool BGR, bool TABLE, int ARITH>
__global__ void __launch_bounds__(kWindowThreads) dense_window_kernel(const DenseParams p) {
  using T = typename OutT<DTYPE>::type;
  constexpr int ESZ = (int)sizeof(T);
  constexpr int PX = 16 / ESZ;
  constexpr int NW = PX / 4;
  constexpr int UVB = FMT == B2_SRC_NV12 ? PX : PX / 2;
  constexpr int UVW = (UVB + 3) / 4;
  extern __shared__ __align__(128) unsigned char window_smem[];  // interleaved: 1536 B per warp
  const int lane = threadIdx.x & 31;

  const int row = blockIdx.y, n = blockIdx.z;
  const int we = p.width & ~1;  // a trailing odd column is left untouched
  uint8_t* grow = reinterpret_cast<uint8_t*>(static_cast<T*>(p.dst) + (long long)n * p.dst_frame_stride +
                                             (long long)row * p.dst_row_pitch);
  // pixels to slide the chunk grid left so that chunks start on 16-byte boundaries of this row
  const int a = (int)((uintptr_t)grow & 15);
  int d;
  if constexpr (LAYOUT == B2_NCHW) d = (a / ESZ) & (PX - 1);                // ESZ*d = a (mod 16)
  else if constexpr (DTYPE == B2_U8) d = (11 * a) & 15;                      // 3d = a (mod 16)
  else if constexpr (DTYPE == B2_BF16) d = (3 * (a >> 1)) & 7;               // 6d = a (mod 16)
  else d = (3 * (a >> 2)) & 3;                                               // 12d = a (mod 16)
  const int cx = blockIdx.x * blockDim.x + threadIdx.x;
  const int x0 = cx * PX - d, wx0 = (cx - lane) * PX - d;
  if (wx0 >= we) return;  // the whole warp lies past the row end

  uint32_t out[1][12];
  if (x0 < we) {
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
    uint32_t yw[1][NW], uw[UVW], vw[UVW];
    load_window<PX>(yb + (size_t)row * (unsigned)p.y_pitch, x0, we, yw[0]);
    const size_t uv_off = (size_t)(row >> 1) * (unsigned)p.uv_pitch;
    if constexpr (FMT == B2_SRC_NV12) {
      load_window<UVB>(ub + uv_off, x0, we, uw);
    } else {
      load_window<UVB>(ub + uv_off, x0 / 2, we / 2, uw);
      load_window<UVB>(vb + uv_off, x0 / 2, we / 2, vw);
    }
    (void)vw;
    convert_chunk<FMT, LAYOUT, DTYPE, BGR, ARITH>(p.mat, p.sb, yw, uw, vw, out);
  }

  if constexpr (LAYOUT == B2_NCHW) {
    if (x0 >= we) return;
    if (x0 >= 0 && x0 + PX <= we) {
#pragma unroll
      for (int s = 0; s < 3; ++s)
        __stcs(reinterpret_cast<uint4*>(grow + (s * p.dst_plane_stride + x0) * (long long)ESZ),
               make_uint4(out[0][4 * s], out[0][4 * s + 1], out[0][4 * s + 2], out[0][4 * s + 3]));
    } else {  // first or last chunk of the row: element by element
#pragma unroll
      for (int s = 0; s < 3; ++s) {
        T* q = reinterpret_cast<T*>(grow) + s * p.dst_plane_stride + x0;
#pragma unroll
        for (int k = 0; k < PX; ++k) {
          if (x0 + k < 0 || x0 + k >= we) continue;
          const uint32_t word = out[0][4 * s + k * ESZ / 4];
          if constexpr (ESZ == 1) reinterpret_cast<uint8_t*>(q)[k] = (uint8_t)(word >> (8 * (k & 3)));
          else if constexpr (ESZ == 2)
            reinterpret_cast<uint16_t*>(q)[k] = (uint16_t)(word >> (16 * (k & 1)));
          else reinterpret_cast<uint32_t*>(q)[k] = word;
        }
      }
    }
  } else {
    unsigned char* seg = window_smem + (threadIdx.x >> 5) * 1536;
    if (x0 < we) {
#pragma unroll
      for (int i = 0; i < 3; ++i)
        *reinterpret_cast<uint4*>(seg + lane * 48 + i * 16) =
            make_uint4(out[0][4 * i], out[0][4 * i + 1], out[0][4 * i + 2], out[0][4 * i + 3]);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    // The warp's 1536-byte segment starts 16-byte aligned at gseg; bytes [s0, s1) of it lie in
    // the row.  Whole 16-byte pieces leave as one bulk copy, the ragged ends byte by byte.
    const int seg_off = wx0 * (3 * ESZ);  // rows are shorter than 2^31 bytes
    uint8_t* gseg = grow + seg_off;
    const int left = we * (3 * ESZ) - seg_off;
    int b0 = 0, b1 = 1536;
    if (seg_off < 0 || left < 1536) {  // first or last segment of the row
      const int s0 = seg_off < 0 ? -seg_off : 0;
      const int s1 = left < 1536 ? left : 1536;
      b0 = (s0 + 15) & ~15;
      b1 = s1 & ~15;
      const int head_end = b1 > b0 ? b0 : s1;
      if (s0 + lane < head_end) gseg[s0 + lane] = seg[s0 + lane];
      if (b1 > b0 && b1 + lane < s1) gseg[b1 + lane] = seg[b1 + lane];
    }
    if (lane == 0 && b1 > b0) {
      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gseg + b0),
                   "r"(smem_addr(seg + b0)), "r"((uint32_t)(b1 - b0))
                   : "memory");
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      // the staging buffer must outlive the engine's reads of it
      asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    }
  }
}

// ---- shift path: any alignment, no block-wide staging --------------------------------------------
// For rows on arbitrary byte boundaries.  A warp owns the same 2-row x 32*PX-pixel block as in the
// vector kernel, but its lanes take the luma words of a row in turn (lane l owns words l, l+32,
// ...), so every access is a coalesced 4-byte access and a row that starts between two words
// costs one funnel shift per word, with no dependence on where the row starts.  The output
// segments of the warp are assembled in shared memory and leave as 4-byte stores shifted the
// other way, with byte stores at the ragged ends.  Needs only __syncwarp.

// The 32-bit word at any address p (its first byte is valid; bytes at or past `end` are not
// needed).  Reads only aligned words that hold at least one valid byte.
__device__ __forceinline__ uint32_t ldg_word_any(const uint8_t* p, const uint8_t* end) {
  const int a = (int)((uintptr_t)p & 3);
  const uint8_t* base = p - a;
  const uint32_t lo = __ldg(reinterpret_cast<const uint32_t*>(base));
  uint32_t hi = 0u;
  if (a != 0 && base + 4 < end) hi = __ldg(reinterpret_cast<const uint32_t*>(base + 4));
  return __funnelshift_r(lo, hi, a * 8);
}

template <int N>
__device__ __forceinline__ void sts_words(unsigned char* q, const uint32_t* w) {
  if constexpr (N % 4 == 0) {
#pragma unroll
    for (int i = 0; i < N; i += 4)
      *reinterpret_cast<uint4*>(q + 4 * i) = make_uint4(w[i], w[i + 1], w[i + 2], w[i + 3]);
  } else if constexpr (N % 2 == 0) {
#pragma unroll
    for (int i = 0; i < N; i += 2) *reinterpret_cast<uint2*>(q + 4 * i) = make_uint2(w[i], w[i + 1]);
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) *reinterpret_cast<uint32_t*>(q + 4 * i) = w[i];
  }
}

// g[0..n) = s[0..n) by one warp for any alignment of g; s is 4-byte aligned shared memory,
// readable up to n + 4 bytes; n <= MAXB.
template <int MAXB>
__device__ __forceinline__ void warp_store(uint8_t* g, const unsigned char* s, int n, int lane) {
  int head = (int)((4 - ((uintptr_t)g & 3)) & 3);
  if (head > n) head = n;
  const int nw = (n - head) >> 2;
  const int tail0 = head + (nw << 2);
  if (lane < head) g[lane] = s[lane];
  if (tail0 + lane < n) g[tail0 + lane] = s[tail0 + lane];
  const uint32_t* sw = reinterpret_cast<const uint32_t*>(s);
  uint32_t* gw = reinterpret_cast<uint32_t*>(g + head);
  const int bs = head * 8;
  if (bs == 0) {
#pragma unroll
    for (int i = 0; i < MAXB / 128; ++i) {
      const int m = lane + 32 * i;
      if (m < nw) __stcs(gw + m, sw[m]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < MAXB / 128; ++i) {
      const int m = lane + 32 * i;
      if (m < nw) __stcs(gw + m, __funnelshift_r(sw[m], sw[m + 1], bs));
    }
  }
}

constexpr int kShiftThreads = 128;
constexpr int kShiftWarpSmem = 2 * 1536 + 16;  // two interleaved or six planar row segments

template <int FMT, int LAYOUT, int DTYPE, bool BGR, bool TABLE, int ARITH>
__global__ void __launch_bounds__(kShiftThreads) dense_shift_kernel(const DenseParams p) {
  using T = typename OutT<DTYPE>::type;
  constexpr int ESZ = (int)sizeof(T);
  constexpr int PX = 16 / ESZ;
  constexpr int NW = PX / 4;
  constexpr int UVB = FMT == B2_SRC_NV12 ? PX : PX / 2;
  constexpr int UVW = (UVB + 3) / 4;
  constexpr int KW = 3 * ESZ;  // interleaved output words per luma word
  constexpr int CW = ESZ;      // planar output words per channel and luma word
  extern __shared__ __align__(128) unsigned char shift_smem[];
  const int lane = threadIdx.x & 31;
  unsigned char* wsm = shift_smem + (threadIdx.x >> 5) * kShiftWarpSmem;

  const int rp = blockIdx.y, n = blockIdx.z;
  const int we = p.width & ~1;  // a trailing odd column is left untouched
  const int wx0 = (blockIdx.x * (kShiftThreads / 32) + (threadIdx.x >> 5)) * 32 * PX;
  if (wx0 >= we) return;  // the whole warp lies past the row end

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
  const uint8_t* y0 = yb + (size_t)(2 * rp) * (unsigned)p.y_pitch;
  const uint8_t* y1 = y0 + p.y_pitch;
  const uint8_t* u0 = ub + (size_t)rp * (unsigned)p.uv_pitch;
  const uint8_t* v0 = FMT == B2_SRC_I420 ? vb + (size_t)rp * (unsigned)p.uv_pitch : nullptr;

  uint32_t yw[2][NW], uw[UVW], vw[UVW];
#pragma unroll
  for (int i = 0; i < UVW; ++i) uw[i] = vw[i] = 0u;
#pragma unroll
  for (int j = 0; j < NW; ++j) {
    const int x = wx0 + 4 * (lane + 32 * j);  // first pixel of this lane's luma word j
    yw[0][j] = yw[1][j] = 0u;
    if (x < we) {
      yw[0][j] = ldg_word_any(y0 + x, y0 + we);
      yw[1][j] = ldg_word_any(y1 + x, y1 + we);
      if constexpr (FMT == B2_SRC_NV12) {
        uw[j] = ldg_word_any(u0 + x, u0 + we);
      } else {  // two bytes per plane under four pixels
        uw[j >> 1] |= (ldg_word_any(u0 + x / 2, u0 + we / 2) & 0xffffu) << (16 * (j & 1));
        vw[j >> 1] |= (ldg_word_any(v0 + x / 2, v0 + we / 2) & 0xffffu) << (16 * (j & 1));
      }
    }
  }
  (void)vw;
  uint32_t out[2][12];
  convert_chunk<FMT, LAYOUT, DTYPE, BGR, ARITH>(p.mat, p.sb, yw, uw, vw, out);
#pragma unroll
  for (int r = 0; r < 2; ++r)
#pragma unroll
    for (int j = 0; j < NW; ++j) {
      const int word = lane + 32 * j;
      if constexpr (LAYOUT == B2_NHWC) {
        sts_words<KW>(wsm + r * 1536 + word * (KW * 4), &out[r][KW * j]);
      } else {
#pragma unroll
        for (int s = 0; s < 3; ++s)
          sts_words<CW>(wsm + (r * 3 + s) * 512 + word * (CW * 4), &out[r][4 * s + CW * j]);
      }
    }
  __syncwarp();

  const int px = we - wx0 < 32 * PX ? we - wx0 : 32 * PX;
  uint8_t* dst = reinterpret_cast<uint8_t*>(static_cast<T*>(p.dst) + (long long)n * p.dst_frame_stride);
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const long long row = 2 * rp + r;
    if constexpr (LAYOUT == B2_NHWC) {
      warp_store<1536>(dst + (row * p.dst_row_pitch + (long long)wx0 * 3) * ESZ, wsm + r * 1536,
                       px * 3 * ESZ, lane);
    } else {
#pragma unroll
      for (int s = 0; s < 3; ++s)
        warp_store<512>(dst + (s * p.dst_plane_stride + row * p.dst_row_pitch + wx0) * ESZ,
                        wsm + (r * 3 + s) * 512, px * ESZ, lane);
    }
  }
}

inline bool mult(long long v, long long m) { return v % m == 0; }

template <int FMT, int LAYOUT, int DTYPE, bool BGR, bool TABLE, int ARITH>
int launch_t(const DenseLaunch& L, const DenseParams& p, bool vec, cudaStream_t stream) {
  using T = typename OutT<DTYPE>::type;
  constexpr int PX = 16 / (int)sizeof(T);
  const int He = L.height & ~1;
  // The window kernel needs destination rows that start on even element pairs (so that its chunk
  // grid starts on a chroma pair) and, for planar output, planes that are equally aligned.
  constexpr int kPair = 2 * (int)sizeof(T);
  bool window = mult((long long)(uintptr_t)p.dst, kPair) &&
                mult((long long)p.dst_row_pitch * (long long)sizeof(T), kPair) &&
                mult(p.dst_frame_stride * (long long)sizeof(T), kPair);
  if (LAYOUT == B2_NCHW) window = window && mult(p.dst_plane_stride * (long long)sizeof(T), 16);
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
      dense_vec_kernel<FMT, LAYOUT, DTYPE, BGR, TABLE, ARITH><<<grid, block, smem, stream>>>(q);
    } else if (window) {
      if (He < 2) continue;
      const int chunks = ((L.width & ~1) + 2 * PX - 2) / PX;  // the grid slides by up to PX-1 pixels
      dim3 grid((chunks + kWindowThreads - 1) / kWindowThreads, He, nn);
      const size_t smem = LAYOUT == B2_NHWC ? (size_t)(kWindowThreads / 32) * 1536 : 0;
      dense_window_kernel<FMT, LAYOUT, DTYPE, BGR, TABLE, ARITH><<<grid, kWindowThreads, smem, stream>>>(q);
    } else {
      if (He < 2) continue;
      const int per_cta = kShiftThreads * PX;  // pixels of a row per CTA
      dim3 grid(((L.width & ~1) + per_cta - 1) / per_cta, He / 2, nn);
      dense_shift_kernel<FMT, LAYOUT, DTYPE, BGR, TABLE, ARITH>
          <<<grid, kShiftThreads, (kShiftThreads / 32) * kShiftWarpSmem, stream>>>(q);
    }
    B2_CUDA(cudaPeekAtLastError(), "launch of the dense conversion kernel failed");
  }
  return B2_OK;
}

template <int FMT, int LAYOUT, int DTYPE, int ARITH>
int launch_fld(const DenseLaunch& L, const DenseParams& p, bool vec, cudaStream_t s) {
  const bool bgr = L.order == B2_BGR, table = L.y_table != nullptr;
  if (bgr) return table ? launch_t<FMT, LAYOUT, DTYPE, true, true, ARITH>(L, p, vec, s)
                        : launch_t<FMT, LAYOUT, DTYPE, true, false, ARITH>(L, p, vec, s);
  return table ? launch_t<FMT, LAYOUT, DTYPE, false, true, ARITH>(L, p, vec, s)
               : launch_t<FMT, LAYOUT, DTYPE, false, false, ARITH>(L, p, vec, s);
}
template <int FMT, int LAYOUT, int ARITH>
int launch_fla(const DenseLaunch& L, const DenseParams& p, bool vec, cudaStream_t s) {
  switch (L.dtype) {
    case B2_U8: return launch_fld<FMT, LAYOUT, B2_U8, ARITH>(L, p, vec, s);
    case B2_F32: return launch_fld<FMT, LAYOUT, B2_F32, ARITH>(L, p, vec, s);
    default: return launch_fld<FMT, LAYOUT, B2_BF16, ARITH>(L, p, vec, s);
  }
}
template <int FMT, int LAYOUT>
int launch_fl(const DenseLaunch& L, const DenseParams& p, bool vec, cudaStream_t s) {
  return L.arith == B2_ARITH_SWSCALE ? launch_fla<FMT, LAYOUT, B2_ARITH_SWSCALE>(L, p, vec, s)
                                     : launch_fla<FMT, LAYOUT, B2_ARITH_REFERENCE>(L, p, vec, s);
}

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
  if (L.dst_row_pitch * esz > 0x7fffffffLL || 3LL * L.width * esz > 0x7fffffffLL)
    return fail(B2_ERR_LIMIT, "output row beyond 2^31-1 bytes");
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

// Dense colour conversion: every pixel of every frame, no resampling.
//
// Three kernels.
//   dense_vec_kernel   the fast path.  One thread owns a 2-row x PX-pixel block (PX = 16 bytes
//                      of output per channel: 16 px for u8, 8 for bf16, 4 for fp32), so the two
//                      rows share one chroma load, every global load is one 4/8/16-byte vector
//                      and every global store is a 16-byte vector.  Planar output is stored
//                      straight from registers (a warp writes 512 contiguous bytes per
//                      instruction).  Interleaved output (48 bytes per thread per row) is staged
//                      in shared memory by the warp and leaves as one bulk asynchronous copy
//                      (cp.async.bulk shared->global) per row segment.
//   dense_flat_kernel  packed OUTPUT frames whose width is not a multiple of the vector size
//                      (854, 1366, 1918 ...) or that start on an unaligned address.  With rows
//                      back to back a frame's output is a flat array in pixel order, so a thread
//                      takes PX consecutive pixels of the frame, counted from the first pixel
//                      whose output is 16-byte aligned.  Every store is then an aligned vector
//                      whatever the width; only the sources are realigned (8-byte loads, word
//                      selects and funnel shifts), a chunk that runs over the end of a row
//                      fetches its second part separately, and the ends of a frame are stored
//                      byte by byte.  Two variants: source rows back to back too (luma is then
//                      one flat array as well), and pitched surfaces / pointer tables.
//   dense_any_kernel   everything else (destinations with a row pitch or on odd addresses, odd
//                      widths): the vector kernel's thread layout, the source realigned with
//                      4-byte loads, the output laid out in shared memory at the destination's
//                      offset modulo 16 so that its aligned interior still leaves as one bulk
//                      copy per row segment.
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
  // dense_flat_kernel only
  int pixels;         // width * height: pixels of a frame
  int y_limit;        // bytes from the start of the luma plane to the end of its last row
  int chroma_limit;   // ... of a chroma plane
  unsigned w_recip;   // 2^32 / width, rounded down: pixel index -> row by multiply-high
  int rows_per_warp;  // rows a warp's run of consecutive pixels can touch
  int flat_packed;    // source rows lie back to back too (pitch == width, no pointer table)
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

// ---- packed frames of any width ------------------------------------------------------------------
// A frame whose rows lie back to back (pitch == width, even) is a flat array of width * height luma
// bytes, its output a flat array of pixels in the same order.  A lane converts PX consecutive
// pixels of that array (one row's worth of convert_chunk); chunks are counted from pixel i0, the
// first even pixel of the frame whose output address is a multiple of 16, so that a lane's 48
// interleaved bytes (or 16 bytes per plane) always leave as aligned vectors.  What is left is
//   in:    luma and chroma windows at arbitrary byte offsets (load_window);
//   rows:  a chunk that starts k1 < PX pixels before the end of an even row continues in the next
//          row under the SAME chroma row: its chroma is fetched in two parts and blended (after an
//          odd row the next chroma row follows in memory, and nothing is to be done);
//   ends:  the first and the last chunk of a frame hold pixels outside it; their bytes are not
//          stored (interleaved: the ragged ends of the warp's staged bytes go out byte by byte).
// 128 threads, two chunks per lane (a warp converts 64 consecutive chunks), 12 CTAs per SM:
// measured best (one or three chunks per lane, CTAs of 64 threads and 10 or 16 CTAs per SM are
// 1-8 % slower).
constexpr int kFlatThreads = 128;
constexpr int kFlatMinBlocks = 12;
constexpr int kFlatChunks = 2;  // chunks per lane: a warp converts 64 consecutive chunks

// load_window for a window that lies at least 8 bytes inside its plane at both ends.  Sixteen
// bytes come as the three aligned 8-byte vectors that cover them (fewer, wider requests than five
// 4-byte words: the lanes of a warp are 16 bytes apart, so every load instruction touches four
// cache lines whatever its width), then a word select and a funnel shift per word; no branch, so
// the loads of all the windows of a lane are in flight together.
template <int NB>
__device__ __forceinline__ void load_window_inside(const uint8_t* base, int x, uint32_t* w) {
  constexpr int NWD = (NB + 3) / 4;
  const uintptr_t addr = (uintptr_t)base + (intptr_t)x;
  if constexpr (NB == 16) {
    const int a = (int)(addr & 7);
    const uint2* q = reinterpret_cast<const uint2*>(addr - a);
    const uint2 v0 = __ldg(q), v1 = __ldg(q + 1), v2 = __ldg(q + 2);
    const bool up = a >= 4;  // the window starts in the upper word of v0
    const uint32_t t0 = up ? v0.y : v0.x, t1 = up ? v1.x : v0.y, t2 = up ? v1.y : v1.x,
                   t3 = up ? v2.x : v1.y, t4 = up ? v2.y : v2.x;
    const int sh = (a & 3) * 8;
    w[0] = __funnelshift_r(t0, t1, sh);
    w[1] = __funnelshift_r(t1, t2, sh);
    w[2] = __funnelshift_r(t2, t3, sh);
    w[3] = __funnelshift_r(t3, t4, sh);
  } else {
    const int a = (int)(addr & 3);
    const uint32_t* q = reinterpret_cast<const uint32_t*>(addr - a);
    uint32_t v[NWD + 1];
#pragma unroll
    for (int i = 0; i <= NWD; ++i) v[i] = __ldg(q + i);
#pragma unroll
    for (int i = 0; i < NWD; ++i) w[i] = __funnelshift_r(v[i], v[i + 1], a * 8);
  }
}

// Luma and chroma words of the chunk that starts at pixel i of the frame (i < p.pixels; negative
// for the partial chunk in front of the frame).  INSIDE: the caller knows that the chunk lies at
// least four rows away from both ends of the frame, so no window needs a bounds check.
template <int FMT, int PX, bool INSIDE, bool PACKED, int NW, int UVW>
__device__ __forceinline__ void flat_load(const DenseParams& p, const uint8_t* yb,
                                          const uint8_t* ub, const uint8_t* vb, int i,
                                          uint32_t (&yw)[1][NW], uint32_t (&uw)[UVW],
                                          uint32_t (&vw)[UVW]) {
  constexpr int CDIV = FMT == B2_SRC_NV12 ? 1 : 2;  // luma columns per chroma byte column
  constexpr int UVB = PX / CDIV;
  // row and column of pixel i; a negative i belongs to the partial chunk in front of row 0
  int y = INSIDE || i > 0 ? (int)__umulhi((unsigned)i, p.w_recip) : 0;
  int x = i - y * p.width;
  if (x >= p.width) {  // the rounded-down reciprocal is short by at most one
    x -= p.width;
    ++y;
  }
  const int k1 = p.width - x;  // pixels of the chunk that lie in row y
  uint32_t u2[UVW], v2[UVW];
  (void)vw;
  (void)v2;
  if constexpr (!PACKED) {
    // Pitched source rows (decoder surfaces, a pointer per frame): a chunk that runs over the end
    // of row y continues at the start of row y + 1, so its luma comes in two parts as well, and
    // its chroma from the row that y + 1 belongs to.
    const bool split = k1 < PX;
    const int la = y * p.y_pitch + x, lb = (y + 1) * p.y_pitch - k1;
    const int ca = (y >> 1) * p.uv_pitch + x / CDIV;  // x is even
    const int cb = ((y + 1) >> 1) * p.uv_pitch - k1 / CDIV;
    uint32_t y2[NW];
    if constexpr (INSIDE) {
      load_window_inside<PX>(yb, la, yw[0]);
      load_window_inside<UVB>(ub, ca, uw);
      if constexpr (FMT == B2_SRC_I420) load_window_inside<UVB>(vb, ca, vw);
      if (split) {
        load_window_inside<PX>(yb, lb, y2);
        load_window_inside<UVB>(ub, cb, u2);
        if constexpr (FMT == B2_SRC_I420) load_window_inside<UVB>(vb, cb, v2);
      }
    } else {
      load_window<PX>(yb, la, p.y_limit, yw[0]);
      load_window<UVB>(ub, ca, p.chroma_limit, uw);
      if constexpr (FMT == B2_SRC_I420) load_window<UVB>(vb, ca, p.chroma_limit, vw);
      if (split) {
        load_window<PX>(yb, lb, p.y_limit, y2);
        load_window<UVB>(ub, cb, p.chroma_limit, u2);
        if constexpr (FMT == B2_SRC_I420) load_window<UVB>(vb, cb, p.chroma_limit, v2);
      }
    }
    if (split) {
      auto keep_mask = [](int m) {  // the low m bytes of a word
        return m >= 4 ? 0xffffffffu : (m <= 0 ? 0u : (1u << (8 * m)) - 1u);
      };
#pragma unroll
      for (int j = 0; j < NW; ++j) {
        const uint32_t keep = keep_mask(k1 - 4 * j);
        yw[0][j] = (yw[0][j] & keep) | (y2[j] & ~keep);
      }
#pragma unroll
      for (int j = 0; j < UVW; ++j) {
        const uint32_t keep = keep_mask(k1 / CDIV - 4 * j);
        uw[j] = (uw[j] & keep) | (u2[j] & ~keep);
        if constexpr (FMT == B2_SRC_I420) vw[j] = (vw[j] & keep) | (v2[j] & ~keep);
      }
    }
    return;
  }
  const int cw = p.width / CDIV;               // bytes of a chroma row
  const int ca = (y >> 1) * cw + x / CDIV;     // x is even
  const bool split = k1 < PX && !(y & 1);      // ... the rest under the same chroma row
  if (INSIDE ||
      (i >= 4 && i + PX + 4 <= p.pixels && ca >= cw + 4 && ca + UVB + 4 <= p.chroma_limit)) {
    load_window_inside<PX>(yb, i, yw[0]);
    load_window_inside<UVB>(ub, ca, uw);
    if constexpr (FMT == B2_SRC_I420) load_window_inside<UVB>(vb, ca, vw);
    if (split) {
      load_window_inside<UVB>(ub, ca - cw, u2);
      if constexpr (FMT == B2_SRC_I420) load_window_inside<UVB>(vb, ca - cw, v2);
    }
  } else {
    load_window<PX>(yb, i, p.pixels, yw[0]);
    load_window<UVB>(ub, ca, p.chroma_limit, uw);
    if constexpr (FMT == B2_SRC_I420) load_window<UVB>(vb, ca, p.chroma_limit, vw);
    if (split) {
      load_window<UVB>(ub, ca - cw, p.chroma_limit, u2);
      if constexpr (FMT == B2_SRC_I420) load_window<UVB>(vb, ca - cw, p.chroma_limit, v2);
    }
  }
  if (split) {
    const int kb = k1 / CDIV;  // chroma bytes that belong to row y
#pragma unroll
    for (int j = 0; j < UVW; ++j) {
      const int m = kb - 4 * j;
      const uint32_t keep = m >= 4 ? 0xffffffffu : (m <= 0 ? 0u : (1u << (8 * m)) - 1u);
      uw[j] = (uw[j] & keep) | (u2[j] & ~keep);
      if constexpr (FMT == B2_SRC_I420) vw[j] = (vw[j] & keep) | (v2[j] & ~keep);
    }
  }
}

template <int FMT, int LAYOUT, int DTYPE, bool BGR, int ARITH, bool PACKED>
__global__ void __launch_bounds__(kFlatThreads, kFlatMinBlocks) dense_flat_kernel(const DenseParams p) {
  using T = typename OutT<DTYPE>::type;
  constexpr int ESZ = (int)sizeof(T);
  constexpr int PX = 16 / ESZ;
  constexpr int NW = PX / 4;
  constexpr int UVW = ((FMT == B2_SRC_NV12 ? PX : PX / 2) + 3) / 4;
  constexpr int CH = kFlatChunks;
  extern __shared__ __align__(128) unsigned char flat_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n = blockIdx.z;
  uint8_t* const dstb =
      reinterpret_cast<uint8_t*>(static_cast<T*>(p.dst) + (long long)n * p.dst_frame_stride);
  // i0: the launcher guarantees that an even one exists (the frame starts on a multiple of
  // 2 * ESZ bytes).  Interleaved: 3 * ESZ * i0 + d = 0 (mod 16); planar: ESZ * i0 + d = 0.
  const int d = (int)((uintptr_t)dstb & 15);
  int i0;
  if constexpr (LAYOUT == B2_NHWC)
    i0 = ESZ == 1 ? (5 * d) & 15 : (ESZ == 2 ? d >> 1 : d >> 2);
  else
    i0 = ((16 - d) & 15) / ESZ;
  const int start = i0 ? i0 - PX : 0;  // first pixel of chunk 0 (negative: a partial chunk)
  // the warp's first pixel: its lanes take chunks lane, lane + 32, ...
  const int wi = start + (int)(blockIdx.x * (kFlatThreads / 32) + warp) * (CH * 32 * PX);
  if (wi >= p.pixels) return;

  const uint8_t *yb, *ub, *vb = nullptr;
  if (!PACKED && p.y_table != nullptr) {  // a pointer per frame and plane
    yb = static_cast<const uint8_t*>(p.y_table[n]);
    ub = static_cast<const uint8_t*>(p.u_table[n]);
    if constexpr (FMT == B2_SRC_I420) vb = static_cast<const uint8_t*>(p.v_table[n]);
  } else {
    yb = p.y + (long long)n * p.y_frame_stride;
    ub = p.u + (long long)n * p.uv_frame_stride;
    if constexpr (FMT == B2_SRC_I420) vb = p.v + (long long)n * p.uv_frame_stride;
  }
  uint32_t yw[CH][1][NW], uw[CH][UVW], vw[CH][UVW];
  // Four rows or more from both ends of the frame (the row estimate may be short by one), every
  // chunk of the warp is whole and none of its windows needs a bounds check.
  const int row0 = wi > 0 ? (int)__umulhi((unsigned)wi, p.w_recip) : 0;
  const bool inside = row0 >= 4 && row0 + p.rows_per_warp + 8 <= p.height;
  if (inside) {
#pragma unroll
    for (int k = 0; k < CH; ++k)
      flat_load<FMT, PX, true, PACKED>(p, yb, ub, vb, wi + (k * 32 + lane) * PX, yw[k], uw[k],
                                       vw[k]);
  } else {
#pragma unroll
    for (int k = 0; k < CH; ++k) {
      const int i = wi + (k * 32 + lane) * PX;
      if (i < p.pixels) flat_load<FMT, PX, false, PACKED>(p, yb, ub, vb, i, yw[k], uw[k], vw[k]);
    }
  }
  unsigned char* wsm = flat_smem + warp * (CH * 32 * 48);
#pragma unroll
  for (int k = 0; k < CH; ++k) {
    const int i = wi + (k * 32 + lane) * PX;
    if (!inside && i >= p.pixels) continue;
    uint32_t out[1][12];
    convert_chunk<FMT, LAYOUT, DTYPE, BGR, ARITH>(p.mat, p.sb, yw[k], uw[k], vw[k], out);
    if constexpr (LAYOUT == B2_NCHW) {
      const bool whole = inside || (i >= 0 && i + PX <= p.pixels);
#pragma unroll
      for (int s = 0; s < 3; ++s) {
        uint8_t* q = dstb + (s * p.dst_plane_stride + i) * ESZ;
        if (whole) {
          __stcs(reinterpret_cast<uint4*>(q), make_uint4(out[0][4 * s], out[0][4 * s + 1],
                                                         out[0][4 * s + 2], out[0][4 * s + 3]));
        } else {
#pragma unroll
          for (int b = 0; b < 16; ++b) {
            const int px = i + b / ESZ;
            if (px >= 0 && px < p.pixels) q[b] = (uint8_t)(out[0][4 * s + b / 4] >> (8 * (b % 4)));
          }
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 3; ++j)
        *reinterpret_cast<uint4*>(wsm + (k * 32 + lane) * 48 + 16 * j) =
            make_uint4(out[0][4 * j], out[0][4 * j + 1], out[0][4 * j + 2], out[0][4 * j + 3]);
    }
  }
  if constexpr (LAYOUT == B2_NHWC) {
    // The warp's CH x 32 x 48 bytes are contiguous in the destination and start on a multiple
    // of 16: the aligned interior leaves as one bulk copy, the ragged ends of a frame byte by byte.
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    const long long first = 3LL * ESZ * wi, total = 3LL * ESZ * p.pixels;  // bytes of the frame
    const long long lo = first > 0 ? first : 0;
    const long long hi = first + CH * 32 * 48 < total ? first + CH * 32 * 48 : total;
    uint8_t* g = dstb + lo;
    const unsigned char* data = wsm + (lo - first);  // congruent to g modulo 16
    const int nbytes = (int)(hi - lo);
    int head = (int)((16 - ((uintptr_t)g & 15)) & 15);
    if (head > nbytes) head = nbytes;
    const int body = (nbytes - head) & ~15;
    const int tail0 = head + body;
    if (lane < head) g[lane] = data[lane];
    if (tail0 + lane < nbytes) g[tail0 + lane] = data[tail0 + lane];
    if (lane == 0 && body > 0) {
      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(g + head),
                   "r"(smem_addr(data + head)), "r"((uint32_t)body)
                   : "memory");
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      // the staging buffer must outlive the engine's reads of it
      asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    }
  }
}

// ---- any-alignment path ------------------------------------------------------------------------
// Rows on arbitrary byte boundaries (packed frames whose width is not a multiple of 16: 854x480,
// 1366x768; crops; surfaces at odd addresses), any width >= 2.  The thread layout is the vector
// kernel's -- a warp owns 2 rows x 32*PX pixels, a lane 2 rows x PX pixels under one chroma row,
// chunks counted from the start of the row so that a chunk starts on a chroma pair -- and the
// alignment work sits at the two ends of it:
//   in:   a lane reads the aligned 4-byte words that cover its bytes and funnel-shifts them into
//         place (load_window);
//   out:  the bytes a warp produces for one row (or one row of one plane) are contiguous in the
//         destination.  The warp lays them out in shared memory at the destination's offset
//         modulo 16 -- a lane shifts its words by the offset modulo 4, taking the spilled bytes
//         of its left neighbour with one shuffle -- so that shared and global addresses are
//         congruent; the 16-byte-aligned interior then leaves as ONE bulk asynchronous copy and
//         the ragged ends (< 16 bytes each) as byte stores.
constexpr int kAnyThreads = 128;
constexpr int kAnyMinBlocks = 10;  // 40 warps per SM: the loads of a warp are all issued up front
constexpr int kAnySegPad = 32;  // the 0..15-byte offset in front, one spilled word behind

// One segment: lane l contributes SEGW words w (stream bytes [4*SEGW*l, 4*SEGW*(l+1))); the first
// `nbytes` stream bytes go to global address g.  seg: this segment's staging area (16-byte
// aligned, 4*SEGW*32 + kAnySegPad bytes).  Issues at most one bulk copy (not yet committed).
template <int SEGW>
__device__ __forceinline__ void stage_and_copy(unsigned char* seg, const uint32_t* w, uint8_t* g,
                                               int nbytes, int lane) {
  const uint32_t a = (uint32_t)((uintptr_t)g & 15), sh = a & 3;
  unsigned char* base = seg + (a - sh) + lane * (4 * SEGW);  // 4-byte aligned
  if (sh == 0) {
    if (((a - sh) & 15) == 0 && SEGW % 4 == 0) {
#pragma unroll
      for (int i = 0; i < SEGW; i += 4)
        *reinterpret_cast<uint4*>(base + 4 * i) = make_uint4(w[i], w[i + 1], w[i + 2], w[i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < SEGW; ++i) *reinterpret_cast<uint32_t*>(base + 4 * i) = w[i];
    }
  } else {
    // shifted stream: word k holds the top `sh` bytes of stream word k-1 and the low bytes of k
    uint32_t prev = __shfl_up_sync(0xffffffffu, w[SEGW - 1], 1);
#pragma unroll
    for (int i = 0; i < SEGW; ++i) {
      *reinterpret_cast<uint32_t*>(base + 4 * i) = __funnelshift_l(prev, w[i], 8 * sh);
      prev = w[i];
    }
    if (lane == 31) *reinterpret_cast<uint32_t*>(base + 4 * SEGW) = prev >> (32 - 8 * sh);
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncwarp();
  const unsigned char* data = seg + a;  // stream byte j sits at data[j]; data + head is 16-aligned
  int head = (int)((16 - a) & 15);
  if (head > nbytes) head = nbytes;
  const int body = (nbytes - head) & ~15;
  const int tail0 = head + body;
  if (lane < head) g[lane] = data[lane];
  if (tail0 + lane < nbytes) g[tail0 + lane] = data[tail0 + lane];
  if (lane == 0 && body > 0)
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(g + head),
                 "r"(smem_addr(data + head)), "r"((uint32_t)body)
                 : "memory");
}

template <int FMT, int LAYOUT, int DTYPE, bool BGR, bool TABLE, int ARITH>
__global__ void __launch_bounds__(kAnyThreads, kAnyMinBlocks) dense_any_kernel(const DenseParams p) {
  using T = typename OutT<DTYPE>::type;
  constexpr int ESZ = (int)sizeof(T);
  constexpr int PX = 16 / ESZ;
  constexpr int NW = PX / 4;
  constexpr int UVB = FMT == B2_SRC_NV12 ? PX : PX / 2;
  constexpr int UVW = (UVB + 3) / 4;
  constexpr int SEGW = LAYOUT == B2_NHWC ? 12 : 4;  // words a lane adds to a segment
  constexpr int NSEG = LAYOUT == B2_NHWC ? 2 : 6;   // rows, or rows x planes
  constexpr int SEGS = 4 * SEGW * 32 + kAnySegPad;  // bytes reserved per segment
  extern __shared__ __align__(128) unsigned char any_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned char* wsm = any_smem + warp * (NSEG * SEGS);

  // warps are numbered through the frame: warp -> (row pair, block of 32*PX pixels in the row),
  // so that rows narrower than a CTA leave no warp without work
  const int n = blockIdx.z;
  const int we = p.width & ~1;  // a trailing odd column is left untouched
  const int segs = (we + 32 * PX - 1) / (32 * PX);
  const int wid = blockIdx.x * (kAnyThreads / 32) + warp;
  const int rp = wid / segs;
  if (2 * rp >= p.height) return;
  const int wx0 = (wid - rp * segs) * 32 * PX;
  const int x0 = wx0 + lane * PX;

  uint32_t out[2][12];
#pragma unroll
  for (int i = 0; i < 12; ++i) out[0][i] = out[1][i] = 0u;
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
    uint32_t yw[2][NW], uw[UVW], vw[UVW];
    const uint8_t* y0 = yb + (size_t)(2 * rp) * (unsigned)p.y_pitch;
    const size_t uv_off = (size_t)rp * (unsigned)p.uv_pitch;
    if (rp >= 1 && 2 * rp + 4 <= p.height) {
      // Not the first or last row pair: the few bytes an aligned vector reads before or behind
      // a row belong to the neighbouring rows of the same plane, so no bounds are checked.
      load_window_inside<PX>(y0, x0, yw[0]);
      load_window_inside<PX>(y0 + p.y_pitch, x0, yw[1]);
      if constexpr (FMT == B2_SRC_NV12) {
        load_window_inside<UVB>(ub + uv_off, x0, uw);
      } else {
        load_window_inside<UVB>(ub + uv_off, x0 / 2, uw);
        load_window_inside<UVB>(vb + uv_off, x0 / 2, vw);
      }
    } else {
      load_window<PX>(y0, x0, we, yw[0]);
      load_window<PX>(y0 + p.y_pitch, x0, we, yw[1]);
      if constexpr (FMT == B2_SRC_NV12) {
        load_window<UVB>(ub + uv_off, x0, we, uw);
      } else {
        load_window<UVB>(ub + uv_off, x0 / 2, we / 2, uw);
        load_window<UVB>(vb + uv_off, x0 / 2, we / 2, vw);
      }
    }
    (void)vw;
    convert_chunk<FMT, LAYOUT, DTYPE, BGR, ARITH>(p.mat, p.sb, yw, uw, vw, out);
  }

  const int px = we - wx0 < 32 * PX ? we - wx0 : 32 * PX;  // pixels of the warp's block in the row
  uint8_t* dst = reinterpret_cast<uint8_t*>(static_cast<T*>(p.dst) + (long long)n * p.dst_frame_stride);
#pragma unroll
  for (int sidx = 0; sidx < NSEG; ++sidx) {
    if constexpr (LAYOUT == B2_NHWC) {
      const long long row = 2 * rp + sidx;
      stage_and_copy<SEGW>(wsm + sidx * SEGS, &out[sidx][0],
                           dst + (row * p.dst_row_pitch + (long long)wx0 * 3) * ESZ, px * 3 * ESZ,
                           lane);
    } else {
      const int r = sidx / 3, slot = sidx % 3;
      const long long row = 2 * rp + r;
      stage_and_copy<SEGW>(wsm + sidx * SEGS, &out[r][4 * slot],
                           dst + (slot * p.dst_plane_stride + row * p.dst_row_pitch + wx0) * ESZ,
                           px * ESZ, lane);
    }
  }
  if (lane == 0) {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    // the staging buffer must outlive the engine's reads of it
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
  }
}

inline bool mult(long long v, long long m) { return v % m == 0; }
enum { kPathAny = 0, kPathVec = 1, kPathFlat = 2 };

template <int FMT, int LAYOUT, int DTYPE, bool BGR, bool TABLE, int ARITH>
int launch_t(const DenseLaunch& L, const DenseParams& p, int path, cudaStream_t stream) {
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
    if (path == kPathFlat) {
      {
        // chunk 0 may start up to PX - 1 pixels before the frame: one chunk more than the pixels
        const long long chunks = ((long long)p.pixels + PX - 1) / PX + 1;
        const int per_cta = kFlatThreads * kFlatChunks;
        dim3 grid((unsigned)((chunks + per_cta - 1) / per_cta), 1, nn);
        const size_t smem = LAYOUT == B2_NHWC ? (size_t)per_cta * 48 : 0;
        if (p.flat_packed)
          dense_flat_kernel<FMT, LAYOUT, DTYPE, BGR, ARITH, true>
              <<<grid, kFlatThreads, smem, stream>>>(q);
        else
          dense_flat_kernel<FMT, LAYOUT, DTYPE, BGR, ARITH, false>
              <<<grid, kFlatThreads, smem, stream>>>(q);
      }
    } else if (path == kPathVec) {
      const int chunks = (L.width + PX - 1) / PX;
      int bx = ((chunks + 31) / 32) * 32;
      if (bx > kDenseThreads) bx = kDenseThreads;
      const int by = kDenseThreads / bx;
      dim3 block(bx, by), grid((chunks + bx - 1) / bx, (He / 2 + by - 1) / by, nn);
      const size_t smem = LAYOUT == B2_NHWC ? (size_t)(kDenseThreads / 32) * 2 * 32 * 48 : 0;
      dense_vec_kernel<FMT, LAYOUT, DTYPE, BGR, TABLE, ARITH><<<grid, block, smem, stream>>>(q);
    } else {
      if (He < 2) continue;
      constexpr int kSegW = LAYOUT == B2_NHWC ? 12 : 4, kSegN = LAYOUT == B2_NHWC ? 2 : 6;
      const size_t smem = (size_t)(kAnyThreads / 32) * kSegN * (4 * kSegW * 32 + kAnySegPad);
      const long long segs = ((L.width & ~1) + 32 * PX - 1) / (32 * PX);  // warps per row pair
      const long long warps = segs * (He / 2);
      dim3 grid((unsigned)((warps + kAnyThreads / 32 - 1) / (kAnyThreads / 32)), 1, nn);
      dense_any_kernel<FMT, LAYOUT, DTYPE, BGR, TABLE, ARITH><<<grid, kAnyThreads, smem, stream>>>(q);
    }
    B2_CUDA(cudaPeekAtLastError(), "launch of the dense conversion kernel failed");
  }
  return B2_OK;
}

template <int FMT, int LAYOUT, int DTYPE, int ARITH>
int launch_fld(const DenseLaunch& L, const DenseParams& p, int path, cudaStream_t s) {
  const bool bgr = L.order == B2_BGR, table = L.y_table != nullptr;
  if (bgr) return table ? launch_t<FMT, LAYOUT, DTYPE, true, true, ARITH>(L, p, path, s)
                        : launch_t<FMT, LAYOUT, DTYPE, true, false, ARITH>(L, p, path, s);
  return table ? launch_t<FMT, LAYOUT, DTYPE, false, true, ARITH>(L, p, path, s)
               : launch_t<FMT, LAYOUT, DTYPE, false, false, ARITH>(L, p, path, s);
}
template <int FMT, int LAYOUT, int ARITH>
int launch_fla(const DenseLaunch& L, const DenseParams& p, int path, cudaStream_t s) {
  switch (L.dtype) {
    case B2_U8: return launch_fld<FMT, LAYOUT, B2_U8, ARITH>(L, p, path, s);
    case B2_F32: return launch_fld<FMT, LAYOUT, B2_F32, ARITH>(L, p, path, s);
    default: return launch_fld<FMT, LAYOUT, B2_BF16, ARITH>(L, p, path, s);
  }
}
template <int FMT, int LAYOUT>
int launch_fl(const DenseLaunch& L, const DenseParams& p, int path, cudaStream_t s) {
  return L.arith == B2_ARITH_SWSCALE ? launch_fla<FMT, LAYOUT, B2_ARITH_SWSCALE>(L, p, path, s)
                                     : launch_fla<FMT, LAYOUT, B2_ARITH_REFERENCE>(L, p, path, s);
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
  int path = vec ? kPathVec : kPathAny;
  // A packed destination (rows back to back, even width of at least one chunk, every frame on a
  // multiple of two elements, planes a multiple of 16 bytes apart) takes the flat kernel, whatever
  // the pitch and alignment of the source; source rows back to back too select its leaner variant.
  const long long He = L.height & ~1;
  const bool nv12 = L.src_format == B2_SRC_NV12;
  const long long cw = nv12 ? L.width : L.width / 2;  // bytes of a chroma row
  if (!vec && L.width % 2 == 0 && L.width >= px && L.y_pitch >= L.width && L.uv_pitch >= cw &&
      L.y_pitch * He < (1LL << 30) && L.uv_pitch * He < (1LL << 30) &&
      L.dst_row_pitch == (L.layout == B2_NCHW ? L.width : 3LL * L.width) &&
      mult((long long)(uintptr_t)L.dst, 2 * esz) && mult(L.dst_frame_stride, 2) &&
      (L.layout != B2_NCHW || mult(L.dst_plane_stride * esz, 16))) {
    path = kPathFlat;
    p.flat_packed = !table && L.y_pitch == L.width && L.uv_pitch == cw;
    p.pixels = (int)(L.width * He);
    p.y_limit = (int)((He - 1) * L.y_pitch + L.width);
    p.chroma_limit = (int)((He / 2 - 1) * L.uv_pitch + cw);
    p.w_recip = (unsigned)((1ULL << 32) / (unsigned)L.width);
    p.rows_per_warp = (kFlatChunks * 32 * px + L.width - 1) / L.width + 1;
  }
  if (nv12)
    return L.layout == B2_NCHW ? launch_fl<B2_SRC_NV12, B2_NCHW>(L, p, path, stream)
                               : launch_fl<B2_SRC_NV12, B2_NHWC>(L, p, path, stream);
  return L.layout == B2_NCHW ? launch_fl<B2_SRC_I420, B2_NCHW>(L, p, path, stream)
                             : launch_fl<B2_SRC_I420, B2_NHWC>(L, p, path, stream);
}

}  // namespace b2

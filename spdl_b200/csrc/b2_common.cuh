// Shared pieces of the sm_100a frame kernels: error plumbing for the C ABI, the
// colour-matrix table and the per-pixel arithmetic.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "b2frames.h"

namespace b2 {

// ---- host: status + thread-local message ----------------------------------------------------
int fail(int code, const char* fmt, ...);
int fail_cuda(cudaError_t e, const char* what);
void clear_error();

#define B2_CUDA(expr, what)                          \
  do {                                               \
    cudaError_t _e = (expr);                         \
    if (_e != cudaSuccess) return ::b2::fail_cuda(_e, what); \
  } while (0)

// Makes `device` current for the scope and restores the previous one.
class DeviceGuard {
 public:
  explicit DeviceGuard(int device);
  ~DeviceGuard();
  cudaError_t status() const { return status_; }

 private:
  int prev_ = -1;
  bool switched_ = false;
  cudaError_t status_ = cudaSuccess;
};

// ---- colour matrix ----------------------------------------------------------------------------
// Every entry of the reference table (src/libspdl/cuda/detail/color_conversion.cu:20-70) has the
// shape {g,0,vr},{g,ug,vg},{g,ub,0}; five numbers describe it.  y_bias is 2^23 + luma offset:
// the kernels turn a byte b into the float 2^23+b with one byte-permute and subtract y_bias.
struct ColorMat {
  float g, vr, ug, vg, ub;
  float y_bias;
  float neg_zero;  // always -0.0f; a run-time value so that the compiler cannot fold it away
};
// arith = B2_ARITH_SWSCALE fills the same struct with libswscale's 16-bit coefficients divided
// by 2^13 (exact in fp32) and vg unused; see sws_chroma2_of.
ColorMat color_matrix(int matrix_coeff, int full_range, int arith = B2_ARITH_REFERENCE);

struct ScaleBias {
  float s[3], b[3];
};

#ifdef __CUDACC__

constexpr float kTwo23 = 8388608.0f;
constexpr float kQuantMagic = 12582912.0f;  // 1.5 * 2^23: ulp is 1 on both sides of zero offset

// float(2^23 + byte k of w): one PRMT, no integer->float conversion instruction.
__device__ __forceinline__ float biased_byte(uint32_t w, int k) {
  return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540u + k));
}

// The reference evaluates  m0*fy + m1*fu + m2*fv  per channel in fp32
// (color_conversion.cu:76-86); as nvcc compiles it the device computes
//     fma(m0, fy, m1*fu) + m2*fv
// -- the first product pair fused, the last add not.  With the table's zeros this is
//     R = g*fy + vr*fv          G = fma(g, fy, ug*fu) + vg*fv          B = fma(g, fy, ub*fu)
// and the four chroma products are shared by the 2x2 quad that shares the chroma sample.
//
// ---- two pixels per instruction ------------------------------------------------------------------
// sm_100 has packed fp32 instructions (add/fma on two fp32 lanes of a 64-bit register pair), each
// lane IEEE-rounded exactly like the scalar instruction.  The vector kernel pairs pixel k of a
// luma word with pixel k+2: lane x then belongs to the first 2x2 quad under the word, lane y to
// the second, so chroma terms pair up the same way and nothing has to be duplicated.
//
// ptxas contracts a packed multiply with a following packed add into one packed fma even when
// both carry an explicit rounding mode (observed on CUDA 12.9: a mul.rn.f32x2 -> add.rn.f32x2
// chain differs from the scalar chain in 16 % of all 2^24 inputs while each single packed
// instruction is exact).  That would change which products are rounded, so every product that
// feeds an add is written as fma(a, b, nz) with nz = -0.0 read from the kernel parameters: adding
// -0.0 is an exact identity, the compiler cannot know the value, and an fma result cannot be
// contracted into a later add.
__device__ __forceinline__ unsigned long long pack2(float2 v) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(v.x), "f"(v.y));
  return r;
}
__device__ __forceinline__ float2 unpack2(unsigned long long v) {
  float2 r;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(v));
  return r;
}
__device__ __forceinline__ float2 x2_add(float2 a, float2 b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(pack2(a)), "l"(pack2(b)));
  return unpack2(d);
}
__device__ __forceinline__ float2 x2_add_rz(float2 a, float2 b) {
  unsigned long long d;
  asm("add.rz.f32x2 %0, %1, %2;" : "=l"(d) : "l"(pack2(a)), "l"(pack2(b)));
  return unpack2(d);
}
__device__ __forceinline__ float2 x2_fma(float2 a, float2 b, float2 c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(pack2(a)), "l"(pack2(b)), "l"(pack2(c)));
  return unpack2(d);
}
__device__ __forceinline__ float2 dup2(float a) { return make_float2(a, a); }

__device__ __forceinline__ float2 x2_fma_rm(float2 a, float2 b, float2 c) {
  unsigned long long d;
  asm("fma.rm.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(pack2(a)), "l"(pack2(b)), "l"(pack2(c)));
  return unpack2(d);
}

// ---- libswscale's arithmetic -----------------------------------------------------------------
// The x86 SIMD converter libswscale uses for unscaled yuv420p -> rgb24 works on 16-bit lanes:
//     y' = (Y << 3) - yOffset          u' = (U << 3) - 1024          v' = (V << 3) - 1024
//     each product = (x' * coeff) >> 16                   (signed high half: a floor)
//     R = y'' + vr'',   G = y'' + (ug'' + vg''),   B = y'' + ub'',   saturated to 0..255
// with coeff = round(c * 2^13) from its colourspace table.  yOffset is 128 or 0, so every x' is
// 8 * (byte - k) and a product is floor((byte - k) * coeff / 2^13).  (byte - k) * coeff stays
// below 2^23, so fp32 holds it exactly, and ONE fused multiply-add that adds 1.5 * 2^23 and rounds
// toward minus infinity leaves 1.5 * 2^23 + floor(product): no integer instruction is needed.
// ColorMat carries coeff / 2^13 for this arithmetic (exact: a 16-bit integer times 2^-13).
// Chroma2.ug holds ug'' + vg''; Chroma2.vg is unused.
//
// The arithmetic below reads the matrix through a small interface -- g2(), vr2(), ... return a
// coefficient in both lanes -- so that a kernel can either duplicate the scalars where they are
// used (MatDup: fine when a thread converts many pixels in straight-line code) or hold the pairs
// in registers across a loop (MatPairs; pin2 keeps the compiler from rebuilding a pair from the
// kernel parameters at every use, which costs two moves each time).
struct MatDup {
  const ColorMat& m;
  __device__ __forceinline__ float2 g2() const { return dup2(m.g); }
  __device__ __forceinline__ float2 vr2() const { return dup2(m.vr); }
  __device__ __forceinline__ float2 ug2() const { return dup2(m.ug); }
  __device__ __forceinline__ float2 vg2() const { return dup2(m.vg); }
  __device__ __forceinline__ float2 ub2() const { return dup2(m.ub); }
  __device__ __forceinline__ float2 neg_ybias2() const { return dup2(-m.y_bias); }
  __device__ __forceinline__ float2 nz2() const { return dup2(m.neg_zero); }
  __device__ __forceinline__ float2 coff2() const { return dup2(-(kTwo23 + 128.0f)); }
  __device__ __forceinline__ float2 magic2() const { return dup2(kQuantMagic); }
  __device__ __forceinline__ float2 neg_magic2() const { return dup2(-kQuantMagic); }
};
__device__ __forceinline__ float2 pin2(float2 v) {
  unsigned long long r = pack2(v);
  asm volatile("" : "+l"(r));
  return unpack2(r);
}
template <int ARITH>
struct MatPairs {  // only the pairs the arithmetic reads are built (and held)
  float2 g, vr, ug, vg, ub, neg_ybias, coff, magic, extra;  // extra: -0.0 or -1.5 * 2^23
  __device__ __forceinline__ explicit MatPairs(const ColorMat& m)
      : g(pin2(dup2(m.g))), vr(pin2(dup2(m.vr))), ug(pin2(dup2(m.ug))), vg(pin2(dup2(m.vg))),
        ub(pin2(dup2(m.ub))), neg_ybias(pin2(dup2(-m.y_bias))),
        coff(pin2(dup2(-(kTwo23 + 128.0f)))), magic(pin2(dup2(kQuantMagic))),
        extra(pin2(dup2(ARITH == B2_ARITH_REFERENCE ? m.neg_zero : -kQuantMagic))) {}
  __device__ __forceinline__ float2 g2() const { return g; }
  __device__ __forceinline__ float2 vr2() const { return vr; }
  __device__ __forceinline__ float2 ug2() const { return ug; }
  __device__ __forceinline__ float2 vg2() const { return vg; }
  __device__ __forceinline__ float2 ub2() const { return ub; }
  __device__ __forceinline__ float2 neg_ybias2() const { return neg_ybias; }
  __device__ __forceinline__ float2 nz2() const { return extra; }
  __device__ __forceinline__ float2 coff2() const { return coff; }
  __device__ __forceinline__ float2 magic2() const { return magic; }
  __device__ __forceinline__ float2 neg_magic2() const { return extra; }
};

struct Chroma2 {
  float2 vr, ug, vg, ub;  // lane x: first quad, lane y: second quad
};
// bu, bv: {2^23 + U, 2^23 + V} of the two quads
template <int ARITH, class M>
__device__ __forceinline__ Chroma2 chroma2_of(const M& m, float2 bu, float2 bv) {
  const float2 fu = x2_add(bu, m.coff2()), fv = x2_add(bv, m.coff2());
  Chroma2 c;
  if constexpr (ARITH == B2_ARITH_REFERENCE) {
    c.vr = x2_fma(m.vr2(), fv, m.nz2());
    c.ug = x2_fma(m.ug2(), fu, m.nz2());
    c.vg = x2_fma(m.vg2(), fv, m.nz2());
    c.ub = x2_fma(m.ub2(), fu, m.nz2());
  } else {
    // libswscale (see below): floors of the four products; ug carries ug'' + vg''
    c.vr = x2_add(x2_fma_rm(m.vr2(), fv, m.magic2()), m.neg_magic2());
    c.ub = x2_add(x2_fma_rm(m.ub2(), fu, m.magic2()), m.neg_magic2());
    c.ug = x2_add(x2_add(x2_fma_rm(m.ug2(), fu, m.magic2()), m.neg_magic2()),
                  x2_add(x2_fma_rm(m.vg2(), fv, m.magic2()), m.neg_magic2()));
    c.vg = dup2(0.0f);
  }
  return c;
}
template <int ARITH = B2_ARITH_REFERENCE>
__device__ __forceinline__ Chroma2 chroma2_of(const ColorMat& m, float2 bu, float2 bv) {
  return chroma2_of<ARITH>(MatDup{m}, bu, bv);
}

// Two pixels (one per quad): by = {2^23 + Y, 2^23 + Y'}.  Results are the channel values plus
// 1.5*2^23 rounded toward zero, i.e. floor(x) sits in the low 16 mantissa bits as a signed halfword (see clamp2_bits).
template <int ARITH, class M>
__device__ __forceinline__ void pixel2_bits(const M& m, float2 by, const Chroma2& c, float2& r,
                                            float2& g, float2& b) {
  const float2 fy = x2_add(by, m.neg_ybias2());
  if constexpr (ARITH == B2_ARITH_REFERENCE) {
    const float2 ly = x2_fma(m.g2(), fy, m.nz2());
    r = x2_add_rz(x2_add(ly, c.vr), m.magic2());
    g = x2_add_rz(x2_add(x2_fma(m.g2(), fy, c.ug), c.vg), m.magic2());
    b = x2_add_rz(x2_fma(m.g2(), fy, c.ub), m.magic2());
  } else {
    const float2 lm = x2_fma_rm(m.g2(), fy, m.magic2());  // 1.5*2^23 + y''
    r = x2_add(lm, c.vr);  // sums of small integers and the magic constant: exact
    g = x2_add(lm, c.ug);
    b = x2_add(lm, c.ub);
  }
}
template <int ARITH = B2_ARITH_REFERENCE>
__device__ __forceinline__ void pixel2_bits(const ColorMat& m, float2 by, const Chroma2& c,
                                            float2& r, float2& g, float2& b) {
  pixel2_bits<ARITH>(MatDup{m}, by, c, r, g, b);
}
// The same two pixels for 8-bit output.  The last step of each channel is a multiply by 2^-149
// with round-toward-zero: the result is the subnormal whose mantissa is trunc(|x|), so its BIT
// PATTERN, read as a signed integer, is trunc(x) for x >= 0 and a negative number for x < 0
// (sign bit set) -- exactly what a saturating integer pack needs (see pack4_sat).
__device__ __forceinline__ float2 x2_mul_rz(float2 a, float2 b) {
  unsigned long long d;
  asm("mul.rz.f32x2 %0, %1, %2;" : "=l"(d) : "l"(pack2(a)), "l"(pack2(b)));
  return unpack2(d);
}
template <int ARITH = B2_ARITH_REFERENCE>
__device__ __forceinline__ void pixel2_ints(const ColorMat& m, float2 by, const Chroma2& c,
                                            float2& r, float2& g, float2& b);
template <>
__device__ __forceinline__ void pixel2_ints<B2_ARITH_SWSCALE>(const ColorMat& m, float2 by,
                                                              const Chroma2& c, float2& r,
                                                              float2& g, float2& b) {
  const float2 unit = dup2(__uint_as_float(1u));  // 2^-149
  const float2 fy = x2_add(by, dup2(-m.y_bias));
  const float2 ly = x2_add(x2_fma_rm(dup2(m.g), fy, dup2(kQuantMagic)), dup2(-kQuantMagic));
  r = x2_mul_rz(x2_add(ly, c.vr), unit);  // integer-valued floats: the subnormal's bits are the value
  g = x2_mul_rz(x2_add(ly, c.ug), unit);
  b = x2_mul_rz(x2_add(ly, c.ub), unit);
}
template <>
__device__ __forceinline__ void pixel2_ints<B2_ARITH_REFERENCE>(const ColorMat& m, float2 by,
                                                                const Chroma2& c, float2& r,
                                                                float2& g, float2& b) {
  const float2 g2 = dup2(m.g), unit = dup2(__uint_as_float(1u));  // 2^-149
  const float2 fy = x2_add(by, dup2(-m.y_bias));
  const float2 ly = x2_fma(g2, fy, dup2(m.neg_zero));
  r = x2_mul_rz(x2_add(ly, c.vr), unit);
  g = x2_mul_rz(x2_add(x2_fma(g2, fy, c.ug), c.vg), unit);
  b = x2_mul_rz(x2_fma(g2, fy, c.ub), unit);
}
// Truncate-and-clamp (color_conversion.cu:72-74) of four values produced by pixel2_ints and
// pack them as bytes {v0, v1, v2, v3}, v0 lowest: two saturating packs (s32 -> u8: negative -> 0,
// above 255 -> 255).
__device__ __forceinline__ uint32_t pack4_sat(float v0, float v1, float v2, float v3) {
  uint32_t hi, d;
  asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;"
      : "=r"(hi)
      : "r"(__float_as_uint(v3)), "r"(__float_as_uint(v2)), "r"(0u));
  asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;"
      : "=r"(d)
      : "r"(__float_as_uint(v1)), "r"(__float_as_uint(v0)), "r"(hi));
  return d;
}
// Clamp two magic-added values (as produced by pixel2_bits) to 0..255 in two 16-bit lanes.
__device__ __forceinline__ uint32_t clamp2_bits(float a, float b) {
  return __vimin_s16x2_relu(__byte_perm(__float_as_uint(a), __float_as_uint(b), 0x5410u),
                            0x00FF00FFu);
}

template <int DTYPE>
struct OutT;
template <>
struct OutT<B2_U8> { using type = uint8_t; };
template <>
struct OutT<B2_F32> { using type = float; };
template <>
struct OutT<B2_BF16> { using type = __nv_bfloat16; };

#endif  // __CUDACC__

// ---- launchers shared between translation units ------------------------------------------------
struct DenseLaunch {
  const uint8_t* y;
  const uint8_t* u;
  const uint8_t* v;
  const void* const* y_table;
  const void* const* u_table;
  const void* const* v_table;
  int64_t y_pitch, uv_pitch, y_frame_stride, uv_frame_stride;
  int src_format, width, height, num_frames;
  ColorMat mat;
  void* dst;
  int64_t dst_row_pitch;     // elements (NCHW: between rows of a plane; NHWC: between rows)
  int64_t dst_plane_stride;  // elements (NCHW only)
  int64_t dst_frame_stride;  // elements
  int layout, dtype, order;
  ScaleBias sb;
  int arith;  // b2_arith; `mat` must come from color_matrix(..., arith)
};
int launch_dense(const DenseLaunch& L, cudaStream_t stream);

}  // namespace b2

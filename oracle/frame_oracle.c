/*
 * CPU oracle for the post-decode frame path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference's colour
 * conversion and of the fused resize/crop/normalise semantics built on it.
 * Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
 * load it; nothing in the shipped package calls into it.
 *
 * Reference lines each function follows (paths within facebookresearch/spdl):
 *   orc_matrix           src/libspdl/cuda/detail/color_conversion.cu:20-70
 *                        (table, index = matrix_coefficients-1, out-of-range -> 1
 *                        at :120-123)
 *   orc_clamp8           src/libspdl/cuda/detail/color_conversion.cu:72-74
 *   orc_pixel            src/libspdl/cuda/detail/color_conversion.cu:76-86
 *   orc_convert_dense    src/libspdl/cuda/detail/color_conversion.cu:98-137
 *                        (2x2 quad, chroma at (x&~1, y/2), odd tail untouched)
 *                        and src/libspdl/cuda/color_conversion.cpp:34-54 (shapes)
 *   orc_gather_frames    src/libspdl/cuda/nvdec/detail/buffer.cpp:31-74
 *                        (pitched surface -> packed [N, H*3/2, W] slot)
 *   orc_sws_coeffs /     the reference's CPU route: "format=pix_fmts=rgb24"
 *   orc_sws_pixel        (src/spdl/io/_preprocessing.py:250-251) run by the filter graph of
 *                        src/libspdl/core/detail/ffmpeg/filter_graph.cpp:50-65,154-173, i.e. by
 *                        FFmpeg's libswscale.  libswscale is a third-party dependency whose
 *                        source is NOT under the reference tree (the reference loads FFmpeg 4-8
 *                        at run time); the arithmetic restated here is that of its unscaled
 *                        yuv420p -> rgb24 converter on x86 (libswscale/x86/yuv_2_rgb.asm, 16-bit
 *                        lanes) with the constants of ff_yuv2rgb_c_init_tables
 *                        (libswscale/yuv2rgb.c) and the colourspace table behind
 *                        sws_getCoefficients.  Pinned against libswscale 9.1.100 (FFmpeg 8) as
 *                        bundled with the opencv wheel: identical over all 2^24 (Y,U,V) for
 *                        BT.709 and BT.601, limited and full range (tests/golden/sws_golden.json,
 *                        tests/test_swscale_oracle.py).
 *
 * Parity status.  The limited-range planar u8 conversion is pinned by the three
 * known-answer triplets of tests/cuda/nvdec_video_decoding_test.py:335-348 and
 * by fixtures produced by running the reference's own kernel source (compiled
 * unmodified) on a GPU.  Everything the reference does not implement --
 * interleaved output, float/bf16 output with scale and bias, full-range
 * matrices, planar-chroma (I420) input, bilinear resize and crop -- is defined
 * here and is "parity unpinned": this file is the definition.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#define ORC_EXPORT __attribute__((visibility("default")))

/* ORC_RGBP / ORC_RGBI: already-decoded RGB (planar / interleaved), as a JPEG decoder emits
 * it (src/libspdl/cuda/nvjpeg/decoding.cpp:56-95); only the resize path takes them. */
enum { ORC_NV12 = 0, ORC_I420 = 1, ORC_RGBP = 2, ORC_RGBI = 3 };
enum { ORC_NCHW = 0, ORC_NHWC = 1 };
enum { ORC_U8 = 0, ORC_F32 = 1, ORC_BF16 = 2 };
enum { ORC_RGB = 0, ORC_BGR = 1 };
/* Which arithmetic converts a pixel: the reference's CUDA kernel (fp32, default) or the integer
 * arithmetic of libswscale, the reference's CPU route. */
enum { ORC_ARITH_REFERENCE = 0, ORC_ARITH_SWSCALE = 1 };
/* How the three products of one output channel are combined in fp32.
 * The reference source writes  m0*fy + m1*fu + m2*fv ; nvcc fuses multiplies
 * and adds by default, so the device result depends on which products are
 * fused.  ORC_FMA_DEVICE is what the reference kernel, compiled by nvcc 12.9 for
 * sm_100a, computes -- established by comparing all 2^24 inputs on a B200 (see
 * tests/golden).  The others are candidates kept for identification. */
enum {
  ORC_FMA_NONE = 0,         /* (m0*fy + m1*fu) + m2*fv, every operation rounded   */
  ORC_FMA_LUMA_FIRST = 1,   /* fma(m2,fv, fma(m1,fu, m0*fy))                       */
  ORC_FMA_CHROMA_FIRST = 2, /* fma(m2,fv, fma(m0,fy, m1*fu))                       */
  ORC_FMA_DEVICE = 4        /* fma(m0,fy, m1*fu) + m2*fv                           */
};

/* Distinct numbers of the reference table.  Every matrix has the shape
 *   { g, 0, vr }, { g, ug, vg }, { g, ub, 0 }
 * so five numbers describe one entry. */
typedef struct { float g, vr, ug, vg, ub; } orc_coeffs;

static const orc_coeffs k_limited[10] = {
    /* 1 BT709        */ {1.1644f, 1.8337f, -0.2181f, -0.5451f, 2.1606f},
    /* 2 unspecified  */ {1.1644f, 1.8337f, -0.2181f, -0.5451f, 2.1606f},
    /* 3 reserved     */ {1.1644f, 1.8337f, -0.2181f, -0.5451f, 2.1606f},
    /* 4 FCC          */ {1.1644f, 1.6301f, -0.3864f, -0.8289f, 2.0726f},
    /* 5 BT470        */ {1.1644f, 1.6325f, -0.4007f, -0.8315f, 2.0633f},
    /* 6 BT601        */ {1.1644f, 1.6325f, -0.4007f, -0.8315f, 2.0633f},
    /* 7 SMPTE240M    */ {1.1644f, 1.8351f, -0.2639f, -0.5550f, 2.1262f},
    /* 8 "YCgCo"      */ {1.1644f, 1.8337f, -0.2181f, -0.5451f, 2.1606f},
    /* 9 BT2020       */ {1.1689f, 1.7237f, -0.1924f, -0.6679f, 2.1992f},
    /* 10 BT2020C     */ {1.1689f, 1.7237f, -0.1924f, -0.6679f, 2.1992f},
};

/* Full-range (JFIF-style) matrices: not in the reference.  Derived from the
 * luma weights (Kr, Kb) of each standard:  vr = 2(1-Kr), ub = 2(1-Kb),
 * ug = -2Kb(1-Kb)/Kg, vg = -2Kr(1-Kr)/Kg, rounded to six decimals; unit luma
 * gain and no luma offset. */
static const orc_coeffs k_full[10] = {
    /* 1 BT709   Kr .2126 Kb .0722 */ {1.0f, 1.574800f, -0.187324f, -0.468124f, 1.855600f},
    /* 2 */ {1.0f, 1.574800f, -0.187324f, -0.468124f, 1.855600f},
    /* 3 */ {1.0f, 1.574800f, -0.187324f, -0.468124f, 1.855600f},
    /* 4 FCC     Kr .30   Kb .11   */ {1.0f, 1.400000f, -0.331864f, -0.711864f, 1.780000f},
    /* 5 BT470BG Kr .299  Kb .114  */ {1.0f, 1.402000f, -0.344136f, -0.714136f, 1.772000f},
    /* 6 BT601   Kr .299  Kb .114  */ {1.0f, 1.402000f, -0.344136f, -0.714136f, 1.772000f},
    /* 7 240M    Kr .212  Kb .087  */ {1.0f, 1.576000f, -0.226622f, -0.476622f, 1.826000f},
    /* 8 */ {1.0f, 1.574800f, -0.187324f, -0.468124f, 1.855600f},
    /* 9 BT2020  Kr .2627 Kb .0593 */ {1.0f, 1.474600f, -0.164553f, -0.571353f, 1.881400f},
    /* 10 */ {1.0f, 1.474600f, -0.164553f, -0.571353f, 1.881400f},
};

/* m: 9 floats row-major (R row, G row, B row); *y_off: luma offset (16 or 0). */
ORC_EXPORT void orc_matrix(int coeff, int full_range, float* m, int* y_off) {
  if (coeff <= 0 || coeff > 10) coeff = 1;
  const orc_coeffs* c = full_range ? &k_full[coeff - 1] : &k_limited[coeff - 1];
  m[0] = c->g; m[1] = 0.0f;  m[2] = c->vr;
  m[3] = c->g; m[4] = c->ug; m[5] = c->vg;
  m[6] = c->g; m[7] = c->ub; m[8] = 0.0f;
  *y_off = full_range ? 0 : 16;
}

static inline uint8_t orc_clamp8(float x) {
  return x < 0.0f ? 0 : (x > 255.0f ? 255 : (uint8_t)x);
}

/* Fused multiply-add with a single rounding.  The generic build calls libm's
 * fmaf (exact by contract); the clone compiled for FMA hardware inlines it. */
#define ORC_FMA(a, b, c) __builtin_fmaf((a), (b), (c))

static inline float orc_channel(const float* r, float fy, float fu, float fv, int mode) {
  /* The translation unit is compiled with -ffp-contract=off, so the compiler never fuses on its
   * own: every fusion below is explicit.  a*b = luma product, c*d = U product, e*f = V product. */
  const float a = r[0], b = fy, c = r[1], d = fu, e = r[2], f = fv;
  switch (mode) {
    case ORC_FMA_LUMA_FIRST:   return ORC_FMA(e, f, ORC_FMA(c, d, a * b));
    case ORC_FMA_CHROMA_FIRST: return ORC_FMA(e, f, ORC_FMA(a, b, c * d));
    /* further candidates, kept so the fusion order of a new compiler can be identified */
    case 3: { float t = a * b; float s = c * d; return ORC_FMA(e, f, t + s); }
    case ORC_FMA_DEVICE: { float t = ORC_FMA(a, b, c * d); float s = e * f; return t + s; }
    case 5: { float t = ORC_FMA(c, d, a * b); float s = e * f; return t + s; }
    case 6: return ORC_FMA(a, b, ORC_FMA(c, d, e * f));
    case 7: return ORC_FMA(c, d, ORC_FMA(a, b, e * f));
    case 8: return ORC_FMA(a, b, ORC_FMA(e, f, c * d));
    case 9: return ORC_FMA(c, d, ORC_FMA(e, f, a * b));
    default: break;
  }
  float t = a * b;
  float s = c * d;
  t = t + s;
  s = e * f;
  return t + s;
}

static inline void orc_pixel_impl(int y, int u, int v, const float* m, int y_off, int mode,
                                  uint8_t* rgb) {
  float fy = (float)(y - y_off), fu = (float)(u - 128), fv = (float)(v - 128);
  rgb[0] = orc_clamp8(orc_channel(m + 0, fy, fu, fv, mode));
  rgb[1] = orc_clamp8(orc_channel(m + 3, fy, fu, fv, mode));
  rgb[2] = orc_clamp8(orc_channel(m + 6, fy, fu, fv, mode));
}

ORC_EXPORT void orc_pixel(int y, int u, int v, int coeff, int full_range, int mode, uint8_t* rgb) {
  float m[9]; int y_off;
  orc_matrix(coeff, full_range, m, &y_off);
  orc_pixel_impl(y, u, v, m, y_off, mode, rgb);
}

/* The same conversion with exact integer arithmetic: the limited-range table has
 * four decimals, so coefficients x 10^4 are integers and
 *   c = floor((m0*fy + m1*fu + m2*fv) / 10^4)   (negative sums clamp to 0)
 * has no rounding at all.  Used to bound how far fp32 evaluation can be from the
 * mathematically exact value (never more than 1). */
ORC_EXPORT void orc_pixel_exact(int y, int u, int v, int coeff, uint8_t* rgb) {
  float m[9]; int y_off;
  orc_matrix(coeff, 0, m, &y_off);
  int fy = y - y_off, fu = u - 128, fv = v - 128;
  for (int r = 0; r < 3; ++r) {
    int64_t acc = 0;
    acc += (int64_t)lrint((double)m[3 * r + 0] * 10000.0) * fy;
    acc += (int64_t)lrint((double)m[3 * r + 1] * 10000.0) * fu;
    acc += (int64_t)lrint((double)m[3 * r + 2] * 10000.0) * fv;
    int64_t q = acc < 0 ? 0 : acc / 10000;
    rgb[r] = (uint8_t)(q > 255 ? 255 : q);
  }
}

/* ---- libswscale's integer arithmetic ----------------------------------------------------- */

/* The table behind sws_getCoefficients(): 16.16 fixed point {V->R, U->B, -(U->G), -(V->G)},
 * indexed by SWS_CS_*; 8 and out-of-range numbers select the BT.601 row, as that function does. */
static const int k_sws_table[11][4] = {
    {104597, 132201, 25675, 53279}, {117489, 138438, 13975, 34925},
    {104597, 132201, 25675, 53279}, {104597, 132201, 25675, 53279},
    {104448, 132798, 24759, 53109}, {104597, 132201, 25675, 53279},
    {104597, 132201, 25675, 53279}, {117579, 136230, 16907, 35559},
    {104597, 132201, 25675, 53279}, {110013, 140363, 12277, 42626},
    {110013, 140363, 12277, 42626},
};

typedef struct { int yc, vr, ug, vg, ub, yo; } orc_sws;

static inline int orc_round16(int64_t f) {  /* roundToInt16 of yuv2rgb.c */
  int64_t r = (f + (1 << 15)) >> 16;
  return (int)(r < -0x8000 ? -0x8000 : (r > 0x7FFF ? 0x7FFF : r));
}

/* 16-bit SIMD constants for colourspace `cs`, default brightness/contrast/saturation.
 * out: {yCoeff, vrCoeff, ugCoeff, vgCoeff, ubCoeff, yOffset}. */
ORC_EXPORT void orc_sws_coeffs(int cs, int full_range, int* out) {
  if (cs < 0 || cs > 10) cs = 5;
  int64_t crv = k_sws_table[cs][0], cbu = k_sws_table[cs][1];
  int64_t cgu = -k_sws_table[cs][2], cgv = -k_sws_table[cs][3];
  int64_t cy = 1 << 16, oy = 0;
  if (!full_range) {
    cy = (cy * 255) / 219;
    oy = 16 << 16;
  } else {
    crv = (crv * 224) / 255;
    cbu = (cbu * 224) / 255;
    cgu = (cgu * 224) / 255;
    cgv = (cgv * 224) / 255;
  }
  out[0] = orc_round16(cy * 8192);
  out[1] = orc_round16(crv * 8192);
  out[2] = orc_round16(cgu * 8192);
  out[3] = orc_round16(cgv * 8192);
  out[4] = orc_round16(cbu * 8192);
  out[5] = orc_round16(oy * 8);
}

static inline int orc_sat16(int v) { return v < -32768 ? -32768 : (v > 32767 ? 32767 : v); }
static inline uint8_t orc_satu8(int v) { return (uint8_t)(v < 0 ? 0 : (v > 255 ? 255 : v)); }

/* One pixel as the 16-bit lanes compute it: x' = (byte << 3) - offset, products keep the high
 * 16 bits of the signed 32-bit product, sums saturate to 16 bits, the pack saturates to 8. */
static inline void orc_sws_pixel_impl(int y, int u, int v, const orc_sws* k, uint8_t* rgb) {
  const int ys = (int16_t)((y << 3) - k->yo), us = (int16_t)((u << 3) - 1024),
            vs = (int16_t)((v << 3) - 1024);
  const int ym = (ys * k->yc) >> 16;
  const int ub = (us * k->ub) >> 16, ug = (us * k->ug) >> 16;
  const int vr = (vs * k->vr) >> 16, vg = (vs * k->vg) >> 16;
  rgb[0] = orc_satu8(orc_sat16(ym + vr));
  rgb[1] = orc_satu8(orc_sat16(ym + orc_sat16(ug + vg)));
  rgb[2] = orc_satu8(orc_sat16(ym + ub));
}

static inline orc_sws orc_sws_of(int cs, int full_range) {
  int c[6];
  orc_sws_coeffs(cs, full_range, c);
  orc_sws k = {c[0], c[1], c[2], c[3], c[4], c[5]};
  return k;
}

ORC_EXPORT void orc_sws_pixel(int y, int u, int v, int cs, int full_range, uint8_t* rgb) {
  const orc_sws k = orc_sws_of(cs, full_range);
  orc_sws_pixel_impl(y, u, v, &k, rgb);
}

/* The pixel converter both batch functions call. */
typedef struct { float m[9]; int y_off, fma_mode, arith; orc_sws sws; } orc_conv;
static inline orc_conv orc_conv_of(int coeff, int full_range, int fma_mode, int arith) {
  orc_conv c;
  orc_matrix(coeff, full_range, c.m, &c.y_off);
  c.fma_mode = fma_mode;
  c.arith = arith;
  c.sws = orc_sws_of(coeff, full_range);
  return c;
}
static inline void orc_convert_pixel(const orc_conv* c, int y, int u, int v, uint8_t* rgb) {
  if (c->arith == ORC_ARITH_SWSCALE) orc_sws_pixel_impl(y, u, v, &c->sws, rgb);
  else orc_pixel_impl(y, u, v, c->m, c->y_off, c->fma_mode, rgb);
}

static inline uint16_t orc_f32_to_bf16(float f) {
  uint32_t b; memcpy(&b, &f, 4);
  if ((b & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((b >> 16) | 0x40);
  b += 0x7fffu + ((b >> 16) & 1u);  /* round to nearest even */
  return (uint16_t)(b >> 16);
}

static inline void orc_store(void* dst, size_t idx, int dtype, float val_u8_or_f, const float* sb,
                             int slot) {
  /* val is an integer 0..255 for the dense path, or the interpolated value for
   * the resize path (already rounded by the caller when dtype is u8). */
  if (dtype == ORC_U8) {
    ((uint8_t*)dst)[idx] = (uint8_t)val_u8_or_f;
  } else {
    float o = ORC_FMA(val_u8_or_f, sb[slot], sb[3 + slot]);
    if (dtype == ORC_F32) ((float*)dst)[idx] = o;
    else ((uint16_t*)dst)[idx] = orc_f32_to_bf16(o);
  }
}

typedef struct {
  const uint8_t* y;       /* luma plane of frame 0                                   */
  const uint8_t* u;       /* NV12: interleaved UV plane; I420: U plane               */
  const uint8_t* v;       /* I420 only                                               */
  int64_t y_pitch, uv_pitch;
  int64_t y_frame_stride, uv_frame_stride;
  int32_t src_format, width, height, num_frames;
  int32_t coeff, full_range, fma_mode;
  void* dst;
  int64_t dst_frame_stride;   /* in elements; 0 = packed (3*H*W)                     */
  int32_t layout, dtype, order;
  float scale_bias[6];        /* scale[3], bias[3] per OUTPUT channel slot            */
  int32_t arith;              /* ORC_ARITH_*                                          */
} orc_dense_args;

#define ORC_DENSE_BODY                                                                          \
  const orc_conv cv = orc_conv_of(a->coeff, a->full_range, a->fma_mode, a->arith);              \
  const int W = a->width, H = a->height;                                                        \
  const int We = W & ~1, He = H & ~1;                                                           \
  const int64_t fstride = a->dst_frame_stride ? a->dst_frame_stride : (int64_t)3 * H * W;       \
  const size_t esz = a->dtype == ORC_U8 ? 1 : (a->dtype == ORC_F32 ? 4 : 2);                    \
  _Pragma("omp parallel for collapse(2) schedule(static)")                                      \
  for (int n = 0; n < a->num_frames; ++n) {                                                     \
    for (int y = 0; y < He; ++y) {                                                              \
      const uint8_t* yrow = a->y + n * a->y_frame_stride + (int64_t)y * a->y_pitch;             \
      const uint8_t* urow = a->u + n * a->uv_frame_stride + (int64_t)(y / 2) * a->uv_pitch;     \
      const uint8_t* vrow = a->src_format == ORC_I420                                           \
                                ? a->v + n * a->uv_frame_stride + (int64_t)(y / 2) * a->uv_pitch \
                                : NULL;                                                         \
      char* dbase = (char*)a->dst + (size_t)n * fstride * esz;                                  \
      for (int x = 0; x < We; ++x) {                                                            \
        int cu, cv_;                                                                            \
        if (a->src_format == ORC_I420) { cu = urow[x >> 1]; cv_ = vrow[x >> 1]; }               \
        else { cu = urow[x & ~1]; cv_ = urow[(x & ~1) + 1]; }                                   \
        uint8_t rgb[3];                                                                         \
        orc_convert_pixel(&cv, yrow[x], cu, cv_, rgb);                                          \
        for (int s = 0; s < 3; ++s) {                                                           \
          int ch = a->order == ORC_BGR ? 2 - s : s;                                             \
          size_t idx = a->layout == ORC_NCHW ? ((size_t)s * H + y) * W + x                      \
                                             : ((size_t)y * W + x) * 3 + s;                     \
          orc_store(dbase, idx, a->dtype, (float)rgb[ch], a->scale_bias, s);                    \
        }                                                                                       \
      }                                                                                         \
    }                                                                                           \
  }

__attribute__((target("fma,avx2"))) static void orc_convert_dense_fma(const orc_dense_args* a) {
  ORC_DENSE_BODY
}
static void orc_convert_dense_generic(const orc_dense_args* a) {
  ORC_DENSE_BODY
}

/* Dense conversion of a batch: every even-aligned pixel of every frame.  With
 * (NV12, NCHW, U8, RGB/BGR, limited range) this is exactly the reference kernel. */
ORC_EXPORT void orc_convert_dense(const orc_dense_args* a) {
  if (__builtin_cpu_supports("fma") && __builtin_cpu_supports("avx2")) orc_convert_dense_fma(a);
  else orc_convert_dense_generic(a);
}

/* ---- fused convert -> bilinear resize -> crop -> (normalise) ------------------------------ */

typedef struct {
  uint64_t y_off, u_off, v_off; /* byte offsets from the base pointer                 */
  int32_t y_pitch, uv_pitch;
  int32_t src_w, src_h;
  int32_t crop_x, crop_y;       /* position of output (0,0) in the resized grid        */
  float scale_x, scale_y;       /* source size / resized size, computed in fp32        */
  int32_t resized_w, resized_h; /* size of the resized grid (0 = unbounded): output pixels
                                 * outside it take the pad colour (letterbox)          */
} orc_image_desc;               /* 64 bytes, same layout as the C-ABI descriptor       */

typedef struct {
  const uint8_t* base;
  const orc_image_desc* descs;
  int32_t num_images, src_format;
  int32_t out_w, out_h;
  int32_t coeff, full_range, fma_mode;
  int32_t layout, dtype, order;
  void* dst;
  int64_t dst_image_stride;     /* elements; 0 = packed 3*out_h*out_w                  */
  float scale_bias[6];
  int32_t arith;                /* ORC_ARITH_*                                         */
  int32_t frames_per_group;     /* T > 1: image i starts at (i / T) * group + (i % T) * image */
  int64_t dst_plane_stride;     /* NCHW: elements between colour planes; 0 = out_h*out_w */
  int64_t dst_group_stride;
  float pad_value[3];           /* R, G, B (0..255) of pixels outside the resized grid  */
} orc_resize_args;

static inline void orc_axis(float scale, int g, int n_in, int* i0, int* i1, float* w1) {
  /* bilinear, half-pixel centres, no antialias (align_corners=False) */
  float s = ORC_FMA(scale, (float)g + 0.5f, -0.5f);
  if (s < 0.0f) s = 0.0f;
  int a = (int)s;
  if (a > n_in - 1) a = n_in - 1;
  *i0 = a;
  *i1 = a + 1 < n_in ? a + 1 : n_in - 1;
  *w1 = s - (float)a;
}

/* An image whose descriptor makes no sense (empty source, non-positive or non-finite scale) is
 * left untouched, like the kernel does (it reports a status bit instead). */
#define ORC_RESIZE_BODY                                                                         \
  const orc_conv cv = orc_conv_of(a->coeff, a->full_range, a->fma_mode, a->arith);              \
  const int OW = a->out_w, OH = a->out_h;                                                       \
  const int64_t istride = a->dst_image_stride ? a->dst_image_stride : (int64_t)3 * OH * OW;     \
  const int64_t pstride = a->dst_plane_stride ? a->dst_plane_stride : (int64_t)OH * OW;         \
  const size_t esz = a->dtype == ORC_U8 ? 1 : (a->dtype == ORC_F32 ? 4 : 2);                    \
  _Pragma("omp parallel for collapse(2) schedule(dynamic, 8)")                                  \
  for (int n = 0; n < a->num_images; ++n) {                                                     \
    for (int oy = 0; oy < OH; ++oy) {                                                           \
      const orc_image_desc* d = &a->descs[n];                                                   \
      if (d->src_w < 1 || d->src_h < 1 || !(d->scale_x > 0.0f) || !(d->scale_y > 0.0f)) continue; \
      int64_t ioff = (int64_t)n * istride;                                                      \
      if (a->frames_per_group > 1)                                                              \
        ioff = (int64_t)(n / a->frames_per_group) * a->dst_group_stride +                       \
               (int64_t)(n % a->frames_per_group) * istride;                                    \
      char* dbase = (char*)a->dst + (size_t)ioff * esz;                                         \
      const int gy = d->crop_y + oy;                                                            \
      const int row_out = d->resized_h > 0 && (gy < 0 || gy >= d->resized_h);                   \
      int ys[2]; float wy1;                                                                     \
      orc_axis(d->scale_y, gy, d->src_h, &ys[0], &ys[1], &wy1);                                 \
      float wy0 = 1.0f - wy1;                                                                   \
      for (int ox = 0; ox < OW; ++ox) {                                                         \
        const int gx = d->crop_x + ox;                                                          \
        const int outside = row_out || (d->resized_w > 0 && (gx < 0 || gx >= d->resized_w));    \
        int xs[2]; float wx1;                                                                   \
        orc_axis(d->scale_x, gx, d->src_w, &xs[0], &xs[1], &wx1);                               \
        float wx0 = 1.0f - wx1;                                                                 \
        uint8_t tap[2][2][3];                                                                   \
        for (int j = 0; j < 2 && !outside; ++j)                                                 \
          for (int i = 0; i < 2; ++i) {                                                         \
            int sx = xs[i], sy = ys[j];                                                         \
            if (a->src_format == ORC_RGBP) {                                                    \
              tap[j][i][0] = a->base[d->y_off + (uint64_t)sy * d->y_pitch + sx];                \
              tap[j][i][1] = a->base[d->u_off + (uint64_t)sy * d->uv_pitch + sx];               \
              tap[j][i][2] = a->base[d->v_off + (uint64_t)sy * d->uv_pitch + sx];               \
              continue;                                                                         \
            }                                                                                   \
            if (a->src_format == ORC_RGBI) {                                                    \
              const uint8_t* q = a->base + d->y_off + (uint64_t)sy * d->y_pitch + 3 * sx;       \
              tap[j][i][0] = q[0]; tap[j][i][1] = q[1]; tap[j][i][2] = q[2];                    \
              continue;                                                                         \
            }                                                                                   \
            int Y = a->base[d->y_off + (uint64_t)sy * d->y_pitch + sx];                         \
            int cu, cv_;                                                                        \
            if (a->src_format == ORC_I420) {                                                    \
              cu = a->base[d->u_off + (uint64_t)(sy >> 1) * d->uv_pitch + (sx >> 1)];           \
              cv_ = a->base[d->v_off + (uint64_t)(sy >> 1) * d->uv_pitch + (sx >> 1)];          \
            } else {                                                                            \
              const uint8_t* p = a->base + d->u_off + (uint64_t)(sy >> 1) * d->uv_pitch + (sx & ~1); \
              cu = p[0]; cv_ = p[1];                                                            \
            }                                                                                   \
            orc_convert_pixel(&cv, Y, cu, cv_, tap[j][i]);                                      \
          }                                                                                     \
        for (int s = 0; s < 3; ++s) {                                                           \
          int ch = a->order == ORC_BGR ? 2 - s : s;                                             \
          float val;                                                                            \
          if (outside) {                                                                        \
            val = a->pad_value[ch];                                                             \
          } else {                                                                              \
            float top = ORC_FMA(wx1, (float)tap[0][1][ch], wx0 * (float)tap[0][0][ch]);         \
            float bot = ORC_FMA(wx1, (float)tap[1][1][ch], wx0 * (float)tap[1][0][ch]);         \
            val = ORC_FMA(wy1, bot, wy0 * top);                                                 \
          }                                                                                     \
          if (a->dtype == ORC_U8) {                                                             \
            float q = floorf(val + 0.5f);                                                       \
            val = q < 0.0f ? 0.0f : (q > 255.0f ? 255.0f : q);                                  \
          }                                                                                     \
          size_t idx = a->layout == ORC_NCHW ? (size_t)s * pstride + (size_t)oy * OW + ox       \
                                             : ((size_t)oy * OW + ox) * 3 + s;                  \
          orc_store(dbase, idx, a->dtype, val, a->scale_bias, s);                               \
        }                                                                                       \
      }                                                                                         \
    }                                                                                           \
  }

__attribute__((target("fma,avx2"))) static void orc_convert_resize_fma(const orc_resize_args* a) {
  ORC_RESIZE_BODY
}
static void orc_convert_resize_generic(const orc_resize_args* a) {
  ORC_RESIZE_BODY
}

ORC_EXPORT void orc_convert_resize(const orc_resize_args* a) {
  if (__builtin_cpu_supports("fma") && __builtin_cpu_supports("avx2")) orc_convert_resize_fma(a);
  else orc_convert_resize_generic(a);
}

/* Exhaustive table: for every (y,u,v) in 0..255^3 write the three converted bytes
 * (order y-major, then u, then v; 3 bytes each).  50,331,648 bytes. */
ORC_EXPORT void orc_exhaustive(int coeff, int full_range, int mode, uint8_t* out) {
  float m[9]; int y_off;
  orc_matrix(coeff, full_range, m, &y_off);
#pragma omp parallel for schedule(static)
  for (int y = 0; y < 256; ++y)
    for (int u = 0; u < 256; ++u)
      for (int v = 0; v < 256; ++v)
        orc_pixel_impl(y, u, v, m, y_off, mode, out + 3 * (((size_t)y * 256 + u) * 256 + v));
}

/* The same table for libswscale's arithmetic (colourspace number `cs`). */
ORC_EXPORT void orc_sws_exhaustive(int cs, int full_range, uint8_t* out) {
  const orc_sws k = orc_sws_of(cs, full_range);
#pragma omp parallel for schedule(static)
  for (int y = 0; y < 256; ++y)
    for (int u = 0; u < 256; ++u)
      for (int v = 0; v < 256; ++v)
        orc_sws_pixel_impl(y, u, v, &k, out + 3 * (((size_t)y * 256 + u) * 256 + v));
}

/* Pitched decoder surfaces (one pointer each) -> packed [N, H*3/2, W] batch. */
ORC_EXPORT void orc_gather_frames(const uint8_t* const* surfaces, const int64_t* pitches, int n,
                                  int width, int height, uint8_t* dst) {
  const int h2 = height + height / 2;
  for (int i = 0; i < n; ++i)
    for (int r = 0; r < h2; ++r)
      memcpy(dst + ((size_t)i * h2 + r) * width, surfaces[i] + (size_t)r * pitches[i], width);
}

/* Order-sensitive 64-bit checksum of a byte range: sum of (byte+1) * (1 + (i mod 65521)). */
ORC_EXPORT uint64_t orc_checksum(const uint8_t* p, size_t n) {
  uint64_t s = 0;
  for (size_t i = 0; i < n; ++i) s += (uint64_t)(p[i] + 1u) * (uint64_t)(1u + (i % 65521u));
  return s;
}

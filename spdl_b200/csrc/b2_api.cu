// extern "C" surface of libb2frames.so: argument validation, device selection, error messages.
#include <cmath>
#include <cstdarg>
#include <cstddef>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <thread>
#if defined(__x86_64__)
#include <emmintrin.h>
#endif
#include <vector>

#include "b2_common.cuh"

namespace b2 {

int launch_resize(const b2_resize_args& a, cudaStream_t stream);
int launch_gather(const void* const* surfaces, const int64_t* pitches, int num_frames, int width,
                  int height, uint8_t* dst, cudaStream_t stream);
int launch_checksum(const uint8_t* src, int64_t frame_bytes, int num_frames, uint64_t* out,
                    cudaStream_t stream);

namespace {
thread_local char g_err[512] = "";
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
int fail_cuda(cudaError_t e, const char* what) {
  snprintf(g_err, sizeof(g_err), "%s (%s: %s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
  return B2_ERR_CUDA;
}
void clear_error() { g_err[0] = 0; }

DeviceGuard::DeviceGuard(int device) {
  status_ = cudaGetDevice(&prev_);
  if (status_ == cudaSuccess && prev_ != device) {
    status_ = cudaSetDevice(device);
    switched_ = status_ == cudaSuccess;
  }
}
DeviceGuard::~DeviceGuard() {
  if (switched_) cudaSetDevice(prev_);
}

// The reference table (src/libspdl/cuda/detail/color_conversion.cu:20-70), one row of five
// numbers per matrix_coefficients value 1..10: luma gain, V->R, U->G, V->G, U->B.
static const float kLimited[10][5] = {
    {1.1644f, 1.8337f, -0.2181f, -0.5451f, 2.1606f},  // 1 BT.709
    {1.1644f, 1.8337f, -0.2181f, -0.5451f, 2.1606f},  // 2 unspecified
    {1.1644f, 1.8337f, -0.2181f, -0.5451f, 2.1606f},  // 3 reserved
    {1.1644f, 1.6301f, -0.3864f, -0.8289f, 2.0726f},  // 4 FCC
    {1.1644f, 1.6325f, -0.4007f, -0.8315f, 2.0633f},  // 5 BT.470
    {1.1644f, 1.6325f, -0.4007f, -0.8315f, 2.0633f},  // 6 BT.601
    {1.1644f, 1.8351f, -0.2639f, -0.5550f, 2.1262f},  // 7 SMPTE 240M
    {1.1644f, 1.8337f, -0.2181f, -0.5451f, 2.1606f},  // 8 "YCgCo" (BT.709 numbers)
    {1.1689f, 1.7237f, -0.1924f, -0.6679f, 2.1992f},  // 9 BT.2020
    {1.1689f, 1.7237f, -0.1924f, -0.6679f, 2.1992f},  // 10 BT.2020 constant luminance
};
// Full-range companions (not in the reference): unit luma gain, no luma offset, chroma gains
// 2(1-Kr), -2Kb(1-Kb)/Kg, -2Kr(1-Kr)/Kg, 2(1-Kb) of each standard, six decimals.
static const float kFull[10][5] = {
    {1.0f, 1.574800f, -0.187324f, -0.468124f, 1.855600f},
    {1.0f, 1.574800f, -0.187324f, -0.468124f, 1.855600f},
    {1.0f, 1.574800f, -0.187324f, -0.468124f, 1.855600f},
    {1.0f, 1.400000f, -0.331864f, -0.711864f, 1.780000f},
    {1.0f, 1.402000f, -0.344136f, -0.714136f, 1.772000f},
    {1.0f, 1.402000f, -0.344136f, -0.714136f, 1.772000f},
    {1.0f, 1.576000f, -0.226622f, -0.476622f, 1.826000f},
    {1.0f, 1.574800f, -0.187324f, -0.468124f, 1.855600f},
    {1.0f, 1.474600f, -0.164553f, -0.571353f, 1.881400f},
    {1.0f, 1.474600f, -0.164553f, -0.571353f, 1.881400f},
};

// libswscale's colourspace table (the values sws_getCoefficients() returns, 16.16 fixed point:
// V->R, U->B, -U->G, -V->G), indexed by its SWS_CS_* number; 8 and anything outside 0..10 fall
// back to the BT.601 row, as that function does.  FFmpeg's source is not part of the reference
// tree; the numbers are pinned against the loaded library by the test-suite.
static const int kSwsTable[11][4] = {
    {104597, 132201, 25675, 53279},  // 0 default
    {117489, 138438, 13975, 34925},  // 1 ITU-R BT.709
    {104597, 132201, 25675, 53279},  // 2 unspecified
    {104597, 132201, 25675, 53279},  // 3 reserved
    {104448, 132798, 24759, 53109},  // 4 FCC
    {104597, 132201, 25675, 53279},  // 5 ITU-R BT.601 (624)
    {104597, 132201, 25675, 53279},  // 6 SMPTE 170M
    {117579, 136230, 16907, 35559},  // 7 SMPTE 240M
    {104597, 132201, 25675, 53279},  // 8 (no entry of its own)
    {110013, 140363, 12277, 42626},  // 9 BT.2020 non-constant luminance
    {110013, 140363, 12277, 42626},  // 10 BT.2020 constant luminance
};

// The 16-bit coefficients of libswscale's SIMD converter for default brightness, contrast and
// saturation: round(c * 2^13) of the 16.16 table entries, luma gain 255/219 and chroma as
// tabulated for limited-range sources, luma gain 1 and chroma scaled by 224/255 for full-range
// ones (integer arithmetic throughout, as the library computes them).
static ColorMat sws_matrix(int k, int full_range) {
  if (k < 0 || k > 10) k = 5;
  long long crv = kSwsTable[k][0], cbu = kSwsTable[k][1], cgu = -kSwsTable[k][2],
            cgv = -kSwsTable[k][3], cy = 1 << 16;
  if (!full_range) {
    cy = cy * 255 / 219;
  } else {
    crv = crv * 224 / 255;
    cbu = cbu * 224 / 255;
    cgu = cgu * 224 / 255;
    cgv = cgv * 224 / 255;
  }
  auto coeff = [](long long c) {  // round(c * 2^13 / 2^16) clipped to 16 bits, then / 2^13
    long long r = (c * 8192 + 32768) >> 16;
    r = r < -32768 ? -32768 : (r > 32767 ? 32767 : r);
    return (float)r / 8192.0f;
  };
  ColorMat m;
  m.g = coeff(cy); m.vr = coeff(crv); m.ug = coeff(cgu); m.vg = coeff(cgv); m.ub = coeff(cbu);
  m.y_bias = 8388608.0f + (full_range ? 0.0f : 16.0f);
  m.neg_zero = -0.0f;
  return m;
}

ColorMat color_matrix(int k, int full_range, int arith) {
  if (arith == B2_ARITH_SWSCALE) return sws_matrix(k, full_range);
  if (k <= 0 || k > 10) k = 1;  // color_conversion.cu:120-123
  const float* r = full_range ? kFull[k - 1] : kLimited[k - 1];
  ColorMat m;
  m.g = r[0]; m.vr = r[1]; m.ug = r[2]; m.vg = r[3]; m.ub = r[4];
  m.y_bias = 8388608.0f + (full_range ? 0.0f : 16.0f);
  m.neg_zero = -0.0f;
  return m;
}

namespace {

bool valid_enum(int v, int hi) { return v >= 0 && v <= hi; }

int planar_entry(void* stream, const uint8_t* src, int src_pitch, uint8_t* dst, int dst_pitch,
                 int width, int height, int num_frames, int coeff, int order) {
  clear_error();
  if (width < 0 || height < 0 || num_frames < 0)
    return fail(B2_ERR_INVALID, "negative size: width %d, height %d, num_frames %d", width, height,
                num_frames);
  if (num_frames == 0 || width == 0 || height == 0) return B2_OK;
  if (!src || !dst) return fail(B2_ERR_INVALID, "null %s pointer", src ? "dst" : "src");
  if (src_pitch < width || dst_pitch < width)
    return fail(B2_ERR_INVALID, "pitch smaller than width (%d, %d < %d)", src_pitch, dst_pitch,
                width);
  DenseLaunch L{};
  L.y = src;
  L.u = src + (long long)height * src_pitch;  // color_conversion.cu:117
  L.y_pitch = L.uv_pitch = src_pitch;
  // the reference strides frames by width, not by pitch (color_conversion.cu:106-107)
  L.y_frame_stride = L.uv_frame_stride = (long long)(height + height / 2) * width;
  L.src_format = B2_SRC_NV12;
  L.width = width; L.height = height; L.num_frames = num_frames;
  L.mat = color_matrix(coeff, 0);
  L.dst = dst;
  L.dst_row_pitch = dst_pitch;
  L.dst_plane_stride = (long long)height * dst_pitch;   // color_conversion.cu:136
  L.dst_frame_stride = 3LL * height * width;            // color_conversion.cu:107
  L.layout = B2_NCHW; L.dtype = B2_U8; L.order = order;
  for (int i = 0; i < 3; ++i) { L.sb.s[i] = 1.0f; L.sb.b[i] = 0.0f; }
  return launch_dense(L, static_cast<cudaStream_t>(stream));
}

}  // namespace
}  // namespace b2

using namespace b2;

extern "C" {

B2_API const char* b2_last_error(void) { return g_err; }
B2_API int b2_abi_version(void) { return B2_ABI_VERSION; }

B2_API int b2_init(int device) {
  clear_error();
  DeviceGuard g(device);
  B2_CUDA(g.status(), "selecting the device failed");
  B2_CUDA(cudaFree(nullptr), "creating the primary context failed");
  return B2_OK;
}

B2_API int b2_device_count(int* count) {
  clear_error();
  if (!count) return fail(B2_ERR_INVALID, "null count pointer");
  B2_CUDA(cudaGetDeviceCount(count), "querying the device count failed");
  return B2_OK;
}

B2_API int b2_stream_synchronize(int device, void* stream) {
  clear_error();
  DeviceGuard g(device);
  B2_CUDA(g.status(), "selecting the device failed");
  B2_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)),
          "Failed to synchronize stream");
  return B2_OK;
}

B2_API int b2_nv12_to_planar_rgb(void* stream, const uint8_t* src, int src_pitch, uint8_t* dst,
                          int dst_pitch, int width, int height, int num_frames, int coeff) {
  return planar_entry(stream, src, src_pitch, dst, dst_pitch, width, height, num_frames, coeff,
                      B2_RGB);
}
B2_API int b2_nv12_to_planar_bgr(void* stream, const uint8_t* src, int src_pitch, uint8_t* dst,
                          int dst_pitch, int width, int height, int num_frames, int coeff) {
  return planar_entry(stream, src, src_pitch, dst, dst_pitch, width, height, num_frames, coeff,
                      B2_BGR);
}

B2_API int b2_convert_dense(const b2_dense_args* args, void* stream) {
  clear_error();
  if (!args) return fail(B2_ERR_INVALID, "null argument struct");
  // version 1 of the struct ended (with its tail padding) where `arith` starts now
  constexpr size_t kV1 = offsetof(b2_dense_args, arith);
  if (args->struct_size != sizeof(b2_dense_args) && args->struct_size != kV1)
    return fail(B2_ERR_INVALID, "b2_dense_args.struct_size is %u, this library expects %zu (or %zu)",
                args->struct_size, sizeof(b2_dense_args), kV1);
  b2_dense_args local{};
  memcpy(&local, args, args->struct_size);
  const b2_dense_args* a = &local;
  if (!valid_enum(a->arith, 1)) return fail(B2_ERR_INVALID, "unknown arith (%d)", a->arith);
  if (!valid_enum(a->src_format, 1) || !valid_enum(a->layout, 1) || !valid_enum(a->dtype, 2) ||
      !valid_enum(a->order, 1))
    return fail(B2_ERR_INVALID, "unknown src_format/layout/dtype/order (%d, %d, %d, %d)",
                a->src_format, a->layout, a->dtype, a->order);
  if (a->width < 0 || a->height < 0 || a->num_frames < 0)
    return fail(B2_ERR_INVALID, "negative size: width %d, height %d, num_frames %d", a->width,
                a->height, a->num_frames);
  if (a->num_frames == 0 || a->width == 0 || a->height == 0) return B2_OK;
  const bool table = a->y_table != nullptr;
  const bool i420 = a->src_format == B2_SRC_I420;
  if (table) {
    if (!a->u_table || (i420 && !a->v_table))
      return fail(B2_ERR_INVALID, "y_table given without u_table%s", i420 ? "/v_table" : "");
  } else if (!a->y || !a->u || (i420 && !a->v)) {
    return fail(B2_ERR_INVALID, "null source plane pointer");
  }
  if (!a->dst) return fail(B2_ERR_INVALID, "null dst pointer");
  // a trailing odd column is never converted, so its chroma is never read
  const long long min_uv = i420 ? a->width / 2 : (a->width & ~1);
  if (a->y_pitch < a->width || a->uv_pitch < min_uv)
    return fail(B2_ERR_INVALID, "pitch smaller than the row (y_pitch %lld, uv_pitch %lld, width %d)",
                (long long)a->y_pitch, (long long)a->uv_pitch, a->width);
  const long long packed = 3LL * a->height * a->width;
  if (a->dst_frame_stride != 0 && a->dst_frame_stride < packed)
    return fail(B2_ERR_INVALID, "dst_frame_stride %lld is smaller than one frame (%lld elements)",
                (long long)a->dst_frame_stride, packed);
  DeviceGuard g(a->device);
  B2_CUDA(g.status(), "selecting the device failed");
  DenseLaunch L{};
  L.y = static_cast<const uint8_t*>(a->y);
  L.u = static_cast<const uint8_t*>(a->u);
  L.v = static_cast<const uint8_t*>(a->v);
  L.y_table = a->y_table; L.u_table = a->u_table; L.v_table = a->v_table;
  L.y_pitch = a->y_pitch; L.uv_pitch = a->uv_pitch;
  L.y_frame_stride = a->y_frame_stride; L.uv_frame_stride = a->uv_frame_stride;
  L.src_format = a->src_format;
  L.width = a->width; L.height = a->height; L.num_frames = a->num_frames;
  L.mat = color_matrix(a->matrix_coeff, a->full_range, a->arith);
  L.arith = a->arith;
  L.dst = a->dst;
  L.layout = a->layout; L.dtype = a->dtype; L.order = a->order;
  L.dst_row_pitch = a->layout == B2_NCHW ? a->width : 3LL * a->width;
  L.dst_plane_stride = (long long)a->height * a->width;
  L.dst_frame_stride = a->dst_frame_stride ? a->dst_frame_stride : packed;
  for (int i = 0; i < 3; ++i) { L.sb.s[i] = a->scale[i]; L.sb.b[i] = a->bias[i]; }
  return launch_dense(L, static_cast<cudaStream_t>(stream));
}

B2_API int b2_convert_resize(const b2_resize_args* args, void* stream) {
  clear_error();
  if (!args) return fail(B2_ERR_INVALID, "null argument struct");
  constexpr size_t kV1 = offsetof(b2_resize_args, arith);  // where version 1 of the struct ended
  if (args->struct_size != sizeof(b2_resize_args) && args->struct_size != kV1)
    return fail(B2_ERR_INVALID,
                "b2_resize_args.struct_size is %u, this library expects %zu (or %zu)",
                args->struct_size, sizeof(b2_resize_args), kV1);
  b2_resize_args local{};
  memcpy(&local, args, args->struct_size);
  const b2_resize_args* a = &local;
  if (!valid_enum(a->src_format, 3) || !valid_enum(a->layout, 1) || !valid_enum(a->dtype, 2) ||
      !valid_enum(a->order, 1) || !valid_enum(a->arith, 1))
    return fail(B2_ERR_INVALID, "unknown src_format/layout/dtype/order/arith (%d, %d, %d, %d, %d)",
                a->src_format, a->layout, a->dtype, a->order, a->arith);
  if (a->num_images < 0 || a->out_w < 0 || a->out_h < 0 || a->max_src_w < 0)
    return fail(B2_ERR_INVALID, "negative size: num_images %d, out %dx%d, max_src_w %d",
                a->num_images, a->out_w, a->out_h, a->max_src_w);
  if (a->num_images == 0 || a->out_w == 0 || a->out_h == 0) return B2_OK;
  if (!a->base || !a->descs || !a->dst)
    return fail(B2_ERR_INVALID, "null base, descs or dst pointer");
  if (a->max_src_w < 1) return fail(B2_ERR_INVALID, "max_src_w must be at least 1");
  const long long plane = (long long)a->out_w * a->out_h;
  if (a->dst_plane_stride != 0) {
    if (a->layout != B2_NCHW)
      return fail(B2_ERR_INVALID, "dst_plane_stride needs the planar (NCHW) layout");
    if (a->dst_plane_stride < plane)
      return fail(B2_ERR_INVALID, "dst_plane_stride %lld is smaller than one plane",
                  (long long)a->dst_plane_stride);
    if (a->dst_image_stride != 0 && a->dst_image_stride < plane)
      return fail(B2_ERR_INVALID, "dst_image_stride %lld is smaller than one plane",
                  (long long)a->dst_image_stride);
  } else if (a->dst_image_stride != 0 && a->dst_image_stride < 3 * plane) {
    return fail(B2_ERR_INVALID, "dst_image_stride %lld is smaller than one image",
                (long long)a->dst_image_stride);
  }
  if (a->frames_per_group < 0 || (a->frames_per_group > 1 && a->dst_group_stride <= 0))
    return fail(B2_ERR_INVALID, "frames_per_group %d needs a positive dst_group_stride (%lld)",
                a->frames_per_group, (long long)a->dst_group_stride);
  const bool yuv_src = a->src_format == B2_SRC_NV12 || a->src_format == B2_SRC_I420;
  if ((a->luma_row_map == nullptr) != (a->chroma_row_map == nullptr) && yuv_src)
    return fail(B2_ERR_INVALID, "luma_row_map and chroma_row_map go together for YUV sources");
  if (a->chroma_row_map != nullptr && a->luma_row_map == nullptr)
    return fail(B2_ERR_INVALID, "chroma_row_map given without luma_row_map");
  for (int i = 0; i < 3; ++i)
    if (!(a->pad_value[i] >= 0.0f && a->pad_value[i] <= 255.0f))
      return fail(B2_ERR_INVALID, "pad_value[%d] = %g is outside 0..255", i, a->pad_value[i]);
  DeviceGuard g(a->device);
  B2_CUDA(g.status(), "selecting the device failed");
  return launch_resize(*a, static_cast<cudaStream_t>(stream));
}

B2_API int b2_touched_rows(const b2_image_desc* d, int src_format, int out_h, int32_t* luma_map,
                    int32_t* chroma_map, int32_t* n_luma, int32_t* n_chroma) {
  clear_error();
  if (!d || !luma_map || !n_luma) return fail(B2_ERR_INVALID, "null pointer argument");
  if (!valid_enum(src_format, 3)) return fail(B2_ERR_INVALID, "unknown src_format (%d)", src_format);
  const bool yuv = src_format == B2_SRC_NV12 || src_format == B2_SRC_I420;
  if (yuv && (!chroma_map || !n_chroma))
    return fail(B2_ERR_INVALID, "a YUV source needs chroma_map and n_chroma");
  if (d->src_w < 1 || d->src_h < 1 || !(d->scale_y > 0.0f) || out_h < 0)
    return fail(B2_ERR_INVALID, "the descriptor has an empty source or a non-positive scale");
  const int ch = (d->src_h + 1) / 2;
  for (int r = 0; r < d->src_h; ++r) luma_map[r] = -1;
  if (yuv)
    for (int r = 0; r < ch; ++r) chroma_map[r] = -1;
  for (int oy = 0; oy < out_h; ++oy) {
    const int gy = d->crop_y + oy;
    if (d->resized_h > 0 && (gy < 0 || gy >= d->resized_h)) continue;  // a row of padding
    // the kernel's axis_of: fma, clamp at zero, truncate, clamp at the last row
    float s = fmaf(d->scale_y, (float)gy + 0.5f, -0.5f);
    if (!(s > 0.0f)) s = 0.0f;
    if (!(s < 4194304.0f)) return fail(B2_ERR_INVALID, "source coordinates beyond 2^22");
    int y0 = (int)s;
    if (y0 > d->src_h - 1) y0 = d->src_h - 1;
    const int y1 = y0 + 1 < d->src_h ? y0 + 1 : d->src_h - 1;
    luma_map[y0] = luma_map[y1] = 0;
    if (yuv) chroma_map[y0 >> 1] = chroma_map[y1 >> 1] = 0;
  }
  int nl = 0, nc = 0;
  for (int r = 0; r < d->src_h; ++r)
    if (luma_map[r] == 0) luma_map[r] = nl++;
  if (yuv)
    for (int r = 0; r < ch; ++r)
      if (chroma_map[r] == 0) chroma_map[r] = nc++;
  *n_luma = nl;
  if (n_chroma) *n_chroma = nc;
  return B2_OK;
}

// Host threads a large b2_copy_rows call may use: B2_HOST_COPY_THREADS, else half the hardware
// threads, eight at most (callers are pipeline worker threads, several at a time).
static long long host_copy_threads() {
  if (const char* e = std::getenv("B2_HOST_COPY_THREADS")) {
    const long long v = std::atoll(e);
    if (v >= 1) return v < 64 ? v : 64;
  }
  const unsigned hw = std::thread::hardware_concurrency();
  const long long half = hw / 2;
  return half < 1 ? 1 : (half > 8 ? 8 : half);
}

// A copy into a staging buffer that the copy engine reads next: streaming stores (the data goes
// to memory instead of lingering in this core's cache, from where the engine would have to fetch
// it line by line: an upload right after a cached copy ran at half the link's rate).
static void stream_copy(char* dst, const char* src, size_t n) {
#if defined(__x86_64__)
  if (n >= 1024) {
    const size_t head = (16 - ((uintptr_t)dst & 15)) & 15;
    memcpy(dst, src, head);
    dst += head; src += head; n -= head;
    const size_t body = n & ~(size_t)63;
    for (size_t i = 0; i < body; i += 64) {
      const __m128i a0 = _mm_loadu_si128(reinterpret_cast<const __m128i*>(src + i));
      const __m128i a1 = _mm_loadu_si128(reinterpret_cast<const __m128i*>(src + i + 16));
      const __m128i a2 = _mm_loadu_si128(reinterpret_cast<const __m128i*>(src + i + 32));
      const __m128i a3 = _mm_loadu_si128(reinterpret_cast<const __m128i*>(src + i + 48));
      _mm_stream_si128(reinterpret_cast<__m128i*>(dst + i), a0);
      _mm_stream_si128(reinterpret_cast<__m128i*>(dst + i + 16), a1);
      _mm_stream_si128(reinterpret_cast<__m128i*>(dst + i + 32), a2);
      _mm_stream_si128(reinterpret_cast<__m128i*>(dst + i + 48), a3);
    }
    _mm_sfence();
    memcpy(dst + body, src + body, n - body);
    return;
  }
#endif
  memcpy(dst, src, n);
}

// memcpy by several host threads: one per 2 MiB at least, slices cut on 4 KiB boundaries.
static void host_copy(void* dst, const void* src, size_t n) {
  long long threads = (long long)(n / (2u << 20));
  const long long cap = host_copy_threads();
  if (threads > cap) threads = cap;
  if (threads <= 1) {
    stream_copy(static_cast<char*>(dst), static_cast<const char*>(src), n);
    return;
  }
  const size_t slice = ((n / (size_t)threads) + 4095) & ~(size_t)4095;
  auto part = [=](size_t first) {
    if (first < n)
      stream_copy(static_cast<char*>(dst) + first, static_cast<const char*>(src) + first,
                  n - first < slice ? n - first : slice);
  };
  std::vector<std::thread> pool;
  pool.reserve((size_t)threads - 1);
  size_t mine = 0;  // slices from here on are still to be copied by this thread
  try {
    for (long long t = 1; t < threads; ++t) pool.emplace_back(part, (size_t)t * slice);
  } catch (...) {  // no more threads to be had
    mine = (pool.size() + 1) * slice;
  }
  part(0);
  if (mine)
    for (size_t first = mine; first < n; first += slice) part(first);
  for (auto& th : pool) th.join();
}

B2_API int b2_copy_host(void* dst, const void* src, size_t nbytes) {
  clear_error();
  if (nbytes == 0) return B2_OK;
  if (!dst || !src) return fail(B2_ERR_INVALID, "null pointer argument");
  host_copy(dst, src, nbytes);
  return B2_OK;
}

B2_API int b2_pack_host(void* dst, const void* const* srcs, const int64_t* sizes,
                 const int64_t* dst_offsets, int num_items) {
  clear_error();
  if (num_items < 0) return fail(B2_ERR_INVALID, "negative number of items: %d", num_items);
  if (num_items == 0) return B2_OK;
  if (!dst || !srcs || !sizes || !dst_offsets) return fail(B2_ERR_INVALID, "null pointer argument");
  long long total = 0;
  for (int i = 0; i < num_items; ++i) {
    if (sizes[i] < 0 || dst_offsets[i] < 0 || (sizes[i] > 0 && !srcs[i]))
      return fail(B2_ERR_INVALID, "item %d: size %lld, offset %lld, source %p", i,
                  (long long)sizes[i], (long long)dst_offsets[i], srcs[i]);
    total += sizes[i];
  }
  // whole items per thread, cut where the running byte count passes a multiple of total / threads
  long long threads = total / (2LL << 20);
  const long long cap = host_copy_threads();
  if (threads > cap) threads = cap;
  if (threads > num_items) threads = num_items;
  if (threads < 1) threads = 1;
  auto copy_items = [=](int first, int last) {
    for (int i = first; i < last; ++i)
      if (sizes[i])
        stream_copy(static_cast<char*>(dst) + dst_offsets[i], static_cast<const char*>(srcs[i]),
                    (size_t)sizes[i]);
  };
  if (threads == 1) {
    copy_items(0, num_items);
    return B2_OK;
  }
  std::vector<int> cut((size_t)threads + 1, num_items);
  cut[0] = 0;
  long long seen = 0;
  int t = 1;
  for (int i = 0; i < num_items && t < threads; ++i) {
    seen += sizes[i];
    while (t < threads && seen >= total * t / threads) cut[(size_t)t++] = i + 1;
  }
  std::vector<std::thread> pool;
  pool.reserve((size_t)threads - 1);
  int mine_from = num_items;  // items from here on are still to be copied by this thread
  try {
    for (long long k = 1; k < threads; ++k)
      pool.emplace_back(copy_items, cut[(size_t)k], cut[(size_t)k + 1]);
  } catch (...) {  // no more threads to be had
    mine_from = cut[pool.size() + 1];
  }
  copy_items(0, cut[1]);
  copy_items(mine_from, num_items);
  for (auto& th : pool) th.join();
  return B2_OK;
}

B2_API int b2_copy_rows(void* dst, int64_t dst_frame_stride, const void* src, int64_t src_frame_stride,
                 int64_t src_pitch, const int32_t* rows, int num_rows, int64_t row_bytes,
                 int num_frames) {
  clear_error();
  if (num_rows < 0 || num_frames < 0 || row_bytes < 0)
    return fail(B2_ERR_INVALID, "negative size: num_rows %d, num_frames %d, row_bytes %lld", num_rows,
                num_frames, (long long)row_bytes);
  if (num_rows == 0 || num_frames == 0 || row_bytes == 0) return B2_OK;
  if (!dst || !src || !rows) return fail(B2_ERR_INVALID, "null pointer argument");
  for (int i = 0; i < num_rows; ++i)
    if (rows[i] < 0) return fail(B2_ERR_INVALID, "rows[%d] = %d is negative", i, rows[i]);
  // (frame, row) items in frame-major order, cut into one contiguous range per thread; inside a
  // range, rows that follow one another in the source and in the destination go as one memcpy.
  const long long items = (long long)num_frames * num_rows;
  auto copy_range = [=](long long first, long long last) {
    long long it = first;
    while (it < last) {
      const long long f = it / num_rows;
      const int i = (int)(it - f * num_rows);
      const long long frame_end = (f + 1) * (long long)num_rows < last ? (f + 1) * (long long)num_rows : last;
      int run = 1;
      if (src_pitch == row_bytes)
        while (it + run < frame_end && rows[i + run] == rows[i] + run) ++run;
      stream_copy(static_cast<char*>(dst) + f * dst_frame_stride + (long long)i * row_bytes,
                  static_cast<const char*>(src) + f * src_frame_stride +
                      (long long)rows[i] * src_pitch,
                  (size_t)row_bytes * run);
      it += run;
    }
  };
  const long long total = items * row_bytes;
  long long threads = total / (2LL << 20);  // a thread per 2 MiB at least
  const long long cap = host_copy_threads();
  if (threads > cap) threads = cap;
  if (threads > items) threads = items;
  if (threads <= 1) {
    copy_range(0, items);
    return B2_OK;
  }
  std::vector<std::thread> pool;
  pool.reserve((size_t)threads - 1);
  try {
    for (long long t = 1; t < threads; ++t)
      pool.emplace_back(copy_range, items * t / threads, items * (t + 1) / threads);
  } catch (...) {  // no more threads to be had: this one does what the missing ones would have
    copy_range(items * ((long long)pool.size() + 1) / threads, items);
  }
  copy_range(0, items / threads);
  for (auto& th : pool) th.join();
  return B2_OK;
}

B2_API int b2_gather_surfaces(const void* const* surfaces, const int64_t* pitches, int num_frames,
                       int width, int height, uint8_t* dst, int device, void* stream) {
  clear_error();
  if (num_frames < 0 || width < 0 || height < 0)
    return fail(B2_ERR_INVALID, "negative size: num_frames %d, width %d, height %d", num_frames,
                width, height);
  if (num_frames == 0 || width == 0 || height == 0) return B2_OK;
  if (!surfaces || !pitches || !dst) return fail(B2_ERR_INVALID, "null pointer argument");
  if (height % 2) return fail(B2_ERR_INVALID, "NV12 height must be even. Found: %d", height);
  DeviceGuard g(device);
  B2_CUDA(g.status(), "selecting the device failed");
  return launch_gather(surfaces, pitches, num_frames, width, height, dst,
                       static_cast<cudaStream_t>(stream));
}

B2_API int b2_transfer_h2d(void* dst, const void* host_src, size_t nbytes, int src_is_pinned, int device,
                    void* stream) {
  clear_error();
  if (nbytes == 0) return B2_OK;
  if (!dst || !host_src) return fail(B2_ERR_INVALID, "null pointer argument");
  DeviceGuard g(device);
  B2_CUDA(g.status(), "selecting the device failed");
  if (src_is_pinned) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    B2_CUDA(cudaMemcpyAsync(dst, host_src, nbytes, cudaMemcpyHostToDevice, s),
            "Failed to initiate async memory copy from host to device.");
    B2_CUDA(cudaStreamSynchronize(s), "Failed to synchronize the stream.");
  } else {
    B2_CUDA(cudaMemcpy(dst, host_src, nbytes, cudaMemcpyHostToDevice),
            "Failed to copy data from host to device.");
  }
  return B2_OK;
}

B2_API int b2_transfer_h2d_async(void* dst, const void* host_src, size_t nbytes, int device,
                          void* stream) {
  clear_error();
  if (nbytes == 0) return B2_OK;
  if (!dst || !host_src) return fail(B2_ERR_INVALID, "null pointer argument");
  DeviceGuard g(device);
  B2_CUDA(g.status(), "selecting the device failed");
  B2_CUDA(cudaMemcpyAsync(dst, host_src, nbytes, cudaMemcpyHostToDevice,
                          static_cast<cudaStream_t>(stream)),
          "Failed to initiate async memory copy from host to device.");
  return B2_OK;
}

namespace {
struct EventPair {  // two events without timing, destroyed on every way out
  cudaEvent_t ev[2] = {nullptr, nullptr};
  ~EventPair() {
    for (auto e : ev)
      if (e) cudaEventDestroy(e);
  }
};
}  // namespace

B2_API int b2_transfer_h2d_staged(void* dst, const void* host_src, size_t nbytes, void* staging,
                           size_t staging_bytes, int device, void* stream) {
  clear_error();
  if (nbytes == 0) return B2_OK;
  if (!dst || !host_src || !staging) return fail(B2_ERR_INVALID, "null pointer argument");
  const size_t half = (staging_bytes / 2) & ~(size_t)255;
  if (half == 0)
    return fail(B2_ERR_INVALID, "the staging buffer must hold 512 bytes at least. Found: %zu",
                staging_bytes);
  DeviceGuard g(device);
  B2_CUDA(g.status(), "selecting the device failed");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  EventPair done;
  for (auto& e : done.ev)
    B2_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "Failed to create an event.");
  bool used[2] = {false, false};
  int k = 0;
  for (size_t off = 0; off < nbytes; k ^= 1) {
    const size_t n = nbytes - off < half ? nbytes - off : half;
    char* slot = static_cast<char*>(staging) + (size_t)k * half;
    if (used[k])  // the upload that last read this half has finished
      B2_CUDA(cudaEventSynchronize(done.ev[k]), "Failed to wait for an upload.");
    host_copy(slot, static_cast<const char*>(host_src) + off, n);
    B2_CUDA(cudaMemcpyAsync(static_cast<char*>(dst) + off, slot, n, cudaMemcpyHostToDevice, s),
            "Failed to initiate async memory copy from host to device.");
    B2_CUDA(cudaEventRecord(done.ev[k], s), "Failed to record an event.");
    used[k] = true;
    off += n;
  }
  B2_CUDA(cudaStreamSynchronize(s), "Failed to synchronize the stream.");
  return B2_OK;
}

B2_API int b2_transfer_d2h(void* host_dst, const void* src, size_t nbytes, int device) {
  clear_error();
  if (nbytes == 0) return B2_OK;
  if (!host_dst || !src) return fail(B2_ERR_INVALID, "null pointer argument");
  DeviceGuard g(device);
  B2_CUDA(g.status(), "selecting the device failed");
  B2_CUDA(cudaMemcpy(host_dst, src, nbytes, cudaMemcpyDeviceToHost),
          "Failed to copy data from device to host.");
  return B2_OK;
}

B2_API int b2_transfer_d2h_staged(void* host_dst, const void* src, size_t nbytes, void* staging,
                           size_t staging_bytes, int device, void* stream) {
  clear_error();
  if (nbytes == 0) return B2_OK;
  if (!host_dst || !src || !staging) return fail(B2_ERR_INVALID, "null pointer argument");
  const size_t half = (staging_bytes / 2) & ~(size_t)255;
  if (half == 0)
    return fail(B2_ERR_INVALID, "the staging buffer must hold 512 bytes at least. Found: %zu",
                staging_bytes);
  DeviceGuard g(device);
  B2_CUDA(g.status(), "selecting the device failed");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  EventPair done;
  for (auto& e : done.ev)
    B2_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "Failed to create an event.");
  // the download of chunk i + 1 into one half runs under the copy of chunk i out of the other
  const size_t chunks = (nbytes + half - 1) / half;
  auto download = [&](size_t i) -> cudaError_t {
    const size_t off = i * half, n = nbytes - off < half ? nbytes - off : half;
    cudaError_t e = cudaMemcpyAsync(static_cast<char*>(staging) + (i & 1) * half,
                                    static_cast<const char*>(src) + off, n,
                                    cudaMemcpyDeviceToHost, s);
    return e != cudaSuccess ? e : cudaEventRecord(done.ev[i & 1], s);
  };
  B2_CUDA(download(0), "Failed to initiate async memory copy from device to host.");
  for (size_t i = 0; i < chunks; ++i) {
    if (i + 1 < chunks)
      B2_CUDA(download(i + 1), "Failed to initiate async memory copy from device to host.");
    B2_CUDA(cudaEventSynchronize(done.ev[i & 1]), "Failed to wait for a download.");
    const size_t off = i * half, n = nbytes - off < half ? nbytes - off : half;
    host_copy(static_cast<char*>(host_dst) + off, static_cast<char*>(staging) + (i & 1) * half, n);
  }
  return B2_OK;
}

B2_API int b2_alloc_pinned(void** host_ptr, size_t nbytes) {
  clear_error();
  if (!host_ptr) return fail(B2_ERR_INVALID, "null pointer argument");
  if (nbytes == 0) return fail(B2_ERR_INVALID, "`size` must be greater than 0.");
  B2_CUDA(cudaHostAlloc(host_ptr, nbytes, cudaHostAllocDefault),
          "Failed to allocate pinned memory.");
  return B2_OK;
}

B2_API int b2_free_pinned(void* host_ptr) {
  clear_error();
  if (!host_ptr) return B2_OK;
  B2_CUDA(cudaFreeHost(host_ptr), "Failed to free pinned memory.");
  return B2_OK;
}

B2_API int b2_device_alloc(void** ptr, size_t nbytes, int device) {
  clear_error();
  if (!ptr) return fail(B2_ERR_INVALID, "null pointer argument");
  if (nbytes == 0) return fail(B2_ERR_INVALID, "`size` must be greater than 0.");
  DeviceGuard g(device);
  B2_CUDA(g.status(), "selecting the device failed");
  B2_CUDA(cudaMalloc(ptr, nbytes), "Failed to allocate CUDA memory");
  return B2_OK;
}

B2_API int b2_device_free(void* ptr, int device) {
  clear_error();
  if (!ptr) return B2_OK;
  DeviceGuard g(device);
  B2_CUDA(g.status(), "selecting the device failed");
  B2_CUDA(cudaFree(ptr), "Failed to free CUDA memory");
  return B2_OK;
}

B2_API int b2_frame_checksum(const uint8_t* src, int64_t frame_bytes, int num_frames, uint64_t* out,
                      int device, void* stream) {
  clear_error();
  if (num_frames < 0 || frame_bytes < 0)
    return fail(B2_ERR_INVALID, "negative size: num_frames %d, frame_bytes %lld", num_frames,
                (long long)frame_bytes);
  if (num_frames == 0) return B2_OK;
  if (!out || (!src && frame_bytes)) return fail(B2_ERR_INVALID, "null pointer argument");
  DeviceGuard g(device);
  B2_CUDA(g.status(), "selecting the device failed");
  return launch_checksum(src, frame_bytes, num_frames, out, static_cast<cudaStream_t>(stream));
}

}  // extern "C"

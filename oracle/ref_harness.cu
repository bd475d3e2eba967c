// extern "C" doorway to the reference's own colour-conversion launchers
// (src/libspdl/cuda/detail/color_conversion.cu:155-193), so that tests and the
// benchmark can run the unmodified reference kernel on a GPU through ctypes.
// TEST INFRASTRUCTURE ONLY: nothing in the shipped package links this.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <exception>

namespace spdl::cuda::detail {
void nv12_to_planar_rgb(CUstream, uint8_t*, int, uint8_t*, int, int, int, int, int);
void nv12_to_planar_bgr(CUstream, uint8_t*, int, uint8_t*, int, int, int, int, int);
}  // namespace spdl::cuda::detail

namespace {
template <class F>
int guarded(F&& f) {
  try {
    f();
  } catch (const std::exception& e) {
    std::fprintf(stderr, "ref_harness: %s\n", e.what());
    return 1;
  }
  return 0;
}
}  // namespace

extern "C" {
int ref_nv12_to_planar_rgb(void* stream, uint8_t* src, int src_pitch, uint8_t* dst, int dst_pitch,
                           int width, int height, int num_frames, int coeff) {
  return guarded([&] {
    spdl::cuda::detail::nv12_to_planar_rgb((CUstream)stream, src, src_pitch, dst, dst_pitch, width,
                                           height, num_frames, coeff);
  });
}
int ref_nv12_to_planar_bgr(void* stream, uint8_t* src, int src_pitch, uint8_t* dst, int dst_pitch,
                           int width, int height, int num_frames, int coeff) {
  return guarded([&] {
    spdl::cuda::detail::nv12_to_planar_bgr((CUstream)stream, src, src_pitch, dst, dst_pitch, width,
                                           height, num_frames, coeff);
  });
}
}

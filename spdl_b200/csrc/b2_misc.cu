// Frame batching (pitched surfaces -> packed batch) and the per-frame checksum.
#include "b2_common.cuh"

namespace b2 {
namespace {

// One CTA row copies one row of one surface.  16-byte vectors when both ends allow it.
__global__ void __launch_bounds__(128) gather_kernel(const void* const* surfaces,
                                                     const long long* pitches, int width, int h2,
                                                     uint8_t* dst) {
  const int n = blockIdx.z;
  const int row = blockIdx.y;
  const uint8_t* s = static_cast<const uint8_t*>(surfaces[n]) + (long long)row * pitches[n];
  uint8_t* d = dst + ((long long)n * h2 + row) * width;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if ((((uintptr_t)s | (uintptr_t)d) & 15) == 0) {
    const int nvec = width >> 4;
    if (t < nvec)
      __stcs(reinterpret_cast<uint4*>(d) + t, __ldcs(reinterpret_cast<const uint4*>(s) + t));
    const int tail = width - (nvec << 4);
    if (t < tail) d[(nvec << 4) + t] = s[(nvec << 4) + t];
  } else {
    for (int i = t * 16; i < min(width, t * 16 + 16); ++i) d[i] = s[i];
  }
}

// Sum over a frame of (byte+1) * (1 + j mod 65521), j the byte's index in the frame.
__global__ void __launch_bounds__(256) checksum_kernel(const uint8_t* src, long long frame_bytes,
                                                       unsigned long long* out) {
  const int n = blockIdx.y;
  const uint8_t* f = src + (long long)n * frame_bytes;
  unsigned long long acc = 0;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const bool vec = (((uintptr_t)f) & 15) == 0;
  const long long nvec = vec ? frame_bytes >> 4 : 0;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    const uint4 q = __ldcs(reinterpret_cast<const uint4*>(f) + i);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    uint32_t k = (uint32_t)((i << 4) % 65521);
    if (k + 15u < 65521u) {
      // no wrap of the weight inside these 16 bytes:
      //   sum (b_i + 1)(1 + k + i) = (1 + k)(sum b_i + 16) + (sum i*b_i + 120)
      // with both byte sums from four-way dot products
      uint32_t s1 = 16u, s2 = 120u;
      s1 = __dp4a(w[0], 0x01010101u, s1);
      s1 = __dp4a(w[1], 0x01010101u, s1);
      s1 = __dp4a(w[2], 0x01010101u, s1);
      s1 = __dp4a(w[3], 0x01010101u, s1);
      s2 = __dp4a(w[0], 0x03020100u, s2);
      s2 = __dp4a(w[1], 0x07060504u, s2);
      s2 = __dp4a(w[2], 0x0B0A0908u, s2);
      s2 = __dp4a(w[3], 0x0F0E0D0Cu, s2);
      acc += (unsigned long long)(1u + k) * s1 + s2;
    } else {
#pragma unroll
      for (int b = 0; b < 16; ++b) {
        acc += (unsigned long long)(((w[b >> 2] >> (8 * (b & 3))) & 255u) + 1u) * (1u + k);
        k = k + 1 == 65521u ? 0u : k + 1;
      }
    }
  }
  for (long long j = (nvec << 4) + (long long)blockIdx.x * blockDim.x + threadIdx.x;
       j < frame_bytes; j += stride)
    acc += (unsigned long long)(f[j] + 1u) * (1u + (uint32_t)(j % 65521));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  __shared__ unsigned long long part[8];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long s = 0;
    for (int i = 0; i < 8; ++i) s += part[i];
    atomicAdd(out + n, s);
  }
}

}  // namespace

int launch_gather(const void* const* surfaces, const int64_t* pitches, int num_frames, int width,
                  int height, uint8_t* dst, cudaStream_t stream) {
  const int h2 = height + height / 2;
  if (num_frames == 0 || width == 0 || h2 == 0) return B2_OK;
  const int per_row = (width + 15) / 16;
  for (int n0 = 0; n0 < num_frames; n0 += 65535) {
    const int nn = num_frames - n0 < 65535 ? num_frames - n0 : 65535;
    dim3 grid((per_row + 127) / 128, h2, nn);
    gather_kernel<<<grid, 128, 0, stream>>>(surfaces + n0,
                                            reinterpret_cast<const long long*>(pitches) + n0, width,
                                            h2, dst + (long long)n0 * h2 * width);
    B2_CUDA(cudaPeekAtLastError(), "launch of the surface gather kernel failed");
  }
  return B2_OK;
}

int launch_checksum(const uint8_t* src, int64_t frame_bytes, int num_frames, uint64_t* out,
                    cudaStream_t stream) {
  if (num_frames == 0) return B2_OK;
  B2_CUDA(cudaMemsetAsync(out, 0, sizeof(uint64_t) * (size_t)num_frames, stream),
          "clearing the checksum output failed");
  if (frame_bytes == 0) return B2_OK;
  // about four 16-byte vectors per thread, at most 1024 CTAs per frame
  long long blocks = (frame_bytes / 16 + 1023) / 1024;
  if (blocks > 1024) blocks = 1024;
  if (blocks < 1) blocks = 1;
  for (int n0 = 0; n0 < num_frames; n0 += 65535) {
    const int nn = num_frames - n0 < 65535 ? num_frames - n0 : 65535;
    checksum_kernel<<<dim3((unsigned)blocks, nn), 256, 0, stream>>>(
        src + (long long)n0 * frame_bytes, frame_bytes,
        reinterpret_cast<unsigned long long*>(out) + n0);
    B2_CUDA(cudaPeekAtLastError(), "launch of the checksum kernel failed");
  }
  return B2_OK;
}

}  // namespace b2

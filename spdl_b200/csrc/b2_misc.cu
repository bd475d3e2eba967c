// Frame batching (pitched surfaces -> packed batch) and the per-frame checksum.
#include "b2_common.cuh"

namespace b2 {
namespace {

// One thread copies 16 bytes of kGatherRows consecutive rows of one surface: all loads are issued
// before the first store, so each thread keeps several 16-byte requests in flight.
constexpr int kGatherRows = 4;
__global__ void __launch_bounds__(128) gather_kernel(const void* const* surfaces,
                                                     const long long* pitches, int width, int h2,
                                                     uint8_t* dst) {
  const int n = blockIdx.z;
  const int row0 = blockIdx.y * kGatherRows;
  const long long pitch = pitches[n];
  const uint8_t* s = static_cast<const uint8_t*>(surfaces[n]) + (long long)row0 * pitch;
  uint8_t* d = dst + ((long long)n * h2 + row0) * width;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  const int rows = min(kGatherRows, h2 - row0);
  // every row of the group is 16-byte aligned on both sides
  if ((((uintptr_t)s | (uintptr_t)d | (uintptr_t)pitch | (uintptr_t)width) & 15) == 0) {
    if (t >= (width >> 4)) return;
    uint4 v[kGatherRows];
#pragma unroll
    for (int r = 0; r < kGatherRows; ++r)
      if (r < rows) v[r] = __ldcs(reinterpret_cast<const uint4*>(s + r * pitch) + t);
#pragma unroll
    for (int r = 0; r < kGatherRows; ++r)
      if (r < rows) __stcs(reinterpret_cast<uint4*>(d + (long long)r * width) + t, v[r]);
  } else {
    for (int r = 0; r < rows; ++r) {
      const uint8_t* sr = s + r * pitch;
      uint8_t* dr = d + (long long)r * width;
      if ((((uintptr_t)sr | (uintptr_t)dr) & 15) == 0) {
        const int nvec = width >> 4;
        if (t < nvec)
          __stcs(reinterpret_cast<uint4*>(dr) + t, __ldcs(reinterpret_cast<const uint4*>(sr) + t));
        const int tail = width - (nvec << 4);
        if (t < tail) dr[(nvec << 4) + t] = sr[(nvec << 4) + t];
      } else {
        for (int i = t * 16; i < min(width, t * 16 + 16); ++i) dr[i] = sr[i];
      }
    }
  }
}

// Sum over a frame of (byte+1) * (1 + j mod 65521), j the byte's index in the frame.
// The weighted sum of one aligned 16-byte vector whose first byte has weight index k:
//   no wrap inside the vector:  sum (b_i + 1)(1 + k + i) = (1 + k)(sum b_i + 16) + (sum i*b_i + 120)
// with both byte sums from four-way dot products.
__device__ __forceinline__ unsigned long long checksum_vec(const uint4 q, uint32_t k) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
  if (k + 15u < 65521u) {
    uint32_t s1 = 16u, s2 = 120u;
    s1 = __dp4a(w[0], 0x01010101u, s1);
    s1 = __dp4a(w[1], 0x01010101u, s1);
    s1 = __dp4a(w[2], 0x01010101u, s1);
    s1 = __dp4a(w[3], 0x01010101u, s1);
    s2 = __dp4a(w[0], 0x03020100u, s2);
    s2 = __dp4a(w[1], 0x07060504u, s2);
    s2 = __dp4a(w[2], 0x0B0A0908u, s2);
    s2 = __dp4a(w[3], 0x0F0E0D0Cu, s2);
    return (unsigned long long)(1u + k) * s1 + s2;
  }
  unsigned long long acc = 0;  // the weight wraps inside these 16 bytes
#pragma unroll
  for (int b = 0; b < 16; ++b) {
    acc += (unsigned long long)(((w[b >> 2] >> (8 * (b & 3))) & 255u) + 1u) * (1u + k);
    k = k + 1 == 65521u ? 0u : k + 1;
  }
  return acc;
}

constexpr int kChecksumUnroll = 4;
__global__ void __launch_bounds__(256) checksum_kernel(const uint8_t* src, long long frame_bytes,
                                                       unsigned long long* out) {
  const int n = blockIdx.y;
  const uint8_t* f = src + (long long)n * frame_bytes;
  unsigned long long acc = 0;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const bool vec = (((uintptr_t)f) & 15) == 0;
  const long long nvec = vec ? frame_bytes >> 4 : 0;
  const uint4* fv = reinterpret_cast<const uint4*>(f);
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  // weight index of vector i, advanced by the stride without a division per vector
  uint32_t k = (uint32_t)((i << 4) % 65521);
  const uint32_t kstep = (uint32_t)((stride << 4) % 65521);
  for (; i + (kChecksumUnroll - 1) * stride < nvec; i += kChecksumUnroll * stride) {
    uint4 q[kChecksumUnroll];
#pragma unroll
    for (int u = 0; u < kChecksumUnroll; ++u) q[u] = __ldcs(fv + i + u * stride);
#pragma unroll
    for (int u = 0; u < kChecksumUnroll; ++u) {
      acc += checksum_vec(q[u], k);
      k += kstep;
      k = k >= 65521u ? k - 65521u : k;
    }
  }
  for (; i < nvec; i += stride) {
    acc += checksum_vec(__ldcs(fv + i), k);
    k += kstep;
    k = k >= 65521u ? k - 65521u : k;
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
    for (int i2 = 0; i2 < 8; ++i2) s += part[i2];
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
    dim3 grid((per_row + 127) / 128, (h2 + kGatherRows - 1) / kGatherRows, nn);
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

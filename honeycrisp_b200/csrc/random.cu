// Device-side input generation bit-compatible with Honeycrisp's CPU generator: Philox-4x32-10
// keyed by the 64-bit seed, counter = (offset, 0), four 32-bit words per counter value
// (Sources/Honeycrisp/BackendCPU.swift:177-199).
//   uniform: word -> Float(Double(word) / Double(0xffffffff)), four values per counter; the
//            reference's loop runs `stride(from: 0, through: count, by: 4)` and therefore
//            consumes count/4 + 1 counter values (BackendCPU.swift:89-99);
//   normal : Box-Muller on word pairs in Float arithmetic, two counters' worth of pairs ->
//            four values per counter; `stride(from: 0, through: count, by: 2)` consumes
//            count/2 + 1 counter values and every counter's four outputs overwrite positions
//            i..i+3 of the loop index i, so consecutive counters overlap by two (:100-121).
// float16 results are the Float values narrowed once (writeBuffer).
#include "common.cuh"

namespace hc {
namespace {

__device__ __forceinline__ void philox4x32_10(unsigned long long seed, unsigned long long offset, uint32_t (&c)[4]) {
  c[0] = (uint32_t)(offset & 0xffffffffull);
  c[1] = (uint32_t)(offset >> 32);
  c[2] = 0;
  c[3] = 0;
  uint32_t k0 = (uint32_t)(seed & 0xffffffffull), k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; r++) {
    const uint32_t p0 = c[0], p2 = c[2];
    c[0] = __umulhi(0xCD9E8D57u, p2) ^ c[1] ^ k0;
    c[2] = __umulhi(0xD2511F53u, p0) ^ c[3] ^ k1;
    c[1] = 0xCD9E8D57u * p2;
    c[3] = 0xD2511F53u * p0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}

template <typename T> __device__ __forceinline__ T narrow(float v);
template <> __device__ __forceinline__ float narrow<float>(float v) { return v; }
template <> __device__ __forceinline__ __half narrow<__half>(float v) { return __float2half_rn(v); }

template <typename T>
__global__ void uniform_kernel(unsigned long long seed, unsigned long long offset, int64_t count, T* __restrict__ out) {
  const int64_t groups = (count + 3) / 4;
  for (int64_t g = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; g < groups; g += (int64_t)gridDim.x * blockDim.x) {
    uint32_t c[4];
    philox4x32_10(seed, offset + (unsigned long long)g, c);
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int64_t i = g * 4 + j;
      if (i < count) out[i] = narrow<T>((float)((double)c[j] / 4294967295.0));
    }
  }
}

// Output i comes from the counter of loop index 2*floor(i/2) when that index exists in the
// reference's loop, i.e. the LAST writer of position i: loop index s (even) writes s..s+3, so
// position i is written by s = i - (i % 2) - 2 (its third/fourth output) and then overwritten by
// s = i - (i % 2) (its first/second output).  The final value is the latter.
template <typename T>
__global__ void normal_kernel(unsigned long long seed, unsigned long long offset, int64_t count, T* __restrict__ out) {
  const int64_t pairs = (count + 1) / 2;
  for (int64_t g = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; g < pairs; g += (int64_t)gridDim.x * blockDim.x) {
    uint32_t c[4];
    philox4x32_10(seed, offset + (unsigned long long)g, c);
    const float u1 = fmaxf(1e-5f, (float)c[0] / 4294967296.0f);   // Float(0xffffffff) rounds to 2^32
    const float u2 = (float)c[1] / 4294967296.0f;
    const float r = sqrtf(-2.0f * logf(u1));
    const float phi = 2.0f * 3.14159274101257324f * u2;
    const int64_t i = g * 2;
    out[i] = narrow<T>(r * cosf(phi));
    if (i + 1 < count) out[i + 1] = narrow<T>(r * sinf(phi));
  }
}

int grid_for(int64_t n, int threads) {
  int64_t b = (n + threads - 1) / threads;
  return (int)(b > 148 * 16 ? 148 * 16 : (b < 1 ? 1 : b));
}

}  // namespace

cudaError_t launch_random(int normal, hc_dtype dtype, unsigned long long seed, unsigned long long offset, int64_t count,
                          void* out, cudaStream_t stream) {
  if (count <= 0) return cudaSuccess;
  const int threads = 256;
  if (!normal) {
    const int grid = grid_for((count + 3) / 4, threads);
    if (dtype == HC_F16) uniform_kernel<__half><<<grid, threads, 0, stream>>>(seed, offset, count, (__half*)out);
    else uniform_kernel<float><<<grid, threads, 0, stream>>>(seed, offset, count, (float*)out);
  } else {
    const int grid = grid_for((count + 1) / 2, threads);
    if (dtype == HC_F16) normal_kernel<__half><<<grid, threads, 0, stream>>>(seed, offset, count, (__half*)out);
    else normal_kernel<float><<<grid, threads, 0, stream>>>(seed, offset, count, (float*)out);
  }
  return cudaGetLastError();
}

}  // namespace hc

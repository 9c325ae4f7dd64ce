// The small operations either side of a Linear layer's products, so that its forward and
// backward pass stay on the device: the bias gradient (a column sum), dtype casts, and the
// elementwise add of gradient accumulation.  All three are bound by HBM bandwidth.
//
// They restate the reference CPU backend exactly:
//   reduce(.sum) over the leading axis: one float accumulator per column, rows in ascending
//     order, narrowed once (Sources/Honeycrisp/BackendCPU.swift:808-827);
//   cast: widen/narrow through Float (BackendCPU.swift:2018-2058);
//   binaryOp(.add) on equal shapes: widen, add, narrow (BackendCPU.swift:295-303).
#include "common.cuh"

namespace hc {
namespace {

template <typename T> __device__ __forceinline__ float widen(T v);
template <> __device__ __forceinline__ float widen<float>(float v) { return v; }
template <> __device__ __forceinline__ float widen<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T narrow(float v);
template <> __device__ __forceinline__ float narrow<float>(float v) { return v; }
template <> __device__ __forceinline__ __half narrow<__half>(float v) { return __float2half_rn(v); }

// One thread per column (or per pair of float16 columns) walks the rows in order - the
// reference's summation order - with 32 loads in flight; consecutive threads read consecutive
// columns, so every row is read coalesced.
template <typename T>
__global__ void __launch_bounds__(128) column_sum_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t rows,
                                                         int64_t cols) {
  const int64_t c = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float sum = 0.0f;
  int64_t r = 0;
  for (; r + 32 <= rows; r += 32) {
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = widen<T>(x[(r + i) * cols + c]);
#pragma unroll
    for (int i = 0; i < 32; i++) sum = __fadd_rn(sum, v[i]);
  }
  for (; r < rows; r++) sum = __fadd_rn(sum, widen<T>(x[r * cols + c]));
  out[c] = narrow<T>(sum);
}

// float16 with an even number of columns: two columns per thread through 4-byte loads.
__global__ void __launch_bounds__(128) column_sum_half2_kernel(const __half2* __restrict__ x, __half2* __restrict__ out,
                                                               int64_t rows, int64_t col_pairs) {
  const int64_t c = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (c >= col_pairs) return;
  float s0 = 0.0f, s1 = 0.0f;
  int64_t r = 0;
  for (; r + 32 <= rows; r += 32) {
    __half2 v[32];
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = x[(r + i) * col_pairs + c];
#pragma unroll
    for (int i = 0; i < 32; i++) {
      const float2 f = __half22float2(v[i]);
      s0 = __fadd_rn(s0, f.x);
      s1 = __fadd_rn(s1, f.y);
    }
  }
  for (; r < rows; r++) {
    const float2 f = __half22float2(x[r * col_pairs + c]);
    s0 = __fadd_rn(s0, f.x);
    s1 = __fadd_rn(s1, f.y);
  }
  out[c] = __floats2half2_rn(s0, s1);
}

// The same sum for tall inputs, fed through shared memory.  One thread per column keeps the
// reference's order but leaves too few loads in flight to fill HBM (8192 threads x 32 loads for
// 16384 float16 columns: about 1 TB/s).  Here a CTA owns a strip of kStripBytes of every row; all
// 256 threads stream the strip through a ring of four 128-row stages with 16-byte asynchronous
// copies, and the strip's kStripBytes / 4 summing threads walk each stage top to bottom: the same
// additions in the same order, one accumulator per column, narrowed once.
template <typename T, int kStripBytes>
__global__ void __launch_bounds__(256) column_sum_staged_kernel(const T* __restrict__ x, T* __restrict__ out,
                                                                int64_t rows, int64_t cols) {
  constexpr int ROWS = 128, STAGES = 4, CHUNKS = kStripBytes / 16, PER_STAGE = ROWS * CHUNKS;
  extern __shared__ __align__(16) unsigned char ring[];   // [STAGES][ROWS][kStripBytes]
  const int tid = threadIdx.x;
  const int64_t row_bytes = cols * (int64_t)sizeof(T);
  const int64_t col0b = (int64_t)blockIdx.x * kStripBytes;
  const int valid_chunks = (int)min((int64_t)CHUNKS, (row_bytes - col0b + 15) / 16);
  const unsigned char* src = (const unsigned char*)x + col0b;
  const int64_t blocks = (rows + ROWS - 1) / ROWS;

  auto load = [&](int64_t rb) {
    if (rb < blocks) {
      unsigned char* dst = ring + (size_t)(rb % STAGES) * ROWS * kStripBytes;
      for (int idx = tid; idx < PER_STAGE; idx += 256) {
        const int r = idx / CHUNKS, ch = idx % CHUNKS;
        const int64_t grow = rb * ROWS + r;
        if (grow < rows && ch < valid_chunks) {
          const unsigned int d = (unsigned int)__cvta_generic_to_shared(dst + r * kStripBytes + ch * 16);
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src + grow * row_bytes + ch * 16)
                       : "memory");
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");   // one group per stage, empty past the end
  };

  for (int s = 0; s < STAGES - 1; s++) load(s);
  float s0 = 0.0f, s1 = 0.0f;
  const bool summing = tid < kStripBytes / 4;
  for (int64_t rb = 0; rb < blocks; rb++) {
    asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
    __syncthreads();                 // stage rb has landed for every thread; stage rb - 1 is free
    load(rb + STAGES - 1);
    if (summing) {
      const unsigned char* st = ring + (size_t)(rb % STAGES) * ROWS * kStripBytes + tid * 4;
      const int n = (int)min((int64_t)ROWS, rows - rb * ROWS);
      // The additions of one column form a dependent chain (that is the reference's order); the
      // shared-memory reads do not, so a full stage is unrolled far enough to keep them ahead.
      if (sizeof(T) == 2) {
        if (n == ROWS) {
#pragma unroll 32
          for (int r = 0; r < ROWS; r++) {
            const float2 f = __half22float2(*(const __half2*)(st + r * kStripBytes));
            s0 = __fadd_rn(s0, f.x);
            s1 = __fadd_rn(s1, f.y);
          }
        } else {
          for (int r = 0; r < n; r++) {
            const float2 f = __half22float2(*(const __half2*)(st + r * kStripBytes));
            s0 = __fadd_rn(s0, f.x);
            s1 = __fadd_rn(s1, f.y);
          }
        }
      } else {
        if (n == ROWS) {
#pragma unroll 32
          for (int r = 0; r < ROWS; r++) s0 = __fadd_rn(s0, *(const float*)(st + r * kStripBytes));
        } else {
          for (int r = 0; r < n; r++) s0 = __fadd_rn(s0, *(const float*)(st + r * kStripBytes));
        }
      }
    }
  }
  if (summing) {
    const int64_t byte = col0b + tid * 4;
    if (byte < row_bytes) {
      if (sizeof(T) == 2) *(__half2*)((unsigned char*)out + byte) = __floats2half2_rn(s0, s1);
      else *(float*)((unsigned char*)out + byte) = s0;
    }
  }
}

template <typename T, int kStripBytes>
cudaError_t launch_column_sum_staged(const T* x, T* out, int64_t rows, int64_t cols, cudaStream_t stream) {
  constexpr size_t smem = 4 * 128 * (size_t)kStripBytes;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(column_sum_staged_kernel<T, kStripBytes>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int64_t strips = (cols * (int64_t)sizeof(T) + kStripBytes - 1) / kStripBytes;
  if (strips > 2147483647LL) return cudaErrorInvalidValue;
  column_sum_staged_kernel<T, kStripBytes><<<(unsigned)strips, 256, smem, stream>>>(x, out, rows, cols);
  return cudaGetLastError();
}

template <typename T>
cudaError_t launch_column_sum_staged_any(const T* x, T* out, int64_t rows, int64_t cols, cudaStream_t stream) {
  // Strips as wide as a cache line when that still gives every SM two CTAs, narrower otherwise.
  const int64_t row_bytes = cols * (int64_t)sizeof(T);
  if (row_bytes >= 128 * 296) return launch_column_sum_staged<T, 128>(x, out, rows, cols, stream);
  if (row_bytes >= 64 * 296) return launch_column_sum_staged<T, 64>(x, out, rows, cols, stream);
  return launch_column_sum_staged<T, 32>(x, out, rows, cols, stream);
}

template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ x, TO* __restrict__ out, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = narrow<TO>(widen<TI>(x[i]));
}

template <typename T>
__global__ void add_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = narrow<T>(__fadd_rn(widen<T>(a[i]), widen<T>(b[i])));
}

// Eight elements per thread through 16-byte accesses (the scalar kernels above move 2-4 bytes
// per access and reach a fraction of the HBM bandwidth); same per-element arithmetic.
template <typename T> struct Vec8;
template <> struct Vec8<__half> {
  uint4 raw;
  __device__ static Vec8 load(const __half* p) { Vec8 v; v.raw = __ldg((const uint4*)p); return v; }
  __device__ void store(__half* p) const { *(uint4*)p = raw; }
  __device__ float get(int i) const { return __half2float(((const __half*)&raw)[i]); }
  __device__ void set(int i, float f) { ((__half*)&raw)[i] = __float2half_rn(f); }
};
template <> struct Vec8<float> {
  alignas(16) float v[8];
  __device__ static Vec8 load(const float* p) {
    Vec8 r;
    *(float4*)&r.v[0] = __ldg((const float4*)p);
    *(float4*)&r.v[4] = __ldg((const float4*)p + 1);
    return r;
  }
  __device__ void store(float* p) const { *(float4*)p = *(const float4*)&v[0]; *((float4*)p + 1) = *(const float4*)&v[4]; }
  __device__ float get(int i) const { return v[i]; }
  __device__ void set(int i, float f) { v[i] = f; }
};

template <typename TI, typename TO>
__global__ void __launch_bounds__(256) cast_vec8_kernel(const TI* __restrict__ x, TO* __restrict__ out, int64_t groups) {
  for (int64_t g = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; g < groups; g += (int64_t)gridDim.x * blockDim.x) {
    const Vec8<TI> v = Vec8<TI>::load(x + g * 8);
    Vec8<TO> o;
#pragma unroll
    for (int i = 0; i < 8; i++) o.set(i, v.get(i));
    o.store(out + g * 8);
  }
}

// Widening cast: four elements per thread, so that every store instruction of a warp writes 512
// contiguous bytes (with eight per thread a lane's two 16-byte stores each cover half of a
// 32-byte sector).
__global__ void __launch_bounds__(256) cast_h2f_vec4_kernel(const __half* __restrict__ x, float* __restrict__ out,
                                                            int64_t quads) {
  for (int64_t g = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; g < quads; g += (int64_t)gridDim.x * blockDim.x) {
    const uint2 raw = __ldg((const uint2*)(x + g * 4));
    const float2 a = __half22float2(*(const __half2*)&raw.x), b = __half22float2(*(const __half2*)&raw.y);
    *(float4*)(out + g * 4) = make_float4(a.x, a.y, b.x, b.y);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) add_vec8_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out,
                                                       int64_t groups) {
  for (int64_t g = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; g < groups; g += (int64_t)gridDim.x * blockDim.x) {
    const Vec8<T> va = Vec8<T>::load(a + g * 8), vb = Vec8<T>::load(b + g * 8);
    Vec8<T> o;
#pragma unroll
    for (int i = 0; i < 8; i++) o.set(i, __fadd_rn(va.get(i), vb.get(i)));
    o.store(out + g * 8);
  }
}

// 2-byte elements: 64 x 64 tiles moved with 4-byte accesses on both sides (a warp reads and
// writes 128 contiguous bytes); rows and columns even, buffers 4-byte aligned.
__global__ void __launch_bounds__(256) transpose_half_kernel(const __half* __restrict__ in, __half* __restrict__ out,
                                                             int64_t rows, int64_t cols) {
  __shared__ __half tile[64][66];
  const int64_t mat = blockIdx.z;
  in += mat * rows * cols;
  out += mat * rows * cols;
  const int64_t c0 = (int64_t)blockIdx.x * 64, r0 = (int64_t)blockIdx.y * 64;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;   // 8 warps
  for (int j = warp; j < 64; j += 8) {
    const int64_t r = r0 + j, c = c0 + 2 * lane;
    if (r < rows && c < cols) *(__half2*)&tile[j][2 * lane] = *(const __half2*)(in + r * cols + c);
  }
  __syncthreads();
  for (int j = warp; j < 64; j += 8) {
    const int64_t c = c0 + j, r = r0 + 2 * lane;   // out is [cols, rows]
    if (c < cols && r < rows) *(__half2*)(out + c * rows + r) = __halves2half2(tile[2 * lane][j], tile[2 * lane + 1][j]);
  }
}

// Materialised transpose of `batch` dense [rows, cols] matrices through 32 x 33 shared tiles.
template <typename T>
__global__ void transpose_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t rows, int64_t cols) {
  __shared__ T tile[32][33];
  const int64_t mat = blockIdx.z;
  in += mat * rows * cols;
  out += mat * rows * cols;
  const int64_t c0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int64_t r = r0 + j, c = c0 + threadIdx.x;
    if (r < rows && c < cols) tile[j][threadIdx.x] = in[r * cols + c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int64_t c = c0 + j, r = r0 + threadIdx.x;   // out is [cols, rows]
    if (r < rows && c < cols) out[c * rows + r] = tile[threadIdx.x][j];
  }
}

int grid_for(int64_t n, int threads) {
  int64_t b = (n + threads - 1) / threads;
  return (int)(b > 148 * 16 ? 148 * 16 : (b < 1 ? 1 : b));
}

}  // namespace

cudaError_t launch_column_sum(hc_dtype dtype, const void* x, void* out, int64_t rows, int64_t cols, cudaStream_t stream) {
  if (cols <= 0) return cudaSuccess;
  // Tall inputs whose rows are 16-byte multiples go through the shared-memory ring.
  const int64_t eb = dtype == HC_F16 ? 2 : 4;
  if (rows >= 512 && (cols * eb) % 16 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 3) == 0) {
    if (dtype == HC_F16) return launch_column_sum_staged_any<__half>((const __half*)x, (__half*)out, rows, cols, stream);
    return launch_column_sum_staged_any<float>((const float*)x, (float*)out, rows, cols, stream);
  }
  const int threads = 128;
  const int64_t blocks = (cols + threads - 1) / threads;
  if (blocks > 2147483647LL) return cudaErrorInvalidValue;
  if (dtype == HC_F16 && cols % 2 == 0 && (((uintptr_t)x | (uintptr_t)out) & 3) == 0) {
    const int64_t pairs = cols / 2, pb = (pairs + threads - 1) / threads;
    column_sum_half2_kernel<<<(unsigned)pb, threads, 0, stream>>>((const __half2*)x, (__half2*)out, rows, pairs);
  } else if (dtype == HC_F16)
    column_sum_kernel<__half><<<(unsigned)blocks, threads, 0, stream>>>((const __half*)x, (__half*)out, rows, cols);
  else
    column_sum_kernel<float><<<(unsigned)blocks, threads, 0, stream>>>((const float*)x, (float*)out, rows, cols);
  return cudaGetLastError();
}

cudaError_t launch_transpose(hc_dtype dtype, int64_t batch, const void* in, void* out, int64_t rows, int64_t cols,
                             cudaStream_t stream) {
  if (batch <= 0 || rows <= 0 || cols <= 0) return cudaSuccess;
  const int64_t gx = (cols + 31) / 32, gy = (rows + 31) / 32;
  if (gy > 65535 || batch > 65535 || gx > 2147483647LL) return cudaErrorInvalidValue;
  if (dtype == HC_F16 && rows % 2 == 0 && cols % 2 == 0 && ((((uintptr_t)in | (uintptr_t)out) & 3) == 0)) {
    const int64_t hx = (cols + 63) / 64, hy = (rows + 63) / 64;
    if (hy <= 65535) {
      transpose_half_kernel<<<dim3((unsigned)hx, (unsigned)hy, (unsigned)batch), 256, 0, stream>>>(
          (const __half*)in, (__half*)out, rows, cols);
      return cudaGetLastError();
    }
  }
  dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)batch), block(32, 8);
  if (dtype == HC_F16)
    transpose_kernel<__half><<<grid, block, 0, stream>>>((const __half*)in, (__half*)out, rows, cols);
  else
    transpose_kernel<float><<<grid, block, 0, stream>>>((const float*)in, (float*)out, rows, cols);
  return cudaGetLastError();
}

cudaError_t launch_cast(hc_dtype from, hc_dtype to, const void* x, void* out, int64_t count, cudaStream_t stream) {
  if (count <= 0) return cudaSuccess;
  const int threads = 256;
  // Bulk in groups of eight through 16-byte accesses, the remainder through the scalar kernel.
  const int64_t groups = ((((uintptr_t)x | (uintptr_t)out) & 15) == 0) ? count / 8 : 0;
  if (groups > 0) {
    const int vg = grid_for(groups, threads);
    if (from == HC_F16 && to == HC_F32)
      cast_h2f_vec4_kernel<<<grid_for(groups * 2, threads), threads, 0, stream>>>((const __half*)x, (float*)out, groups * 2);
    else if (from == HC_F32 && to == HC_F16)
      cast_vec8_kernel<float, __half><<<vg, threads, 0, stream>>>((const float*)x, (__half*)out, groups);
    else if (from == HC_F16)
      cast_vec8_kernel<__half, __half><<<vg, threads, 0, stream>>>((const __half*)x, (__half*)out, groups);
    else
      cast_vec8_kernel<float, float><<<vg, threads, 0, stream>>>((const float*)x, (float*)out, groups);
    const int64_t done = groups * 8;
    if (done == count) return cudaGetLastError();
    const size_t in_b = from == HC_F16 ? 2 : 4, out_b = to == HC_F16 ? 2 : 4;
    x = (const char*)x + done * in_b;
    out = (char*)out + done * out_b;
    count -= done;
  }
  const int grid = grid_for(count, threads);
  if (from == HC_F16 && to == HC_F32)
    cast_kernel<__half, float><<<grid, threads, 0, stream>>>((const __half*)x, (float*)out, count);
  else if (from == HC_F32 && to == HC_F16)
    cast_kernel<float, __half><<<grid, threads, 0, stream>>>((const float*)x, (__half*)out, count);
  else if (from == HC_F16)
    cast_kernel<__half, __half><<<grid, threads, 0, stream>>>((const __half*)x, (__half*)out, count);
  else
    cast_kernel<float, float><<<grid, threads, 0, stream>>>((const float*)x, (float*)out, count);
  return cudaGetLastError();
}

cudaError_t launch_add(hc_dtype dtype, const void* a, const void* b, void* out, int64_t count, cudaStream_t stream) {
  if (count <= 0) return cudaSuccess;
  const int threads = 256;
  const int64_t groups = ((((uintptr_t)a | (uintptr_t)b | (uintptr_t)out) & 15) == 0) ? count / 8 : 0;
  if (groups > 0) {
    const int vg = grid_for(groups, threads);
    if (dtype == HC_F16)
      add_vec8_kernel<__half><<<vg, threads, 0, stream>>>((const __half*)a, (const __half*)b, (__half*)out, groups);
    else
      add_vec8_kernel<float><<<vg, threads, 0, stream>>>((const float*)a, (const float*)b, (float*)out, groups);
    const int64_t done = groups * 8;
    if (done == count) return cudaGetLastError();
    const size_t eb = dtype == HC_F16 ? 2 : 4;
    a = (const char*)a + done * eb; b = (const char*)b + done * eb; out = (char*)out + done * eb;
    count -= done;
  }
  const int grid = grid_for(count, threads);
  if (dtype == HC_F16)
    add_kernel<__half><<<grid, threads, 0, stream>>>((const __half*)a, (const __half*)b, (__half*)out, count);
  else
    add_kernel<float><<<grid, threads, 0, stream>>>((const float*)a, (const float*)b, (float*)out, count);
  return cudaGetLastError();
}

// Backend.constant: every element = the float value narrowed once to the element type.  Whole
// 16-byte groups are written with one store each; the ragged ends (a misaligned start, a count that
// is not a multiple of the group) one element at a time.
template <typename T>
__global__ void fill_kernel(T* __restrict__ out, T value, uint4 pattern, int64_t head, int64_t groups, int64_t n) {
  constexpr int kPer = 16 / (int)sizeof(T);
  const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x, step = (int64_t)gridDim.x * blockDim.x;
  uint4* body = (uint4*)(out + head);
  for (int64_t i = tid; i < groups; i += step) body[i] = pattern;
  for (int64_t i = tid; i < head; i += step) out[i] = value;
  for (int64_t i = head + groups * kPer + tid; i < n; i += step) out[i] = value;
}

template <typename T>
static cudaError_t fill_typed(T* out, T value, int64_t count, cudaStream_t stream) {
  constexpr int64_t kPer = 16 / (int64_t)sizeof(T);
  uint32_t word = 0;
  if (sizeof(T) == 2) {
    uint16_t bits;
    memcpy(&bits, &value, 2);
    word = (uint32_t)bits | ((uint32_t)bits << 16);
  } else {
    memcpy(&word, &value, 4);
  }
  const uint4 pattern = make_uint4(word, word, word, word);
  // elements before the first 16-byte boundary (the pointer is at least element-aligned)
  int64_t head = (int64_t)(((16 - ((uintptr_t)out & 15)) & 15) / sizeof(T));
  if (head > count) head = count;
  const int64_t groups = (count - head) / kPer;
  const int threads = 256;
  const int grid = grid_for(groups > 0 ? groups : count, threads);
  fill_kernel<T><<<grid, threads, 0, stream>>>(out, value, pattern, head, groups, count);
  return cudaGetLastError();
}

cudaError_t launch_constant(hc_dtype dtype, float value, void* out, int64_t count, cudaStream_t stream) {
  if (count <= 0) return cudaSuccess;
  if (dtype == HC_F16) return fill_typed<__half>((__half*)out, __float2half_rn(value), count, stream);
  return fill_typed<float>((float*)out, value, count, stream);
}

}  // namespace hc

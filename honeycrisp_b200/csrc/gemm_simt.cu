// CUDA-core matrix product: the kernel that accepts every shape and alignment.
//
// It serves three purposes:
//   * the products TMA cannot describe (leading dimensions that are not 16-byte multiples,
//     e.g. the reference's own [2,3]x[3,4] and [3,1] test shapes,
//     Sources/HCTestUtils/BackendTests.swift:684-783);
//   * the GPU-side cross-check of the tensor-core kernels at sizes no CPU loop reaches;
//   * in EXACT mode, a bit-for-bit restatement of the reference CPU loop
//     (Sources/Honeycrisp/BackendCPU.swift:1290-1300: `acc = acc + a*b`, k ascending, one
//     float32 accumulator per output, two roundings per step).  For float16 operands the
//     product of two halves is exact in float32, so the fused mode is bit-identical too.
//
// Layout: a 128x128 output tile per 256-thread block, 8x8 outputs per thread, k in slabs of
// 8 through shared memory.  Each output is accumulated by exactly one thread in ascending k,
// which is what makes the EXACT claim hold for any tile decomposition.
#include "common.cuh"

namespace hc {
namespace {

constexpr int BM = 128, BN = 128, BK = 8, TM = 8, TN = 8, THREADS = 256;

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }

template <typename T, bool EXACT>
__global__ void __launch_bounds__(THREADS)
simt_gemm_kernel(const T* __restrict__ A, const T* __restrict__ B, T* __restrict__ C, const T* __restrict__ bias,
                 int64_t M, int64_t N, int64_t K,
                 int64_t a_rs, int64_t a_cs,   // A(m,k) = A[m*a_rs + k*a_cs]
                 int64_t b_rs, int64_t b_cs,   // B(k,n) = B[k*b_rs + n*b_cs]
                 int64_t ldc, int64_t strideA, int64_t strideB, int64_t strideC,
                 int tiles_n) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];

  const int64_t mat = blockIdx.y;
  const int64_t tile_m = blockIdx.x / tiles_n, tile_n = blockIdx.x % tiles_n;
  const int64_t m0 = tile_m * BM, n0 = tile_n * BN;
  A += mat * strideA;
  B += mat * strideB;
  C += mat * strideC;

  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;  // thread owns rows ty*8.., cols tx*8..

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; i++)
#pragma unroll
    for (int j = 0; j < TN; j++) acc[i][j] = 0.0f;

  // Loading order follows the contiguous index of each operand so that a warp reads
  // consecutive addresses whichever way the operand is stored.
  const bool a_k_contig = (a_cs == 1);
  const bool b_n_contig = (b_cs == 1);

  for (int64_t k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int it = 0; it < (BM * BK) / THREADS; it++) {
      int idx = tid + it * THREADS;
      int mm, kk;
      if (a_k_contig) { kk = idx % BK; mm = idx / BK; } else { mm = idx % BM; kk = idx / BM; }
      int64_t gm = m0 + mm, gk = k0 + kk;
      float v = 0.0f;
      if (gm < M && gk < K) v = to_float<T>(A[gm * a_rs + gk * a_cs]);
      As[kk][mm] = v;
    }
#pragma unroll
    for (int it = 0; it < (BN * BK) / THREADS; it++) {
      int idx = tid + it * THREADS;
      int nn, kk;
      if (b_n_contig) { nn = idx % BN; kk = idx / BN; } else { kk = idx % BK; nn = idx / BK; }
      int64_t gn = n0 + nn, gk = k0 + kk;
      float v = 0.0f;
      if (gn < N && gk < K) v = to_float<T>(B[gk * b_rs + gn * b_cs]);
      Bs[kk][nn] = v;
    }
    __syncthreads();

    // Padding k beyond K contributes a*0 + acc: exact in both modes (acc + 0 == acc; the
    // only representable difference, -0 + 0, cannot occur because acc starts at +0).
#pragma unroll
    for (int kk = 0; kk < BK; kk++) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; i++) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; j++) b[j] = Bs[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) {
          if (EXACT) {
            acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(a[i], b[j]));
          } else {
            acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
          }
        }
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < TM; i++) {
    int64_t gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; j++) {
      int64_t gn = n0 + tx * TN + j;
      if (gn < N) {
        T r = from_float<T>(acc[i][j]);
        // Linear's bias: a second operation on the rounded product (widen, add, narrow).
        if (bias) r = from_float<T>(__fadd_rn(to_float<T>(r), to_float<T>(bias[gn])));
        C[gm * ldc + gn] = r;
      }
    }
  }
}

template <typename T>
cudaError_t launch_typed(const GemmProblem& p, bool exact, cudaStream_t stream, LaunchRecord* rec) {
  const int64_t tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN;
  const int64_t a_rs = p.a_mn_major ? 1 : p.lda, a_cs = p.a_mn_major ? p.lda : 1;
  const int64_t b_rs = p.b_mn_major ? p.ldb : 1, b_cs = p.b_mn_major ? 1 : p.ldb;
  if (rec) {
    rec->kernel = exact ? HC_KERNEL_SIMT_EXACT : HC_KERNEL_SIMT;
    rec->tile_m = BM; rec->tile_n = BN; rec->tile_k = BK; rec->stages = 1;
    rec->block = THREADS; rec->tiles = tiles_m * tiles_n * p.batch; rec->scratch_bytes = 0;
    rec->launches = 0;
  }
  // gridDim.y is limited to 65535: walk the batch in slices.
  for (int64_t b0 = 0; b0 < p.batch; b0 += 65535) {
    int64_t nb = p.batch - b0 < 65535 ? p.batch - b0 : 65535;
    dim3 grid((unsigned)(tiles_m * tiles_n), (unsigned)nb);
    const T* A = (const T*)p.A + b0 * p.strideA;
    const T* B = (const T*)p.B + b0 * p.strideB;
    T* C = (T*)p.C + b0 * p.strideC;
    if (exact) {
      simt_gemm_kernel<T, true><<<grid, THREADS, 0, stream>>>(
          A, B, C, (const T*)p.bias, p.M, p.N, p.K, a_rs, a_cs, b_rs, b_cs, p.ldc, p.strideA, p.strideB, p.strideC,
          (int)tiles_n);
    } else {
      simt_gemm_kernel<T, false><<<grid, THREADS, 0, stream>>>(
          A, B, C, (const T*)p.bias, p.M, p.N, p.K, a_rs, a_cs, b_rs, b_cs, p.ldc, p.strideA, p.strideB, p.strideC,
          (int)tiles_n);
    }
    if (rec) { rec->launches++; rec->grid = (int)(tiles_m * tiles_n); }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

}  // namespace

cudaError_t launch_simt(const GemmProblem& p, bool exact, cudaStream_t stream, LaunchRecord* rec) {
  if (p.M <= 0 || p.N <= 0 || p.batch <= 0) return cudaSuccess;  // nothing to write
  if ((p.M + BM - 1) / BM * ((p.N + BN - 1) / BN) > 2147483647LL) return cudaErrorInvalidValue;
  if (p.dtype == HC_F16) return launch_typed<__half>(p, exact, stream, rec);
  return launch_typed<float>(p, exact, stream, rec);
}

}  // namespace hc

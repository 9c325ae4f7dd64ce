// Shared declarations of libhccuda's translation units.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stddef.h>

#include "../../include/hc_cuda.h"

namespace hc {

// A matrix product after the reference's three flags have been folded away.
//
// Backend.matmul computes transOut(op(a)*op(b)) (Sources/Honeycrisp/Backend.swift:650-658).
// transOut(X*Y) = Y^T * X^T, so a transposed output is the plain product of the swapped
// operands with their flags negated; the reference's GPU backend folds it the same way
// (Sources/Honeycrisp/BackendMPS.swift:2200-2205).  What is left is C[M,N] = A[M,K] * B[K,N]
// with C row-major and each operand either "K-major" (the contracted index is the
// contiguous one) or "MN-major" (the row/column index of the product is contiguous).
struct GemmProblem {
  hc_dtype dtype;
  int64_t batch;
  int64_t M, N, K;
  const void* A;   // K-major: stored [M][lda>=K];  MN-major: stored [K][lda>=M]
  const void* B;   // K-major: stored [N][ldb>=K];  MN-major: stored [K][ldb>=N]
  void* C;         // stored [M][ldc>=N]
  int a_mn_major, b_mn_major;
  int64_t lda, ldb, ldc;              // leading dimensions, elements
  int64_t strideA, strideB, strideC;  // distance between consecutive matrices, elements
  // Optional row vector of N elements (same dtype) added to every row of the product after it has
  // been rounded to the output dtype: the `h + bias` of Linear (Trainable.swift:539-544).
  const void* bias = nullptr;
  // The contraction may not be cut into parts (which needs a float32 work area of
  // parts x batch x M x N): set by callers whose work area has a fixed size.
  bool no_split = false;
  // Rows and columns of the whole product when this problem is a block of it (0: not a block).
  // Tile shape and the cut of the contraction are chosen for the whole product, so that a block
  // computed on its own is bitwise the block of the whole.
  int64_t plan_M = 0, plan_N = 0;
};

// Word in device memory that kernels set when a bounded wait gives up.
enum DeviceStatusBits : unsigned int {
  kDevTimeoutProducer = 1u,
  kDevTimeoutMma = 2u,
  kDevTimeoutEpilogue = 4u,
  kDevTimeoutSelfTest = 8u,
  kDevTimeoutBarrier = 16u,    // a rank of a device group did not arrive at a flag barrier in time
};

struct LaunchRecord {
  int kernel = 0;
  int tile_m = 0, tile_n = 0, tile_k = 0, stages = 0, grid = 0, block = 0;
  int64_t tiles = 0;
  size_t scratch_bytes = 0;
  int launches = 0;
};

// CUDA-core kernel: any shape, any alignment.  exact = separate multiply and add.
cudaError_t launch_simt(const GemmProblem& p, bool exact, cudaStream_t stream, LaunchRecord* rec);

// tcgen05 kernel.  Returns cudaErrorNotSupported when TMA cannot describe the operands
// (misaligned base or leading dimension); the caller then uses the CUDA-core kernel.
// `status_word` is the device status word of the context; `scratch`/`scratch_bytes` is a
// caller-provided work area of at least tc_scratch_bytes(p, sm_count) bytes (float32 split
// operands, repacked float16 operands, partial matrices of a cut contraction).
// `extra_out`: up to 7 more result buffers of the same shape and pitch as p.C (other devices'
// copies, mapped into this process); every result tile is stored to each of them as well.
// `cache` (optional): prepared launches of recent products, owned by the caller's context; a
// repeat of a product then skips planning and tensor-map encoding.
// `private_stream`: the caller vouches that nobody but this library launches kernels on `stream`;
// the operand loads of a product may then start before the previous product has finished, when
// that product cannot have written them.
// `scratch_needed` (optional) receives the work-area bytes the product needs; when the area given
// is smaller the call launches nothing and returns cudaErrorInvalidValue, so that the caller can
// grow the area and call again.
struct TcCache;
TcCache* tc_cache_create();
void tc_cache_destroy(TcCache* c);
void tc_cache_clear(TcCache* c);
cudaError_t launch_tc(const GemmProblem& p, cudaStream_t stream, unsigned int* status_word,
                      void* scratch, size_t scratch_bytes, int sm_count, LaunchRecord* rec,
                      void* const* extra_out = nullptr, int n_extra = 0, TcCache* cache = nullptr,
                      size_t* scratch_needed = nullptr, bool private_stream = false);
bool tc_supported(const GemmProblem& p);
// One-thread kernel whose bounded wait is made to expire after `limit_ns` (self-test).
cudaError_t launch_wait_probe(cudaStream_t stream, unsigned int* status_word, unsigned long long limit_ns);
size_t tc_scratch_bytes(const GemmProblem& p, int sm_count);
// The tiling the tensor-core path would choose for `p` (host arithmetic only).
struct PlanSummary { int tile_m, tile_n, ctas, slabs, parts, slots_per_part; int64_t tiles; size_t ws_bytes; };
PlanSummary tc_describe_plan(const GemmProblem& p, int sm_count);

}  // namespace hc

// Elementwise and reduction helpers around a Linear product (csrc/linear_ops.cu).
namespace hc {
cudaError_t launch_column_sum(hc_dtype dtype, const void* x, void* out, int64_t rows, int64_t cols, cudaStream_t stream);
cudaError_t launch_cast(hc_dtype from, hc_dtype to, const void* x, void* out, int64_t count, cudaStream_t stream);
cudaError_t launch_add(hc_dtype dtype, const void* a, const void* b, void* out, int64_t count, cudaStream_t stream);
cudaError_t launch_constant(hc_dtype dtype, float value, void* out, int64_t count, cudaStream_t stream);
cudaError_t launch_transpose(hc_dtype dtype, int64_t batch, const void* in, void* out, int64_t rows, int64_t cols,
                             cudaStream_t stream);
// Philox-4x32-10 samples as Honeycrisp's CPU generator produces them (csrc/random.cu).
cudaError_t launch_random(int normal, hc_dtype dtype, unsigned long long seed, unsigned long long offset,
                          int64_t count, void* out, cudaStream_t stream);
}  // namespace hc

// Context internals shared between translation units (defined in hc_api.cu).
#include <mutex>
namespace hc {
std::mutex& ctx_mutex(hc_ctx* ctx);
cudaStream_t ctx_stream(hc_ctx* ctx);
unsigned int* ctx_status_word(hc_ctx* ctx);
int ctx_sm_count(hc_ctx* ctx);
int ctx_device(hc_ctx* ctx);
hc_status ctx_fail(hc_ctx* ctx, hc_status s, const char* msg);
void ctx_note_launch(hc_ctx* ctx, const LaunchRecord& rec, int64_t flops);
hc_status ctx_build_problem(hc_ctx* ctx, hc_dtype dtype, int64_t count, const void* a, int trans_a, const void* b,
                            int trans_b, int trans_out, int64_t rows, int64_t inner, int64_t cols, void* out,
                            GemmProblem* p);
// Used by the multi-device code (csrc/hc_group.cu); the caller holds the context's mutex and has
// made the context's device current.
hc_status ctx_device_alloc(hc_ctx* ctx, void** ptr, size_t bytes);   // stream-ordered, from the context's pool
void ctx_device_free(hc_ctx* ctx, void* ptr);
void ctx_count_launches(hc_ctx* ctx, int n);
hc_status ctx_run_batched(hc_ctx* ctx, hc_dtype dtype, int64_t count, const void* a, int trans_a, const void* b,
                          int trans_b, int trans_out, int64_t rows, int64_t inner, int64_t cols, void* out);
// Columns [col_begin, col_begin + col_count) of op(a)*op(b), tensor-core kernel, written to
// `block_out` with row pitch `block_ld` (and to `extra[0..n_extra)`, same layout, when given).
hc_status ctx_run_colblock(hc_ctx* ctx, hc_dtype dtype, const void* a, int trans_a, const void* b, int trans_b,
                           int64_t rows, int64_t inner, int64_t cols, int64_t col_begin, int64_t col_count,
                           void* block_out, int64_t block_ld, void* const* extra, int n_extra);
}  // namespace hc

// C ABI of libhccuda: context, memory, ordering, and dispatch of the matrix products.
// Declarations and the reference interfaces they replace are in include/hc_cuda.h.
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <string>

#include <nvtx3/nvToolsExt.h>

#include "common.cuh"

struct hc_ctx {
  int device = 0;
  cudaStream_t own_stream = nullptr;
  cudaStream_t stream = nullptr;
  std::mutex mu;
  unsigned int* status_word = nullptr;  // device memory
  std::string last_error;
  hc::LaunchRecord last;
  int64_t last_flops = 0;
  int64_t launch_count = 0;
  int sm_count = 0;
  // Work area of the float32 split operands; grown on demand, freed with the context.
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  // Device staging buffers of the host-buffer entry point.
  void* stage[3] = {nullptr, nullptr, nullptr};
  size_t stage_bytes[3] = {0, 0, 0};
  // Pipelined host-buffer products: two slots of staging buffers, copy streams in both
  // directions, and the events that chain copy-in -> product -> copy-out.
  struct HostSlot {
    void* buf[3] = {nullptr, nullptr, nullptr};
    size_t bytes[3] = {0, 0, 0};
    cudaEvent_t in_done = nullptr, product_done = nullptr, out_done = nullptr;
    bool busy = false;
  } slot[2];
  cudaStream_t in_stream = nullptr, out_stream = nullptr;
  int next_slot = 0;
  // The context's own stream-ordered pool.  It keeps up to 8 GiB (HC_POOL_RETAIN_MB) of freed
  // memory instead of returning it to the driver at every synchronisation, as the device's
  // default pool does: a backend that allocates a fresh result for every operation, as the
  // reference's do (BackendMPS.swift:538-540), would otherwise pay a driver allocation per call.
  cudaMemPool_t pool = nullptr;
  // Prepared launches of recent tensor-core products (plan + tensor maps), see gemm_tc.cu.
  hc::TcCache* cache = nullptr;
  // Test hook: the next `fail_allocs` device allocations of this context report failure.
  int fail_allocs = 0;
  // Tracing (off by default): an NVTX range around every product's launches and a pair of events
  // from which hc_last_elapsed_ms reads the product's device time.
  bool tracing = false;
  cudaEvent_t trace_begin = nullptr, trace_end = nullptr;
  bool trace_valid = false;
};

struct hc_event {
  hc_ctx* ctx;     // for waiting (status word); not touched by hc_event_destroy
  int device;      // a marker may be destroyed after its context
  cudaEvent_t ev;
};

namespace {

struct DeviceGuard {
  int prev = -1;
  bool ok = true;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
    if (prev != dev) ok = (cudaSetDevice(dev) == cudaSuccess);
  }
  ~DeviceGuard() {
    int cur = -1;
    if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
  }
};

hc_status fail(hc_ctx* ctx, hc_status s, const std::string& msg) {
  if (ctx) ctx->last_error = msg;
  return s;
}

hc_status cuda_fail(hc_ctx* ctx, cudaError_t e, const char* what) {
  hc_status s = HC_ERR_CUDA;
  if (e == cudaErrorMemoryAllocation) s = HC_ERR_ALLOCATION_FAILED;
  std::string msg = std::string(what) + ": " + cudaGetErrorString(e);
  cudaGetLastError();  // clear the sticky-less error state
  return fail(ctx, s, msg);
}

#define HC_CUDA_TRY(ctx, expr)                                   \
  do {                                                           \
    cudaError_t e__ = (expr);                                    \
    if (e__ != cudaSuccess) return cuda_fail(ctx, e__, #expr);   \
  } while (0)

// Device allocation on behalf of the context: stream-ordered from the context's pool, so that
// neither growing a work area nor a fresh result synchronises the device.  Every allocation the
// library makes goes through here, which is also where the allocation-failure test hook sits.
cudaError_t ctx_malloc(hc_ctx* ctx, void** ptr, size_t bytes, cudaStream_t stream) {
  *ptr = nullptr;
  if (ctx->fail_allocs > 0) {
    ctx->fail_allocs--;
    return cudaErrorMemoryAllocation;
  }
  cudaError_t e = ctx->pool ? cudaMallocFromPoolAsync(ptr, bytes ? bytes : 1, ctx->pool, stream)
                            : cudaMallocAsync(ptr, bytes ? bytes : 1, stream);
  if (e != cudaSuccess) {
    *ptr = nullptr;
    cudaGetLastError();
  }
  return e;
}

// Grow-only device buffer owned by the context and used on `stream` only.  The old buffer is
// freed in stream order: work already enqueued keeps reading it, nothing waits.
hc_status ensure_buffer(hc_ctx* ctx, void** buf, size_t* have, size_t need, cudaStream_t stream) {
  if (need <= *have && *buf) return HC_OK;
  const size_t bytes = need ? need : 1;
  void* fresh = nullptr;
  if (ctx_malloc(ctx, &fresh, bytes, stream) != cudaSuccess) {
    // The old buffer stays: the context is as usable as before the call.
    char msg[96];
    snprintf(msg, sizeof msg, "allocation of %zu bytes failed", bytes);
    return fail(ctx, HC_ERR_ALLOCATION_FAILED, msg);
  }
  if (*buf) {
    if (cudaFreeAsync(*buf, stream) != cudaSuccess) cudaGetLastError();
  }
  *buf = fresh;
  *have = bytes;
  return HC_OK;
}

bool mul_overflows(int64_t a, int64_t b, int64_t* out) { return __builtin_mul_overflow(a, b, out); }

// Folds (trans_a, trans_b, trans_out) into operand major-ness; optionally narrows to a
// column block of op(a)*op(b).
hc_status build_problem(hc_ctx* ctx, hc_dtype dtype, int64_t count, const void* a, int trans_a, const void* b,
                        int trans_b, int trans_out, int64_t rows, int64_t inner, int64_t cols, int64_t col_begin,
                        int64_t col_count, void* out, hc::GemmProblem* p) {
  if (dtype != HC_F16 && dtype != HC_F32)
    return fail(ctx, HC_ERR_NOT_IMPLEMENTED, "matmul: only float16 and float32 are implemented");
  if (count < 0 || rows < 0 || inner < 0 || cols < 0) return fail(ctx, HC_ERR_INVALID_ARGUMENT, "negative dimension");
  if (col_begin < 0 || col_count < 0 || col_begin + col_count > cols)
    return fail(ctx, HC_ERR_INVALID_ARGUMENT, "column block outside the product");
  int64_t t;
  if (mul_overflows(rows, inner, &t) || mul_overflows(t, count, &t) || mul_overflows(inner, cols, &t) ||
      mul_overflows(t, count, &t) || mul_overflows(rows, cols, &t) || mul_overflows(t, count, &t) ||
      mul_overflows(t, 4, &t))
    return fail(ctx, HC_ERR_INVALID_ARGUMENT, "operand size overflows int64");
  const bool empty = (count == 0 || rows == 0 || cols == 0 || col_count == 0);
  if (!empty && (!out || (inner > 0 && (!a || !b)))) return fail(ctx, HC_ERR_INVALID_ARGUMENT, "null operand");
  const int64_t eb = dtype == HC_F16 ? 2 : 4;
  const char* ap = (const char*)a;
  const char* bp = (const char*)b;
  char* cp = (char*)out;
  p->dtype = dtype;
  p->batch = count;
  p->K = inner;
  p->strideC = rows * cols;
  if (!trans_out) {
    // C[rows, cols] = op(a) * op(b); block = columns of C and of op(b).
    p->M = rows; p->N = col_count;
    p->A = ap; p->a_mn_major = trans_a ? 1 : 0; p->lda = trans_a ? rows : inner; p->strideA = rows * inner;
    p->b_mn_major = trans_b ? 0 : 1; p->ldb = trans_b ? inner : cols; p->strideB = inner * cols;
    p->B = bp + (trans_b ? col_begin * inner : col_begin) * eb;
    p->C = cp + col_begin * eb; p->ldc = cols;
    p->plan_M = rows; p->plan_N = cols;
  } else {
    // out[cols, rows] = op(b)^T * op(a)^T; block = rows of out.
    p->M = col_count; p->N = rows;
    p->a_mn_major = trans_b ? 0 : 1; p->lda = trans_b ? inner : cols; p->strideA = inner * cols;
    p->A = bp + (trans_b ? col_begin * inner : col_begin) * eb;
    p->B = ap; p->b_mn_major = trans_a ? 1 : 0; p->ldb = trans_a ? rows : inner; p->strideB = rows * inner;
    p->C = cp + col_begin * rows * eb; p->ldc = rows;
    p->plan_M = cols; p->plan_N = rows;
  }
  return HC_OK;
}

// Shapes below this many multiply-adds are served by the CUDA-core kernel under AUTO: a
// 128 x 128 tensor-core tile would be mostly padding.
constexpr int64_t kAutoTensorMinWork = 64ll * 64 * 64;

// Launches the tensor-core path, growing the context's work area when the product needs more.
cudaError_t launch_tensor(hc_ctx* ctx, const hc::GemmProblem& p, void* const* extra, int n_extra, hc_status* st) {
  *st = HC_OK;
  size_t need = 0;
  const bool private_stream = ctx->stream == ctx->own_stream;
  cudaError_t e = hc::launch_tc(p, ctx->stream, ctx->status_word, ctx->scratch, ctx->scratch_bytes, ctx->sm_count,
                                &ctx->last, extra, n_extra, ctx->cache, &need, private_stream);
  if (e == cudaErrorInvalidValue && need > ctx->scratch_bytes) {
    *st = ensure_buffer(ctx, &ctx->scratch, &ctx->scratch_bytes, need, ctx->stream);
    if (*st != HC_OK) return cudaErrorMemoryAllocation;
    hc::tc_cache_clear(ctx->cache);   // prepared launches point into the old work area
    e = hc::launch_tc(p, ctx->stream, ctx->status_word, ctx->scratch, ctx->scratch_bytes, ctx->sm_count, &ctx->last,
                      extra, n_extra, ctx->cache, &need, private_stream);
  }
  return e;
}

struct TraceScope {
  hc_ctx* ctx;
  bool on;
  TraceScope(hc_ctx* c, const hc::GemmProblem& p) : ctx(c), on(c->tracing) {
    if (!on) return;
    char name[96];
    snprintf(name, sizeof name, "hc_matmul %s %lldx[%lldx%lldx%lld]", p.dtype == HC_F16 ? "f16" : "f32",
             (long long)p.batch, (long long)p.M, (long long)p.K, (long long)p.N);
    nvtxRangePushA(name);
    ctx->trace_valid = cudaEventRecord(ctx->trace_begin, ctx->stream) == cudaSuccess;
  }
  ~TraceScope() {
    if (!on) return;
    if (cudaEventRecord(ctx->trace_end, ctx->stream) != cudaSuccess) ctx->trace_valid = false;
    nvtxRangePop();
  }
};

hc_status run_problem(hc_ctx* ctx, hc_kernel kernel, const hc::GemmProblem& p, int64_t flops) {
  ctx->last_flops = flops;
  if (p.batch == 0 || p.M == 0 || p.N == 0) {
    ctx->last = hc::LaunchRecord();
    return HC_OK;
  }
  const int64_t eb = p.dtype == HC_F16 ? 2 : 4;
  if (p.K == 0) {
    // Empty contraction: every output is the empty sum, +0 (BackendCPU.swift:1293 starts at 0).
    for (int64_t m = 0; m < p.batch; m++) {
      HC_CUDA_TRY(ctx, cudaMemset2DAsync((char*)p.C + m * p.strideC * eb, p.ldc * eb, 0, p.N * eb, p.M, ctx->stream));
    }
    ctx->last = hc::LaunchRecord();
    return HC_OK;
  }
  hc_kernel chosen = kernel;
  if (kernel == HC_KERNEL_AUTO) {
    // Tiny products stay on the CUDA cores, in the reference's own arithmetic (separate multiply
    // and add, k ascending: bit-identical to BackendCPU.swift:1290-1300 for every flag combination).
    const bool big = (p.M * p.N >= 64 * 64) && (p.M * p.N * p.K >= kAutoTensorMinWork) && p.K >= 32;
    chosen = (big && hc::tc_supported(p)) ? HC_KERNEL_TENSOR : HC_KERNEL_SIMT_EXACT;
  }
  TraceScope trace(ctx, p);
  cudaError_t e;
  if (chosen == HC_KERNEL_TENSOR) {
    if (!hc::tc_supported(p))
      return fail(ctx, HC_ERR_NOT_IMPLEMENTED, "product too large for the tensor-core kernel's 32-bit tile coordinates");
    hc_status st;
    e = launch_tensor(ctx, p, nullptr, 0, &st);
    if (st != HC_OK) return st;
  } else if (chosen == HC_KERNEL_SIMT || chosen == HC_KERNEL_SIMT_EXACT) {
    e = hc::launch_simt(p, chosen == HC_KERNEL_SIMT_EXACT, ctx->stream, &ctx->last);
  } else {
    return fail(ctx, HC_ERR_INVALID_ARGUMENT, "unknown kernel selector");
  }
  ctx->launch_count += ctx->last.launches;
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(ctx, HC_ERR_KERNEL_FAILED, std::string("kernel launch failed: ") + cudaGetErrorString(e));
  }
  return HC_OK;
}

int64_t flop_count(int64_t count, int64_t rows, int64_t inner, int64_t cols) {
  return 2 * count * rows * inner * cols;
}

}  // namespace

// Accessors for the library's other translation units (hc_ctx is private to this file).
namespace hc {
std::mutex& ctx_mutex(hc_ctx* ctx) { return ctx->mu; }
cudaStream_t ctx_stream(hc_ctx* ctx) { return ctx->stream; }
unsigned int* ctx_status_word(hc_ctx* ctx) { return ctx->status_word; }
int ctx_sm_count(hc_ctx* ctx) { return ctx->sm_count; }
int ctx_device(hc_ctx* ctx) { return ctx->device; }
hc_status ctx_fail(hc_ctx* ctx, hc_status s, const char* msg) { return fail(ctx, s, msg); }
void ctx_note_launch(hc_ctx* ctx, const LaunchRecord& rec, int64_t flops) {
  ctx->last = rec;
  ctx->last_flops = flops;
  ctx->launch_count += rec.launches;
}
hc_status ctx_build_problem(hc_ctx* ctx, hc_dtype dtype, int64_t count, const void* a, int trans_a, const void* b,
                            int trans_b, int trans_out, int64_t rows, int64_t inner, int64_t cols, void* out,
                            GemmProblem* p) {
  return build_problem(ctx, dtype, count, a, trans_a, b, trans_b, trans_out, rows, inner, cols, 0, cols, out, p);
}
hc_status ctx_device_alloc(hc_ctx* ctx, void** ptr, size_t bytes) {
  if (ctx_malloc(ctx, ptr, bytes, ctx->stream) != cudaSuccess) {
    char msg[96];
    snprintf(msg, sizeof msg, "allocation of %zu bytes failed", bytes);
    return fail(ctx, HC_ERR_ALLOCATION_FAILED, msg);
  }
  return HC_OK;
}
void ctx_device_free(hc_ctx* ctx, void* ptr) {
  if (ptr && cudaFreeAsync(ptr, ctx->stream) != cudaSuccess) cudaGetLastError();
}
void ctx_count_launches(hc_ctx* ctx, int n) { ctx->launch_count += n; }
hc_status ctx_run_batched(hc_ctx* ctx, hc_dtype dtype, int64_t count, const void* a, int trans_a, const void* b,
                          int trans_b, int trans_out, int64_t rows, int64_t inner, int64_t cols, void* out) {
  GemmProblem p;
  hc_status s = build_problem(ctx, dtype, count, a, trans_a, b, trans_b, trans_out, rows, inner, cols, 0, cols, out, &p);
  if (s != HC_OK) return s;
  return run_problem(ctx, HC_KERNEL_AUTO, p, flop_count(count, rows, inner, cols));
}
hc_status ctx_run_colblock(hc_ctx* ctx, hc_dtype dtype, const void* a, int trans_a, const void* b, int trans_b,
                           int64_t rows, int64_t inner, int64_t cols, int64_t col_begin, int64_t col_count,
                           void* block_out, int64_t block_ld, void* const* extra, int n_extra) {
  GemmProblem p;
  // Planned as the block of the whole product (so that it is bitwise that block), stored where
  // the caller wants it: `block_out` is the block's first element, `block_ld` its row pitch.
  hc_status s = build_problem(ctx, dtype, 1, a, trans_a, b, trans_b, 0, rows, inner, cols, col_begin, col_count,
                              block_out, &p);
  if (s != HC_OK) return s;
  p.C = block_out;
  p.ldc = block_ld;
  p.strideC = rows * block_ld;
  ctx->last_flops = flop_count(1, rows, inner, col_count);
  if (p.M == 0 || p.N == 0) return HC_OK;
  if (n_extra == 0) return run_problem(ctx, HC_KERNEL_TENSOR, p, ctx->last_flops);
  if (p.K == 0) return fail(ctx, HC_ERR_INVALID_ARGUMENT, "pushed column blocks need a non-empty contraction");
  if (!tc_supported(p)) return fail(ctx, HC_ERR_NOT_IMPLEMENTED, "product too large for the tensor-core kernel");
  TraceScope trace(ctx, p);
  cudaError_t e = launch_tensor(ctx, p, extra, n_extra, &s);
  if (s != HC_OK) return s;
  ctx->launch_count += ctx->last.launches;
  if (e == cudaErrorNotSupported)
    return fail(ctx, HC_ERR_NOT_IMPLEMENTED, "result buffers must be 16-byte aligned with 16-byte row pitch");
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(ctx, HC_ERR_KERNEL_FAILED, std::string("kernel launch failed: ") + cudaGetErrorString(e));
  }
  return HC_OK;
}
}  // namespace hc

extern "C" {

hc_status hc_init(int device, hc_ctx** out) {
  if (!out) return HC_ERR_INVALID_ARGUMENT;
  *out = nullptr;
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || device < 0 || device >= n) {
    cudaGetLastError();
    return HC_ERR_INVALID_ARGUMENT;
  }
  hc_ctx* ctx = new (std::nothrow) hc_ctx();
  if (!ctx) return HC_ERR_ALLOCATION_FAILED;
  ctx->device = device;
  DeviceGuard g(device);
  cudaDeviceProp prop;
  if (!g.ok || cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
    delete ctx;
    return HC_ERR_CUDA;
  }
  if (prop.major != 10) {
    // The kernels in this library are built for sm_100a only.
    delete ctx;
    return HC_ERR_NOT_IMPLEMENTED;
  }
  ctx->sm_count = prop.multiProcessorCount;
  if (cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaMalloc((void**)&ctx->status_word, sizeof(unsigned int)) != cudaSuccess ||
      cudaMemset(ctx->status_word, 0, sizeof(unsigned int)) != cudaSuccess) {
    if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
    if (ctx->status_word) cudaFree(ctx->status_word);
    delete ctx;
    cudaGetLastError();
    return HC_ERR_CUDA;
  }
  ctx->stream = ctx->own_stream;
  {
    cudaMemPoolProps props = {};
    props.allocType = cudaMemAllocationTypePinned;
    props.handleTypes = cudaMemHandleTypeNone;
    props.location.type = cudaMemLocationTypeDevice;
    props.location.id = device;
    if (cudaMemPoolCreate(&ctx->pool, &props) == cudaSuccess) {
      const char* e = getenv("HC_POOL_RETAIN_MB");
      unsigned long long keep = (e ? strtoull(e, nullptr, 10) : 8192ull) << 20;
      if (cudaMemPoolSetAttribute(ctx->pool, cudaMemPoolAttrReleaseThreshold, &keep) != cudaSuccess) cudaGetLastError();
    } else {
      ctx->pool = nullptr;   // fall back to the device's default pool
      cudaGetLastError();
    }
  }
  ctx->cache = hc::tc_cache_create();
  *out = ctx;
  return HC_OK;
}

void hc_destroy(hc_ctx* ctx) {
  if (!ctx) return;
  DeviceGuard g(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  if (ctx->stream != ctx->own_stream) cudaStreamSynchronize(ctx->own_stream);
  hc::tc_cache_destroy(ctx->cache);
  if (ctx->trace_begin) cudaEventDestroy(ctx->trace_begin);
  if (ctx->trace_end) cudaEventDestroy(ctx->trace_end);
  if (ctx->scratch) cudaFreeAsync(ctx->scratch, ctx->own_stream);
  for (int i = 0; i < 3; i++)
    if (ctx->stage[i]) cudaFreeAsync(ctx->stage[i], ctx->own_stream);
  for (auto& sl : ctx->slot) {
    if (sl.out_done) cudaEventSynchronize(sl.out_done);
    for (int i = 0; i < 3; i++)
      if (sl.buf[i]) cudaFreeAsync(sl.buf[i], ctx->own_stream);
    if (sl.in_done) cudaEventDestroy(sl.in_done);
    if (sl.product_done) cudaEventDestroy(sl.product_done);
    if (sl.out_done) cudaEventDestroy(sl.out_done);
  }
  if (ctx->in_stream) cudaStreamDestroy(ctx->in_stream);
  if (ctx->out_stream) cudaStreamDestroy(ctx->out_stream);
  cudaFree(ctx->status_word);
  if (ctx->pool) {
    // Buffers the caller has not freed yet stay valid until they are (the pool's memory goes
    // back to the driver when the last of them has been freed).
    cudaStreamSynchronize(ctx->own_stream);
    cudaMemPoolDestroy(ctx->pool);
  }
  cudaStreamDestroy(ctx->own_stream);
  cudaGetLastError();
  delete ctx;
}

hc_status hc_set_stream(hc_ctx* ctx, void* cuda_stream) {
  if (!ctx) return HC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(ctx->mu);
  cudaStream_t next = cuda_stream ? (cudaStream_t)cuda_stream : ctx->own_stream;
  if (next != ctx->stream) {
    // Work already enqueued may still use the context's work areas (split operands, staging);
    // nothing on the new stream is ordered after it, so let it finish first.
    DeviceGuard g(ctx->device);
    HC_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    ctx->stream = next;
  }
  return HC_OK;
}

void* hc_get_stream(hc_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }
int hc_get_device(hc_ctx* ctx) { return ctx ? ctx->device : -1; }

hc_status hc_alloc(hc_ctx* ctx, size_t bytes, void** dptr) {
  if (!ctx || !dptr) return HC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  *dptr = nullptr;
  const size_t n = bytes ? bytes : 1;
  if (ctx_malloc(ctx, dptr, n, ctx->stream) != cudaSuccess) {
    char msg[96];
    snprintf(msg, sizeof msg, "allocation of %zu bytes failed", n);
    return fail(ctx, HC_ERR_ALLOCATION_FAILED, msg);
  }
  return HC_OK;
}

hc_status hc_free(hc_ctx* ctx, void* dptr) {
  if (!ctx) return HC_ERR_INVALID_ARGUMENT;
  if (!dptr) return HC_OK;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  HC_CUDA_TRY(ctx, cudaFreeAsync(dptr, ctx->stream));
  return HC_OK;
}

hc_status hc_h2d(hc_ctx* ctx, void* dst, const void* src, size_t bytes) {
  if (!ctx || (bytes && (!dst || !src))) return HC_ERR_INVALID_ARGUMENT;
  if (!bytes) return HC_OK;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  HC_CUDA_TRY(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
  return HC_OK;
}

hc_status hc_d2h(hc_ctx* ctx, void* dst, const void* src, size_t bytes) {
  if (!ctx || (bytes && (!dst || !src))) return HC_ERR_INVALID_ARGUMENT;
  if (!bytes) return HC_OK;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  HC_CUDA_TRY(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  return HC_OK;
}

hc_status hc_d2h_async(hc_ctx* ctx, void* dst_host, const void* src_device, size_t bytes, hc_event** done) {
  if (!ctx || !done || (bytes && (!dst_host || !src_device))) return HC_ERR_INVALID_ARGUMENT;
  *done = nullptr;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  if (!ctx->in_stream) {
    HC_CUDA_TRY(ctx, cudaStreamCreateWithFlags(&ctx->in_stream, cudaStreamNonBlocking));
    HC_CUDA_TRY(ctx, cudaStreamCreateWithFlags(&ctx->out_stream, cudaStreamNonBlocking));
  }
  hc_event* ev = new (std::nothrow) hc_event();
  if (!ev) return HC_ERR_ALLOCATION_FAILED;
  ev->ctx = ctx;
  ev->device = ctx->device;
  // The marker first stands for "everything enqueued so far": the side stream waits for it, the
  // copy follows, and the marker is then moved behind the copy.
  cudaError_t e = cudaEventCreate(&ev->ev);
  if (e == cudaSuccess) e = cudaEventRecord(ev->ev, ctx->stream);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->out_stream, ev->ev, 0);
  if (e == cudaSuccess && bytes) e = cudaMemcpyAsync(dst_host, src_device, bytes, cudaMemcpyDeviceToHost, ctx->out_stream);
  if (e == cudaSuccess) e = cudaEventRecord(ev->ev, ctx->out_stream);
  if (e != cudaSuccess) {
    if (ev->ev) cudaEventDestroy(ev->ev);
    delete ev;
    return cuda_fail(ctx, e, "asynchronous read-back");
  }
  *done = ev;
  return HC_OK;
}

hc_status hc_h2d_async(hc_ctx* ctx, void* dst_device, const void* src_host, size_t bytes, hc_event** done) {
  if (!ctx || !done || (bytes && (!dst_device || !src_host))) return HC_ERR_INVALID_ARGUMENT;
  *done = nullptr;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  if (!ctx->in_stream) {
    HC_CUDA_TRY(ctx, cudaStreamCreateWithFlags(&ctx->in_stream, cudaStreamNonBlocking));
    HC_CUDA_TRY(ctx, cudaStreamCreateWithFlags(&ctx->out_stream, cudaStreamNonBlocking));
  }
  hc_event* ev = new (std::nothrow) hc_event();
  if (!ev) return HC_ERR_ALLOCATION_FAILED;
  ev->ctx = ctx;
  ev->device = ctx->device;
  // Ordered after everything enqueued so far, so that earlier readers of the destination are done.
  cudaError_t e = cudaEventCreate(&ev->ev);
  if (e == cudaSuccess) e = cudaEventRecord(ev->ev, ctx->stream);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->in_stream, ev->ev, 0);
  if (e == cudaSuccess && bytes) e = cudaMemcpyAsync(dst_device, src_host, bytes, cudaMemcpyHostToDevice, ctx->in_stream);
  if (e == cudaSuccess) e = cudaEventRecord(ev->ev, ctx->in_stream);
  if (e != cudaSuccess) {
    if (ev->ev) cudaEventDestroy(ev->ev);
    delete ev;
    return cuda_fail(ctx, e, "asynchronous upload");
  }
  *done = ev;
  return HC_OK;
}

hc_status hc_enqueue_wait(hc_ctx* ctx, hc_event* ev) {
  if (!ctx || !ev) return HC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  HC_CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->stream, ev->ev, 0));
  return HC_OK;
}

hc_status hc_sync(hc_ctx* ctx) {
  if (!ctx) return HC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  HC_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
  return HC_OK;
}

hc_status hc_event_record(hc_ctx* ctx, hc_event** out) {
  if (!ctx || !out) return HC_ERR_INVALID_ARGUMENT;
  *out = nullptr;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  hc_event* ev = new (std::nothrow) hc_event();
  if (!ev) return HC_ERR_ALLOCATION_FAILED;
  ev->ctx = ctx;
  ev->device = ctx->device;
  cudaError_t e = cudaEventCreate(&ev->ev);
  if (e == cudaSuccess) e = cudaEventRecord(ev->ev, ctx->stream);
  if (e != cudaSuccess) {
    if (ev->ev) cudaEventDestroy(ev->ev);
    delete ev;
    return cuda_fail(ctx, e, "event record");
  }
  *out = ev;
  return HC_OK;
}

hc_status hc_event_wait(hc_event* ev) {
  if (!ev) return HC_ERR_INVALID_ARGUMENT;
  hc_ctx* ctx = ev->ctx;
  DeviceGuard g(ctx->device);
  cudaError_t e = cudaEventSynchronize(ev->ev);
  std::lock_guard<std::mutex> lock(ctx->mu);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "event wait");
  unsigned int word = 0;
  // The status word is only written by kernels; reading it after the event is race-free for
  // everything enqueued before the event.  The copy runs on the context's own (non-blocking)
  // stream so that it does not synchronise with unrelated streams of the process.
  e = cudaMemcpyAsync(&word, ctx->status_word, sizeof word, cudaMemcpyDeviceToHost, ctx->own_stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->own_stream);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "status read");
  if (word) {
    char msg[96];
    snprintf(msg, sizeof msg, "a bounded device-side wait expired (status bits 0x%x)", word);
    return fail(ctx, HC_ERR_TIMEOUT, msg);
  }
  return HC_OK;
}

hc_status hc_event_elapsed_ms(hc_event* start, hc_event* stop, float* ms) {
  if (!start || !stop || !ms) return HC_ERR_INVALID_ARGUMENT;
  DeviceGuard g(start->ctx->device);
  cudaError_t e = cudaEventElapsedTime(ms, start->ev, stop->ev);
  if (e != cudaSuccess) return cuda_fail(start->ctx, e, "event elapsed");
  return HC_OK;
}

void hc_event_destroy(hc_event* ev) {
  if (!ev) return;
  DeviceGuard g(ev->device);
  cudaEventDestroy(ev->ev);
  delete ev;
}

hc_status hc_batched_matmul_ex(hc_ctx* ctx, hc_kernel kernel, hc_dtype dtype, int64_t matrix_count, const void* a,
                               int trans_a, const void* b, int trans_b, int trans_out, int64_t rows, int64_t inner,
                               int64_t cols, void* out) {
  if (!ctx) return HC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  hc::GemmProblem p;
  hc_status s = build_problem(ctx, dtype, matrix_count, a, trans_a, b, trans_b, trans_out, rows, inner, cols, 0, cols,
                              out, &p);
  if (s != HC_OK) return s;
  return run_problem(ctx, kernel, p, flop_count(matrix_count, rows, inner, cols));
}

hc_status hc_batched_matmul(hc_ctx* ctx, hc_dtype dtype, int64_t matrix_count, const void* a, int trans_a,
                            const void* b, int trans_b, int trans_out, int64_t rows, int64_t inner, int64_t cols,
                            void* out) {
  return hc_batched_matmul_ex(ctx, HC_KERNEL_AUTO, dtype, matrix_count, a, trans_a, b, trans_b, trans_out, rows,
                              inner, cols, out);
}

hc_status hc_matmul(hc_ctx* ctx, hc_dtype dtype, const void* a, int trans_a, const void* b, int trans_b,
                    int trans_out, int64_t rows, int64_t inner, int64_t cols, void* out) {
  return hc_batched_matmul_ex(ctx, HC_KERNEL_AUTO, dtype, 1, a, trans_a, b, trans_b, trans_out, rows, inner, cols,
                              out);
}

hc_status hc_matmul_colblock(hc_ctx* ctx, hc_kernel kernel, hc_dtype dtype, const void* a, int trans_a, const void* b,
                             int trans_b, int trans_out, int64_t rows, int64_t inner, int64_t cols,
                             int64_t col_begin, int64_t col_count, void* out) {
  if (!ctx) return HC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  hc::GemmProblem p;
  hc_status s = build_problem(ctx, dtype, 1, a, trans_a, b, trans_b, trans_out, rows, inner, cols, col_begin,
                              col_count, out, &p);
  if (s != HC_OK) return s;
  return run_problem(ctx, kernel, p, flop_count(1, rows, inner, col_count));
}

hc_status hc_matmul_colblock_push(hc_ctx* ctx, hc_dtype dtype, const void* a, int trans_a, const void* b, int trans_b,
                                  int trans_out, int64_t rows, int64_t inner, int64_t cols, int64_t col_begin,
                                  int64_t col_count, void* out, void* const* peer_outs, int n_peers) {
  if (!ctx) return HC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  if (n_peers < 0 || n_peers > 7 || (n_peers > 0 && !peer_outs))
    return fail(ctx, HC_ERR_INVALID_ARGUMENT, "between 0 and 7 peer results");
  hc::GemmProblem p;
  hc_status s = build_problem(ctx, dtype, 1, a, trans_a, b, trans_b, trans_out, rows, inner, cols, col_begin,
                              col_count, out, &p);
  if (s != HC_OK) return s;
  ctx->last_flops = flop_count(1, rows, inner, col_count);
  if (p.M == 0 || p.N == 0) return HC_OK;
  if (p.K == 0) return fail(ctx, HC_ERR_INVALID_ARGUMENT, "pushed column blocks need a non-empty contraction");
  if (!hc::tc_supported(p))
    return fail(ctx, HC_ERR_NOT_IMPLEMENTED, "tensor-core kernel needs 16-byte aligned operands and leading dimensions");
  // The block sits at the same offset in every device's copy of the result.
  const ptrdiff_t offset = (const char*)p.C - (const char*)out;
  void* extra[7];
  for (int i = 0; i < n_peers; i++) {
    if (!peer_outs[i]) return fail(ctx, HC_ERR_INVALID_ARGUMENT, "null peer result");
    extra[i] = (char*)peer_outs[i] + offset;
  }
  cudaError_t e = launch_tensor(ctx, p, extra, n_peers, &s);
  if (s != HC_OK) return s;
  ctx->launch_count += ctx->last.launches;
  if (e == cudaErrorNotSupported)
    return fail(ctx, HC_ERR_NOT_IMPLEMENTED, "result buffers must be 16-byte aligned with 16-byte row pitch");
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(ctx, HC_ERR_KERNEL_FAILED, std::string("kernel launch failed: ") + cudaGetErrorString(e));
  }
  return HC_OK;
}

hc_status hc_shared_alloc(hc_ctx* ctx, size_t bytes, void** dptr) {
  if (!ctx || !dptr) return HC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  *dptr = nullptr;
  cudaError_t e = cudaMalloc(dptr, bytes ? bytes : 1);
  if (e != cudaSuccess) {
    *dptr = nullptr;
    cudaGetLastError();
    return fail(ctx, HC_ERR_ALLOCATION_FAILED, "shared allocation failed");
  }
  return HC_OK;
}

hc_status hc_shared_free(hc_ctx* ctx, void* dptr) {
  if (!ctx) return HC_ERR_INVALID_ARGUMENT;
  if (!dptr) return HC_OK;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  HC_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
  HC_CUDA_TRY(ctx, cudaFree(dptr));
  return HC_OK;
}

hc_status hc_ipc_export(hc_ctx* ctx, void* dptr, void* handle_out) {
  if (!ctx || !dptr || !handle_out) return HC_ERR_INVALID_ARGUMENT;
  static_assert(sizeof(cudaIpcMemHandle_t) == HC_IPC_HANDLE_BYTES, "handle size");
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  cudaIpcMemHandle_t h;
  HC_CUDA_TRY(ctx, cudaIpcGetMemHandle(&h, dptr));
  memcpy(handle_out, &h, sizeof h);
  return HC_OK;
}

hc_status hc_ipc_open(hc_ctx* ctx, const void* handle, void** dptr) {
  if (!ctx || !handle || !dptr) return HC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof h);
  *dptr = nullptr;
  HC_CUDA_TRY(ctx, cudaIpcOpenMemHandle(dptr, h, cudaIpcMemLazyEnablePeerAccess));
  return HC_OK;
}

hc_status hc_ipc_close(hc_ctx* ctx, void* dptr) {
  if (!ctx) return HC_ERR_INVALID_ARGUMENT;
  if (!dptr) return HC_OK;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  HC_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
  HC_CUDA_TRY(ctx, cudaIpcCloseMemHandle(dptr));
  return HC_OK;
}

namespace {
// Argument checks of the host-buffer products, made before any copy or allocation: dtype, signs,
// sizes that fit, pointers.  `bytes` receives the sizes of a, b and the result.
hc_status host_product_bytes(hc_ctx* ctx, hc_dtype dtype, int64_t matrix_count, const void* a_host,
                             const void* b_host, const void* out_host, int64_t rows, int64_t inner, int64_t cols,
                             size_t bytes[3]) {
  if (dtype != HC_F16 && dtype != HC_F32)
    return fail(ctx, HC_ERR_NOT_IMPLEMENTED, "matmul: only float16 and float32 are implemented");
  if (matrix_count < 0 || rows < 0 || inner < 0 || cols < 0)
    return fail(ctx, HC_ERR_INVALID_ARGUMENT, "negative dimension");
  const int64_t eb = dtype == HC_F16 ? 2 : 4;
  int64_t na, nb, nc;
  if (mul_overflows(rows, inner, &na) || mul_overflows(na, matrix_count, &na) || mul_overflows(na, eb, &na) ||
      mul_overflows(inner, cols, &nb) || mul_overflows(nb, matrix_count, &nb) || mul_overflows(nb, eb, &nb) ||
      mul_overflows(rows, cols, &nc) || mul_overflows(nc, matrix_count, &nc) || mul_overflows(nc, eb, &nc))
    return fail(ctx, HC_ERR_INVALID_ARGUMENT, "operand size overflows int64");
  bytes[0] = (size_t)na; bytes[1] = (size_t)nb; bytes[2] = (size_t)nc;
  if ((bytes[0] && !a_host) || (bytes[1] && !b_host) || (bytes[2] && !out_host))
    return fail(ctx, HC_ERR_INVALID_ARGUMENT, "null operand");
  return HC_OK;
}
}  // namespace

hc_status hc_batched_matmul_host(hc_ctx* ctx, hc_dtype dtype, int64_t matrix_count, const void* a_host, int trans_a,
                                 const void* b_host, int trans_b, int trans_out, int64_t rows, int64_t inner,
                                 int64_t cols, void* out_host) {
  if (!ctx) return HC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  size_t bytes[3];
  hc_status s = host_product_bytes(ctx, dtype, matrix_count, a_host, b_host, out_host, rows, inner, cols, bytes);
  if (s != HC_OK) return s;
  for (int i = 0; i < 3; i++) {
    s = ensure_buffer(ctx, &ctx->stage[i], &ctx->stage_bytes[i], bytes[i], ctx->stream);
    if (s != HC_OK) return s;
  }
  hc::GemmProblem p;
  s = build_problem(ctx, dtype, matrix_count, ctx->stage[0], trans_a, ctx->stage[1], trans_b, trans_out, rows, inner,
                    cols, 0, cols, ctx->stage[2], &p);
  if (s != HC_OK) return s;
  if (bytes[0]) HC_CUDA_TRY(ctx, cudaMemcpyAsync(ctx->stage[0], a_host, bytes[0], cudaMemcpyHostToDevice, ctx->stream));
  if (bytes[1]) HC_CUDA_TRY(ctx, cudaMemcpyAsync(ctx->stage[1], b_host, bytes[1], cudaMemcpyHostToDevice, ctx->stream));
  s = run_problem(ctx, HC_KERNEL_AUTO, p, flop_count(matrix_count, rows, inner, cols));
  if (s != HC_OK) return s;
  if (bytes[2]) HC_CUDA_TRY(ctx, cudaMemcpyAsync(out_host, ctx->stage[2], bytes[2], cudaMemcpyDeviceToHost, ctx->stream));
  HC_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
  return HC_OK;
}

hc_status hc_batched_matmul_host_async(hc_ctx* ctx, hc_dtype dtype, int64_t matrix_count, const void* a_host,
                                       int trans_a, const void* b_host, int trans_b, int trans_out, int64_t rows,
                                       int64_t inner, int64_t cols, void* out_host) {
  if (!ctx) return HC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  size_t bytes[3];
  hc_status s = host_product_bytes(ctx, dtype, matrix_count, a_host, b_host, out_host, rows, inner, cols, bytes);
  if (s != HC_OK) return s;
  if (!ctx->in_stream) {
    HC_CUDA_TRY(ctx, cudaStreamCreateWithFlags(&ctx->in_stream, cudaStreamNonBlocking));
    HC_CUDA_TRY(ctx, cudaStreamCreateWithFlags(&ctx->out_stream, cudaStreamNonBlocking));
  }
  hc_ctx::HostSlot& sl = ctx->slot[ctx->next_slot];
  ctx->next_slot ^= 1;
  if (!sl.in_done) {
    HC_CUDA_TRY(ctx, cudaEventCreateWithFlags(&sl.in_done, cudaEventDisableTiming));
    HC_CUDA_TRY(ctx, cudaEventCreateWithFlags(&sl.product_done, cudaEventDisableTiming));
    HC_CUDA_TRY(ctx, cudaEventCreateWithFlags(&sl.out_done, cudaEventDisableTiming));
  }
  // The slot's previous product (two calls ago) must have left its buffers.
  if (sl.busy) HC_CUDA_TRY(ctx, cudaEventSynchronize(sl.out_done));
  sl.busy = false;
  bool grew = false;
  for (int i = 0; i < 3; i++) {
    if (bytes[i] > sl.bytes[i] || !sl.buf[i]) {
      s = ensure_buffer(ctx, &sl.buf[i], &sl.bytes[i], bytes[i], ctx->stream);
      if (s != HC_OK) return s;
      grew = true;
    }
  }
  if (grew) {
    // The staging memory was allocated in the order of the context's stream; the copy-in stream
    // may use it only from that point on.
    HC_CUDA_TRY(ctx, cudaEventRecord(sl.in_done, ctx->stream));
    HC_CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->in_stream, sl.in_done, 0));
  }
  hc::GemmProblem p;
  s = build_problem(ctx, dtype, matrix_count, sl.buf[0], trans_a, sl.buf[1], trans_b, trans_out, rows, inner, cols, 0,
                    cols, sl.buf[2], &p);
  if (s != HC_OK) return s;
  if (bytes[0]) HC_CUDA_TRY(ctx, cudaMemcpyAsync(sl.buf[0], a_host, bytes[0], cudaMemcpyHostToDevice, ctx->in_stream));
  if (bytes[1]) HC_CUDA_TRY(ctx, cudaMemcpyAsync(sl.buf[1], b_host, bytes[1], cudaMemcpyHostToDevice, ctx->in_stream));
  HC_CUDA_TRY(ctx, cudaEventRecord(sl.in_done, ctx->in_stream));
  HC_CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->stream, sl.in_done, 0));
  s = run_problem(ctx, HC_KERNEL_AUTO, p, flop_count(matrix_count, rows, inner, cols));
  if (s != HC_OK) return s;
  HC_CUDA_TRY(ctx, cudaEventRecord(sl.product_done, ctx->stream));
  HC_CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->out_stream, sl.product_done, 0));
  if (bytes[2])
    HC_CUDA_TRY(ctx, cudaMemcpyAsync(out_host, sl.buf[2], bytes[2], cudaMemcpyDeviceToHost, ctx->out_stream));
  HC_CUDA_TRY(ctx, cudaEventRecord(sl.out_done, ctx->out_stream));
  sl.busy = true;
  return HC_OK;
}

hc_status hc_host_sync(hc_ctx* ctx) {
  if (!ctx) return HC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  for (auto& sl : ctx->slot) {
    if (sl.busy) HC_CUDA_TRY(ctx, cudaEventSynchronize(sl.out_done));
    sl.busy = false;
  }
  return HC_OK;
}

const char* hc_status_string(hc_status s) {
  switch (s) {
    case HC_OK: return "ok";
    case HC_ERR_ALLOCATION_FAILED: return "allocation failed";
    case HC_ERR_KERNEL_FAILED: return "kernel failed";
    case HC_ERR_NOT_IMPLEMENTED: return "not implemented";
    case HC_ERR_INVALID_ARGUMENT: return "invalid argument";
    case HC_ERR_TIMEOUT: return "device-side wait timed out";
    case HC_ERR_CUDA: return "CUDA error";
  }
  return "unknown status";
}

const char* hc_last_error(hc_ctx* ctx) { return ctx ? ctx->last_error.c_str() : ""; }

size_t hc_copy_last_error(hc_ctx* ctx, char* buf, size_t capacity) {
  if (!ctx || !buf || capacity == 0) return 0;
  std::lock_guard<std::mutex> lock(ctx->mu);
  const size_t n = ctx->last_error.size() < capacity - 1 ? ctx->last_error.size() : capacity - 1;
  memcpy(buf, ctx->last_error.data(), n);
  buf[n] = 0;
  return n;
}

hc_status hc_last_launch_info(hc_ctx* ctx, hc_launch_info* out) {
  if (!ctx || !out) return HC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(ctx->mu);
  out->kernel = ctx->last.kernel;
  out->tile_m = ctx->last.tile_m; out->tile_n = ctx->last.tile_n; out->tile_k = ctx->last.tile_k;
  out->stages = ctx->last.stages; out->grid = ctx->last.grid; out->block = ctx->last.block;
  out->tiles = ctx->last.tiles; out->flops = ctx->last_flops; out->scratch_bytes = ctx->last.scratch_bytes;
  return HC_OK;
}

hc_status hc_plan_product(hc_dtype dtype, int64_t matrix_count, int trans_a, int trans_b, int trans_out, int64_t rows,
                          int64_t inner, int64_t cols, int sm_count, hc_plan_info* out) {
  if (!out || (dtype != HC_F16 && dtype != HC_F32) || matrix_count < 1 || rows < 1 || inner < 1 || cols < 1 ||
      sm_count < 2)
    return HC_ERR_INVALID_ARGUMENT;
  // The same folding as build_problem: a transposed output swaps the operand roles.
  hc::GemmProblem p;
  p.dtype = dtype; p.batch = matrix_count; p.K = inner;
  p.A = p.B = nullptr; p.C = nullptr;
  if (!trans_out) {
    p.M = rows; p.N = cols;
    p.a_mn_major = trans_a ? 1 : 0; p.b_mn_major = trans_b ? 0 : 1;
  } else {
    p.M = cols; p.N = rows;
    p.a_mn_major = trans_b ? 0 : 1; p.b_mn_major = trans_a ? 1 : 0;
  }
  p.lda = p.a_mn_major ? p.M : p.K; p.ldb = p.b_mn_major ? p.N : p.K; p.ldc = p.N;
  p.strideA = p.M * p.K; p.strideB = p.N * p.K; p.strideC = p.M * p.N;
  const hc::PlanSummary r = hc::tc_describe_plan(p, sm_count);
  out->tile_m = r.tile_m; out->tile_n = r.tile_n; out->ctas_per_tile = r.ctas;
  out->slabs_per_slot = r.slabs; out->parts = r.parts; out->slots_per_part = r.slots_per_part;
  out->tiles = r.tiles; out->workspace_bytes = r.ws_bytes;
  return HC_OK;
}

int64_t hc_launch_count(hc_ctx* ctx) {
  if (!ctx) return 0;
  std::lock_guard<std::mutex> lock(ctx->mu);
  return ctx->launch_count;
}

hc_status hc_check_device_status(hc_ctx* ctx) {
  if (!ctx) return HC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  HC_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
  unsigned int word = 0;
  HC_CUDA_TRY(ctx, cudaMemcpyAsync(&word, ctx->status_word, sizeof word, cudaMemcpyDeviceToHost, ctx->own_stream));
  HC_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->own_stream));
  if (word) {
    HC_CUDA_TRY(ctx, cudaMemsetAsync(ctx->status_word, 0, sizeof word, ctx->own_stream));
    HC_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->own_stream));
    char msg[96];
    snprintf(msg, sizeof msg, "a bounded device-side wait expired (status bits 0x%x)", word);
    return fail(ctx, HC_ERR_TIMEOUT, msg);
  }
  return HC_OK;
}

hc_status hc_linear_forward(hc_ctx* ctx, hc_dtype dtype, const void* x, const void* weight, const void* bias,
                            int64_t rows, int64_t in_count, int64_t out_count, void* out) {
  if (!ctx) return HC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  hc::GemmProblem p;
  hc_status s = build_problem(ctx, dtype, 1, x, 0, weight, 0, 0, rows, in_count, out_count, 0, out_count, out, &p);
  if (s != HC_OK) return s;
  if (in_count == 0 && bias && rows > 0 && out_count > 0)
    return fail(ctx, HC_ERR_INVALID_ARGUMENT, "linear forward needs a non-empty input dimension");
  p.bias = bias;
  return run_problem(ctx, HC_KERNEL_AUTO, p, flop_count(1, rows, in_count, out_count));
}

hc_status hc_column_sum(hc_ctx* ctx, hc_dtype dtype, const void* x, int64_t rows, int64_t cols, void* out) {
  if (!ctx || rows < 0 || cols < 0 || (cols > 0 && !out) || (rows * cols > 0 && !x)) return HC_ERR_INVALID_ARGUMENT;
  if (dtype != HC_F16 && dtype != HC_F32) return HC_ERR_NOT_IMPLEMENTED;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  cudaError_t e = hc::launch_column_sum(dtype, x, out, rows, cols, ctx->stream);
  ctx->launch_count += 1;
  if (e != cudaSuccess) return cuda_fail(ctx, e, "column sum");
  return HC_OK;
}

hc_status hc_cast(hc_ctx* ctx, hc_dtype from, hc_dtype to, const void* x, int64_t count, void* out) {
  if (!ctx || count < 0 || (count > 0 && (!x || !out))) return HC_ERR_INVALID_ARGUMENT;
  if ((from != HC_F16 && from != HC_F32) || (to != HC_F16 && to != HC_F32)) return HC_ERR_NOT_IMPLEMENTED;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  cudaError_t e = hc::launch_cast(from, to, x, out, count, ctx->stream);
  ctx->launch_count += 1;
  if (e != cudaSuccess) return cuda_fail(ctx, e, "cast");
  return HC_OK;
}

hc_status hc_add(hc_ctx* ctx, hc_dtype dtype, const void* a, const void* b, int64_t count, void* out) {
  if (!ctx || count < 0 || (count > 0 && (!a || !b || !out))) return HC_ERR_INVALID_ARGUMENT;
  if (dtype != HC_F16 && dtype != HC_F32) return HC_ERR_NOT_IMPLEMENTED;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  cudaError_t e = hc::launch_add(dtype, a, b, out, count, ctx->stream);
  ctx->launch_count += 1;
  if (e != cudaSuccess) return cuda_fail(ctx, e, "add");
  return HC_OK;
}

hc_status hc_constant(hc_ctx* ctx, hc_dtype dtype, float value, int64_t count, void* out) {
  if (!ctx || count < 0 || (count > 0 && !out)) return HC_ERR_INVALID_ARGUMENT;
  if (dtype != HC_F16 && dtype != HC_F32) return HC_ERR_NOT_IMPLEMENTED;
  if (((uintptr_t)out & (dtype == HC_F16 ? 1 : 3)) != 0) return HC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  cudaError_t e = hc::launch_constant(dtype, value, out, count, ctx->stream);
  ctx->launch_count += count > 0 ? 1 : 0;
  if (e != cudaSuccess) return cuda_fail(ctx, e, "constant");
  return HC_OK;
}

hc_status hc_transpose(hc_ctx* ctx, hc_dtype dtype, int64_t matrix_count, const void* in, int64_t rows, int64_t cols,
                       void* out) {
  if (!ctx || matrix_count < 0 || rows < 0 || cols < 0) return HC_ERR_INVALID_ARGUMENT;
  if (matrix_count * rows * cols > 0 && (!in || !out)) return HC_ERR_INVALID_ARGUMENT;
  if (dtype != HC_F16 && dtype != HC_F32) return HC_ERR_NOT_IMPLEMENTED;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  cudaError_t e = hc::launch_transpose(dtype, matrix_count, in, out, rows, cols, ctx->stream);
  ctx->launch_count += 1;
  if (e != cudaSuccess) return cuda_fail(ctx, e, "transpose");
  return HC_OK;
}

hc_status hc_random(hc_ctx* ctx, int normal, hc_dtype dtype, uint64_t seed, uint64_t offset, int64_t count, void* out,
                    uint64_t* next_offset) {
  if (!ctx || count < 0 || (count > 0 && !out)) return HC_ERR_INVALID_ARGUMENT;
  if (dtype != HC_F16 && dtype != HC_F32) return HC_ERR_NOT_IMPLEMENTED;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  cudaError_t e = hc::launch_random(normal ? 1 : 0, dtype, seed, offset, count, out, ctx->stream);
  ctx->launch_count += count > 0 ? 1 : 0;
  if (e != cudaSuccess) return cuda_fail(ctx, e, "random");
  // The reference's loops run `through: count`: one counter value more than the outputs need.
  if (next_offset) *next_offset = offset + (uint64_t)(normal ? count / 2 + 1 : count / 4 + 1);
  return HC_OK;
}

hc_status hc_selftest_bounded_wait(hc_ctx* ctx, int limit_ms) {
  if (!ctx || limit_ms < 1 || limit_ms > 1000) return HC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  cudaError_t e = hc::launch_wait_probe(ctx->stream, ctx->status_word, (unsigned long long)limit_ms * 1000000ull);
  ctx->launch_count += 1;
  if (e != cudaSuccess) return cuda_fail(ctx, e, "wait probe launch");
  return HC_OK;
}

hc_status hc_inject_allocation_failures(hc_ctx* ctx, int count) {
  if (!ctx || count < 0) return HC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(ctx->mu);
  ctx->fail_allocs = count;
  return HC_OK;
}

hc_status hc_set_tracing(hc_ctx* ctx, int on) {
  if (!ctx) return HC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  if (on && !ctx->trace_begin) {
    HC_CUDA_TRY(ctx, cudaEventCreate(&ctx->trace_begin));
    HC_CUDA_TRY(ctx, cudaEventCreate(&ctx->trace_end));
  }
  ctx->tracing = on != 0;
  ctx->trace_valid = false;
  return HC_OK;
}

hc_status hc_last_elapsed_ms(hc_ctx* ctx, float* ms) {
  if (!ctx || !ms) return HC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard g(ctx->device);
  if (!ctx->tracing || !ctx->trace_valid)
    return fail(ctx, HC_ERR_INVALID_ARGUMENT, "no traced product: switch tracing on and run one first");
  HC_CUDA_TRY(ctx, cudaEventSynchronize(ctx->trace_end));
  HC_CUDA_TRY(ctx, cudaEventElapsedTime(ms, ctx->trace_begin, ctx->trace_end));
  return HC_OK;
}

const char* hc_version(void) { return "0.2"; }

}  // extern "C"

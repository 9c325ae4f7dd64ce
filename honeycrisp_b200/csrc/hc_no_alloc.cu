// hc_matmul_f32_static_scratch: the float32 tensor-core product for callers that must not
// allocate device memory.
//
// The float32 product runs as 3xTF32 and needs a work area for the low halves of both
// operands (and for a copy of an operand TMA cannot address where it lies).  hc_matmul obtains that area with cudaMalloc on first use and grows it on demand.
// Some hosts cannot tolerate that: a framework whose own caching allocator has already claimed
// the whole device (a cudaMalloc from inside a library then fails or fragments its pool), or a
// latency-critical loop in which the implicit device-wide synchronisation of cudaMalloc/cudaFree
// is not acceptable.  For them this file keeps a fixed work area inside the library image: a
// file-scope __device__ array.  Every GPU that loads the library carries those bytes until the
// process exits, which is why the area is modest and the entry point refuses products that do
// not fit.
//
// The array's name is only a handle in host code - it is not a device address, and passing it
// to a kernel would make the kernel read host memory or fault.  The device address is looked up
// once per device with cudaGetSymbolAddress, with that device current, and cached.  That lookup
// happens in the first call on each device, so make that first call outside any stream capture.
//
// The work area is shared by every call and every context of the process and is never cleared:
// nothing in it has to start at zero, because each call first overwrites exactly the elements
// it later reads (split operands by the pre-pass, partial sums by the product kernel's tiles).  Two calls that overlap on the GPU (different streams, different contexts,
// different host threads on one device) would overwrite each other's split operands; callers
// must order such calls themselves.
#include <cstdio>
#include <mutex>

#include "common.cuh"

// Capacity of the static work area.  A product needs 4 * (rows*inner + inner*cols) bytes plus
// alignment padding (one float32 array per operand; two for a misaligned one), and a long contraction that is cut
// into parts another parts * rows * cols * 4 bytes for its partial sums.
#define HC_STATIC_SCRATCH_BYTES (32u * 1024u * 1024u)

static __device__ __align__(256) unsigned char hc_static_scratch[HC_STATIC_SCRATCH_BYTES];

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_setup_mu;
void* g_scratch_ptr[kMaxDevices] = {};

// Device address of hc_static_scratch on the current device; looked up once per device.
cudaError_t static_scratch_address(int device, void** out) {
  if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_setup_mu);
  if (!g_scratch_ptr[device]) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&ptr, hc_static_scratch);
    if (e != cudaSuccess) return e;
    g_scratch_ptr[device] = ptr;
  }
  *out = g_scratch_ptr[device];
  return cudaSuccess;
}

}  // namespace

extern "C" {

size_t hc_static_scratch_capacity(void) { return (size_t)HC_STATIC_SCRATCH_BYTES; }

hc_status hc_matmul_f32_static_scratch(hc_ctx* ctx, const void* a, int trans_a, const void* b, int trans_b,
                                       int trans_out, int64_t rows, int64_t inner, int64_t cols, void* out) {
  if (!ctx) return HC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(hc::ctx_mutex(ctx));
  const int device = hc::ctx_device(ctx);
  int prev = -1;
  cudaGetDevice(&prev);
  if (prev != device && cudaSetDevice(device) != cudaSuccess) {
    cudaGetLastError();
    return hc::ctx_fail(ctx, HC_ERR_CUDA, "cannot make the context's device current");
  }
  struct Restore {
    int prev, device;
    ~Restore() { if (prev >= 0 && prev != device) cudaSetDevice(prev); }
  } restore{prev, device};

  hc::GemmProblem p;
  hc_status s = hc::ctx_build_problem(ctx, HC_F32, 1, a, trans_a, b, trans_b, trans_out, rows, inner, cols, out, &p);
  if (s != HC_OK) return s;
  if (rows == 0 || cols == 0) return HC_OK;
  if (inner == 0)
    return hc::ctx_fail(ctx, HC_ERR_INVALID_ARGUMENT, "static-scratch product needs a non-empty contraction");
  if (!hc::tc_supported(p))
    return hc::ctx_fail(ctx, HC_ERR_NOT_IMPLEMENTED,
                        "tensor-core kernel needs 16-byte aligned operands and leading dimensions");
  // Planned like the allocating path - a long contraction over few outputs is cut into parts whose
  // float32 partial sums also live in the array - so the bits are that path's.  Only when the
  // operands fit but the partial sums do not is the contraction kept whole.
  size_t need = hc::tc_scratch_bytes(p, hc::ctx_sm_count(ctx));
  if (need > (size_t)HC_STATIC_SCRATCH_BYTES) {
    p.no_split = true;
    need = hc::tc_scratch_bytes(p, hc::ctx_sm_count(ctx));
  }
  if (need > (size_t)HC_STATIC_SCRATCH_BYTES) {
    char msg[160];
    snprintf(msg, sizeof msg,
             "product needs %zu bytes of work area but the static area holds %u; use hc_matmul for this size", need,
             (unsigned)HC_STATIC_SCRATCH_BYTES);
    return hc::ctx_fail(ctx, HC_ERR_INVALID_ARGUMENT, msg);
  }
  void* scratch = nullptr;
  cudaError_t e = static_scratch_address(device, &scratch);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return hc::ctx_fail(ctx, HC_ERR_CUDA, cudaGetErrorString(e));
  }
  hc::LaunchRecord rec;
  e = hc::launch_tc(p, hc::ctx_stream(ctx), hc::ctx_status_word(ctx), scratch, (size_t)HC_STATIC_SCRATCH_BYTES,
                    hc::ctx_sm_count(ctx), &rec);
  hc::ctx_note_launch(ctx, rec, 2 * rows * inner * cols);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return hc::ctx_fail(ctx, HC_ERR_KERNEL_FAILED, cudaGetErrorString(e));
  }
  return HC_OK;
}

}  // extern "C"

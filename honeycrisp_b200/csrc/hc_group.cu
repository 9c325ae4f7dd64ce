// Products split over the GPUs of one box, behind the C ABI (declarations in include/hc_cuda.h).
//
// A group is one rank's view of `world` contexts, one per GPU: ranks are processes (one per GPU)
// or threads of one process (one host, several devices).  The reference has no multi-device code
// (a Backend holds one device, Sources/Honeycrisp/BackendMPS.swift:352), so the contract of every
// entry point here is "equals the single-device result of the same call":
//
//   hc_batched_matmul_sharded   the matrices of a batch are independent
//                               (Sources/Honeycrisp/BackendCPU.swift:1290 loops over them): each
//                               rank multiplies a contiguous range; nothing is exchanged unless the
//                               caller asks for the whole result everywhere.
//   hc_matmul_nsplit_allgather  one large product split over the columns of op(a)*op(b); each rank
//                               computes its block with the tile decomposition of the whole
//                               product, and the blocks are exchanged
//                                 fused == 0: by ncclAllGather of the packed blocks, then one
//                                             kernel that puts them into the row-major result;
//                                 fused == 1: by the product kernel itself, whose epilogue stores
//                                             every finished tile into every rank's result (peer
//                                             stores over NVLink), between two flag barriers.
//
// NCCL is bound at run time (dlopen), preferring a copy the process has already loaded, so the
// library itself has no link-time dependency and loads on machines without NCCL; a group of more
// than one rank then fails with HC_ERR_NOT_IMPLEMENTED.
//
// Nothing here loads from another GPU's memory: peers are written (TMA stores from the product
// kernel, 8-byte flag stores from the barrier kernel) and every rank reads only its own memory.
// Every device-side wait is bounded; on expiry the kernel sets a bit in the context's status word
// and returns, and the host reports HC_ERR_TIMEOUT.
#include <dlfcn.h>
#include <unistd.h>

#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "common.cuh"

#if __has_include(<nccl.h>)
#include <nccl.h>
#else
// The few declarations of NCCL's public interface this file uses.
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef enum { ncclSuccess = 0 } ncclResult_t;
typedef enum { ncclInt8 = 0, ncclChar = 0 } ncclDataType_t;
#endif

namespace {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Broadcast)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  bool ok = false;
};

const NcclApi& nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    // A copy already in the process (the host framework's) first, so that there is one NCCL.
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (!h) {
      const char* path = getenv("HC_NCCL_LIB");
      if (path && *path) h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
    }
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
    if (!h) return;
    api.handle = h;
    api.GetUniqueId = (decltype(api.GetUniqueId))dlsym(h, "ncclGetUniqueId");
    api.CommInitRank = (decltype(api.CommInitRank))dlsym(h, "ncclCommInitRank");
    api.CommDestroy = (decltype(api.CommDestroy))dlsym(h, "ncclCommDestroy");
    api.AllGather = (decltype(api.AllGather))dlsym(h, "ncclAllGather");
    api.Broadcast = (decltype(api.Broadcast))dlsym(h, "ncclBroadcast");
    api.GroupStart = (decltype(api.GroupStart))dlsym(h, "ncclGroupStart");
    api.GroupEnd = (decltype(api.GroupEnd))dlsym(h, "ncclGroupEnd");
    api.GetErrorString = (decltype(api.GetErrorString))dlsym(h, "ncclGetErrorString");
    api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllGather && api.Broadcast &&
             api.GroupStart && api.GroupEnd && api.GetErrorString;
  });
  return api;
}

constexpr int kMaxWorld = 8;

// What a rank tells the others about one of its buffers.  Ranks in other processes map it
// through the CUDA IPC handle; ranks in the same process use the pointer itself.
struct PeerRecord {
  int64_t pid;
  uint64_t ptr;
  int32_t device;
  int32_t pad;
  cudaIpcMemHandle_t handle;
  char fill[128 - 24 - sizeof(cudaIpcMemHandle_t)];
};
static_assert(sizeof(PeerRecord) == 128, "records travel as fixed 128-byte blocks");

// A buffer every rank has allocated with the same size, and this rank's mappings of the others'.
struct SharedBuf {
  void* local = nullptr;
  size_t bytes = 0;
  void* peer[kMaxWorld] = {};       // peer[rank] == local
  bool ipc_opened[kMaxWorld] = {};
};

// Control block of a rank (device memory the peers can write): two sets of arrival counters,
// one word per rank.  Set 0 orders "every rank has entered this call" (the previous result is no
// longer read), set 1 "every rank's tiles have landed".
struct ControlBlock {
  unsigned long long arrived[2][kMaxWorld];
};

}  // namespace

struct hc_group {
  hc_ctx* ctx = nullptr;
  int world = 1, rank = 0;
  ncclComm_t comm = nullptr;
  SharedBuf ctrl;
  unsigned long long epoch[2] = {0, 0};
  std::vector<SharedBuf> results;
  void* xbuf = nullptr;             // packed column blocks of the NCCL form, grow-only
  size_t xbuf_bytes = 0;
  void* records_dev = nullptr;      // kMaxWorld PeerRecords, for the handle exchange
  int timeout_ms = 10000;
};

namespace {

struct DeviceScope {
  int prev = -1, dev;
  bool ok = true;
  explicit DeviceScope(int d) : dev(d) {
    if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
    if (prev != d) ok = cudaSetDevice(d) == cudaSuccess;
  }
  ~DeviceScope() {
    if (prev >= 0 && prev != dev) cudaSetDevice(prev);
  }
};

hc_status cuda_fail(hc_group* g, cudaError_t e, const char* what) {
  std::string msg = std::string(what) + ": " + cudaGetErrorString(e);
  cudaGetLastError();
  return hc::ctx_fail(g->ctx, e == cudaErrorMemoryAllocation ? HC_ERR_ALLOCATION_FAILED : HC_ERR_CUDA, msg.c_str());
}
hc_status nccl_fail(hc_group* g, ncclResult_t r, const char* what) {
  std::string msg = std::string(what) + ": " + nccl().GetErrorString(r);
  return hc::ctx_fail(g->ctx, HC_ERR_CUDA, msg.c_str());
}
#define HCG_CUDA(g, expr)                                      \
  do {                                                         \
    cudaError_t e__ = (expr);                                  \
    if (e__ != cudaSuccess) return cuda_fail(g, e__, #expr);   \
  } while (0)
#define HCG_NCCL(g, expr)                                      \
  do {                                                         \
    ncclResult_t r__ = (expr);                                 \
    if (r__ != ncclSuccess) return nccl_fail(g, r__, #expr);   \
  } while (0)

// Every rank contributes the record of one local buffer and receives everybody's; collective.
hc_status exchange_records(hc_group* g, const PeerRecord& mine, PeerRecord all[kMaxWorld]) {
  all[g->rank] = mine;
  if (g->world == 1) return HC_OK;
  cudaStream_t st = hc::ctx_stream(g->ctx);
  char* dev = (char*)g->records_dev;
  HCG_CUDA(g, cudaMemcpyAsync(dev + g->rank * sizeof(PeerRecord), &mine, sizeof mine, cudaMemcpyHostToDevice, st));
  HCG_NCCL(g, nccl().AllGather(dev + g->rank * sizeof(PeerRecord), dev, sizeof(PeerRecord), ncclChar, g->comm, st));
  HCG_CUDA(g, cudaMemcpyAsync(all, dev, g->world * sizeof(PeerRecord), cudaMemcpyDeviceToHost, st));
  HCG_CUDA(g, cudaStreamSynchronize(st));
  return HC_OK;
}

// Allocates `bytes` on this rank and maps the same allocation of every other rank; collective.
hc_status shared_create(hc_group* g, size_t bytes, SharedBuf* out) {
  SharedBuf sb;
  sb.bytes = bytes ? bytes : 1;
  // cudaMalloc, not the stream-ordered pool: only such memory can be exported to other processes.
  cudaError_t e = cudaMalloc(&sb.local, sb.bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    // The other ranks are inside the same collective: take part with an empty record, so that
    // nobody hangs, and report.
    PeerRecord none;
    memset(&none, 0, sizeof none);
    PeerRecord all[kMaxWorld];
    exchange_records(g, none, all);
    return hc::ctx_fail(g->ctx, HC_ERR_ALLOCATION_FAILED, "allocation of a group-shared buffer failed");
  }
  PeerRecord mine;
  memset(&mine, 0, sizeof mine);
  mine.pid = (int64_t)getpid();
  mine.ptr = (uint64_t)(uintptr_t)sb.local;
  mine.device = hc::ctx_device(g->ctx);
  if (g->world > 1) {
    e = cudaIpcGetMemHandle(&mine.handle, sb.local);
    if (e != cudaSuccess) cudaGetLastError();   // same-process ranks do not need it
  }
  PeerRecord all[kMaxWorld];
  hc_status s = exchange_records(g, mine, all);
  if (s != HC_OK) { cudaFree(sb.local); return s; }
  sb.peer[g->rank] = sb.local;
  bool failed = false;
  for (int r = 0; r < g->world; r++) {
    if (r == g->rank) continue;
    if (all[r].ptr == 0) { failed = true; continue; }
    if (all[r].pid == mine.pid) {
      // Another device of this process: its pointer is valid here once peer access is enabled.
      e = cudaDeviceEnablePeerAccess(all[r].device, 0);
      if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) failed = true;
      cudaGetLastError();
      sb.peer[r] = (void*)(uintptr_t)all[r].ptr;
    } else {
      e = cudaIpcOpenMemHandle(&sb.peer[r], all[r].handle, cudaIpcMemLazyEnablePeerAccess);
      if (e != cudaSuccess) { cudaGetLastError(); sb.peer[r] = nullptr; failed = true; }
      else sb.ipc_opened[r] = true;
    }
  }
  *out = sb;
  if (failed) return hc::ctx_fail(g->ctx, HC_ERR_CUDA, "a rank's shared buffer could not be mapped (allocation or peer access failed)");
  return HC_OK;
}

void shared_unmap(SharedBuf* sb, int world) {
  for (int r = 0; r < world; r++)
    if (sb->ipc_opened[r] && sb->peer[r]) {
      if (cudaIpcCloseMemHandle(sb->peer[r]) != cudaSuccess) cudaGetLastError();
      sb->peer[r] = nullptr;
      sb->ipc_opened[r] = false;
    }
}

// ---- flag barrier ---------------------------------------------------------------------------

struct BarrierArgs {
  unsigned long long* peer_counters[kMaxWorld];   // counters of set `set` in rank r's control block
  unsigned long long* my_counters;
  int rank, world, signal;
  unsigned long long epoch, limit_ns;
  unsigned int* status;
};

__device__ __forceinline__ unsigned long long timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Thread r tells rank r "this rank has reached `epoch`" and then waits until rank r has told this
// rank the same.  Launched as an ordinary kernel on the context's stream, so it starts when the
// work enqueued before it on this rank has completed.  The wait is bounded.
__global__ void group_barrier_kernel(const BarrierArgs a) {
  const int r = threadIdx.x;
  if (r >= a.world) return;
  if (a.signal) {
    __threadfence_system();
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(a.peer_counters[r] + a.rank), "l"(a.epoch) : "memory");
  }
  const unsigned long long t0 = timer_ns();
  for (;;) {
    unsigned long long seen;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(seen) : "l"(a.my_counters + r) : "memory");
    if (seen >= a.epoch) break;
    if (timer_ns() - t0 > a.limit_ns) {
      atomicOr(a.status, hc::kDevTimeoutBarrier);
      break;
    }
    __nanosleep(200);
  }
}

// Enqueues one barrier over counter set `set`.  With signal == false this rank waits without
// announcing itself (the self-test of the timeout path).
hc_status enqueue_barrier(hc_group* g, int set, bool signal, int limit_ms) {
  BarrierArgs a;
  memset(&a, 0, sizeof a);
  for (int r = 0; r < g->world; r++) {
    if (!g->ctrl.peer[r]) return hc::ctx_fail(g->ctx, HC_ERR_CUDA, "group control block of a rank is not mapped");
    a.peer_counters[r] = ((ControlBlock*)g->ctrl.peer[r])->arrived[set];
  }
  a.my_counters = ((ControlBlock*)g->ctrl.local)->arrived[set];
  a.rank = g->rank; a.world = g->world; a.signal = signal ? 1 : 0;
  a.epoch = ++g->epoch[set];
  a.limit_ns = (unsigned long long)limit_ms * 1000000ull;
  a.status = hc::ctx_status_word(g->ctx);
  group_barrier_kernel<<<1, 32, 0, hc::ctx_stream(g->ctx)>>>(a);
  hc::ctx_count_launches(g->ctx, 1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(g, e, "barrier launch");
  return HC_OK;
}

// ---- putting gathered column blocks into the row-major result ---------------------------------

struct UnpackJob {
  const char* src[kMaxWorld];     // packed block of rank r: rows x width_bytes[r]
  long long begin_bytes[kMaxWorld], width_bytes[kMaxWorld];
  char* dst;
  long long dst_pitch_bytes, rows;
};

// blockIdx.y = source block.  T = widest unit every address and width is a multiple of.
template <typename T>
__global__ void __launch_bounds__(256) unpack_blocks_kernel(const UnpackJob j) {
  const int r = blockIdx.y;
  const long long units = j.width_bytes[r] / (long long)sizeof(T);
  const long long total = j.rows * units;
  const T* src = (const T*)j.src[r];
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / units, c = i - row * units;
    *(T*)(j.dst + row * j.dst_pitch_bytes + j.begin_bytes[r] + c * (long long)sizeof(T)) = src[i];
  }
}

int64_t shard_begin(int64_t total, int world, int rank, int64_t* count) {
  const int64_t base = total / world, extra = total % world;
  *count = base + (rank < extra ? 1 : 0);
  return rank * base + (rank < extra ? rank : extra);
}

// Column blocks end on multiples of 256 (the kernel's tile width, which also keeps every block's
// first element 16-byte aligned) while that leaves every rank a block, else on multiples of 8,
// else anywhere.
void column_block(int64_t cols, int world, int rank, int64_t* begin, int64_t* count) {
  const int64_t units_of[3] = {256, 8, 1};
  for (int i = 0; i < 3; i++) {
    const int64_t unit = units_of[i];
    const int64_t units = (cols + unit - 1) / unit;
    if (units >= world || unit == 1) {
      int64_t c;
      const int64_t b = shard_begin(units, world, rank, &c);
      const int64_t lo = b * unit < cols ? b * unit : cols;
      const int64_t hi = (b + c) * unit < cols ? (b + c) * unit : cols;
      *begin = lo;
      *count = hi - lo;
      return;
    }
  }
}

// Every rank holds `bytes_of[r]` bytes at `base + offset_of[r]`, its own part filled in; afterwards
// every rank holds all parts.  One ncclAllGather when the parts are equal, one broadcast per
// rank (in one NCCL group) otherwise.
hc_status gather_parts(hc_group* g, char* base, const size_t offset_of[kMaxWorld], const size_t bytes_of[kMaxWorld]) {
  cudaStream_t st = hc::ctx_stream(g->ctx);
  bool equal = true;
  for (int r = 0; r < g->world; r++)
    if (bytes_of[r] != bytes_of[0] || offset_of[r] != r * bytes_of[0]) equal = false;
  if (equal) {
    if (bytes_of[0] == 0) return HC_OK;
    HCG_NCCL(g, nccl().AllGather(base + offset_of[g->rank], base, bytes_of[0], ncclChar, g->comm, st));
    return HC_OK;
  }
  HCG_NCCL(g, nccl().GroupStart());
  ncclResult_t first = ncclSuccess;
  for (int r = 0; r < g->world; r++) {
    if (bytes_of[r] == 0) continue;
    ncclResult_t x = nccl().Broadcast(base + offset_of[r], base + offset_of[r], bytes_of[r], ncclChar, r, g->comm, st);
    if (x != ncclSuccess && first == ncclSuccess) first = x;
  }
  HCG_NCCL(g, nccl().GroupEnd());
  if (first != ncclSuccess) return nccl_fail(g, first, "ncclBroadcast");
  return HC_OK;
}

}  // namespace

extern "C" {

hc_status hc_group_unique_id(void* id_out) {
  if (!id_out) return HC_ERR_INVALID_ARGUMENT;
  static_assert(sizeof(ncclUniqueId) == HC_GROUP_ID_BYTES, "id size");
  if (!nccl().ok) return HC_ERR_NOT_IMPLEMENTED;
  ncclUniqueId id;
  if (nccl().GetUniqueId(&id) != ncclSuccess) return HC_ERR_CUDA;
  memcpy(id_out, &id, sizeof id);
  return HC_OK;
}

hc_status hc_group_init(hc_ctx* ctx, int world, int rank, const void* id, hc_group** out) {
  if (!ctx || !out || world < 1 || world > kMaxWorld || rank < 0 || rank >= world || (world > 1 && !id))
    return HC_ERR_INVALID_ARGUMENT;
  *out = nullptr;
  std::lock_guard<std::mutex> lock(hc::ctx_mutex(ctx));
  DeviceScope dev(hc::ctx_device(ctx));
  if (!dev.ok) return hc::ctx_fail(ctx, HC_ERR_CUDA, "cannot make the context's device current");
  if (world > 1 && !nccl().ok)
    return hc::ctx_fail(ctx, HC_ERR_NOT_IMPLEMENTED, "no usable libnccl.so.2 in this process or on the library path");
  hc_group* g = new (std::nothrow) hc_group();
  if (!g) return HC_ERR_ALLOCATION_FAILED;
  g->ctx = ctx; g->world = world; g->rank = rank;
  hc_status s = HC_OK;
  if (world > 1) {
    ncclUniqueId uid;
    memcpy(&uid, id, sizeof uid);
    ncclResult_t r = nccl().CommInitRank(&g->comm, world, uid, rank);
    if (r != ncclSuccess) {
      s = nccl_fail(g, r, "ncclCommInitRank");
      delete g;
      return s;
    }
    cudaError_t e = cudaMalloc(&g->records_dev, kMaxWorld * sizeof(PeerRecord));
    if (e != cudaSuccess) {
      s = cuda_fail(g, e, "group setup");
      nccl().CommDestroy(g->comm);
      delete g;
      return s;
    }
  }
  s = shared_create(g, sizeof(ControlBlock), &g->ctrl);
  if (s == HC_OK) {
    cudaError_t e = cudaMemsetAsync(g->ctrl.local, 0, sizeof(ControlBlock), hc::ctx_stream(ctx));
    if (e == cudaSuccess) e = cudaStreamSynchronize(hc::ctx_stream(ctx));
    if (e != cudaSuccess) s = cuda_fail(g, e, "group setup");
  }
  if (s == HC_OK && world > 1) {
    // Nobody may signal a control block that its owner has not cleared yet: one exchange more.
    PeerRecord none, all[kMaxWorld];
    memset(&none, 0, sizeof none);
    s = exchange_records(g, none, all);
  }
  if (s != HC_OK) {
    shared_unmap(&g->ctrl, world);
    if (g->ctrl.local) cudaFree(g->ctrl.local);
    if (g->records_dev) cudaFree(g->records_dev);
    if (g->comm) nccl().CommDestroy(g->comm);
    delete g;
    return s;
  }
  *out = g;
  return HC_OK;
}

void hc_group_destroy(hc_group* g) {
  if (!g) return;
  std::lock_guard<std::mutex> lock(hc::ctx_mutex(g->ctx));
  DeviceScope dev(hc::ctx_device(g->ctx));
  cudaStreamSynchronize(hc::ctx_stream(g->ctx));
  for (auto& sb : g->results) {
    shared_unmap(&sb, g->world);
    if (sb.local) cudaFree(sb.local);
  }
  shared_unmap(&g->ctrl, g->world);
  if (g->comm) nccl().CommDestroy(g->comm);   // collective: every rank's destroy meets here
  if (g->ctrl.local) cudaFree(g->ctrl.local);
  if (g->records_dev) cudaFree(g->records_dev);
  if (g->xbuf) hc::ctx_device_free(g->ctx, g->xbuf);
  cudaGetLastError();
  delete g;
}

int hc_group_rank(hc_group* g) { return g ? g->rank : -1; }
int hc_group_world(hc_group* g) { return g ? g->world : 0; }

hc_status hc_group_set_timeout_ms(hc_group* g, int ms) {
  if (!g || ms < 1 || ms > 600000) return HC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(hc::ctx_mutex(g->ctx));
  g->timeout_ms = ms;
  return HC_OK;
}

hc_status hc_shard_range(int64_t total, int world, int rank, int64_t* begin, int64_t* count) {
  if (total < 0 || world < 1 || rank < 0 || rank >= world || !begin || !count) return HC_ERR_INVALID_ARGUMENT;
  *begin = shard_begin(total, world, rank, count);
  return HC_OK;
}

hc_status hc_column_block(int64_t cols, int world, int rank, int64_t* begin, int64_t* count) {
  if (cols < 0 || world < 1 || rank < 0 || rank >= world || !begin || !count) return HC_ERR_INVALID_ARGUMENT;
  column_block(cols, world, rank, begin, count);
  return HC_OK;
}

hc_status hc_group_result_alloc(hc_group* g, size_t bytes, void** dptr) {
  if (!g || !dptr) return HC_ERR_INVALID_ARGUMENT;
  *dptr = nullptr;
  std::lock_guard<std::mutex> lock(hc::ctx_mutex(g->ctx));
  DeviceScope dev(hc::ctx_device(g->ctx));
  SharedBuf sb;
  hc_status s = shared_create(g, bytes, &sb);
  if (s != HC_OK) {
    shared_unmap(&sb, g->world);
    if (sb.local) cudaFree(sb.local);
    return s;
  }
  g->results.push_back(sb);
  *dptr = sb.local;
  return HC_OK;
}

hc_status hc_group_result_free(hc_group* g, void* dptr) {
  if (!g) return HC_ERR_INVALID_ARGUMENT;
  if (!dptr) return HC_OK;
  std::lock_guard<std::mutex> lock(hc::ctx_mutex(g->ctx));
  DeviceScope dev(hc::ctx_device(g->ctx));
  for (size_t i = 0; i < g->results.size(); i++) {
    if (g->results[i].local != dptr) continue;
    // Two barriers on the stream and a host wait: nobody unmaps while a peer may still store
    // into the mapping, nobody frees while a peer still has it mapped.
    hc_status s = enqueue_barrier(g, 1, true, g->timeout_ms);
    if (s != HC_OK) return s;
    HCG_CUDA(g, cudaStreamSynchronize(hc::ctx_stream(g->ctx)));
    shared_unmap(&g->results[i], g->world);
    s = enqueue_barrier(g, 1, true, g->timeout_ms);
    if (s != HC_OK) return s;
    HCG_CUDA(g, cudaStreamSynchronize(hc::ctx_stream(g->ctx)));
    HCG_CUDA(g, cudaFree(dptr));
    g->results.erase(g->results.begin() + (long)i);
    return HC_OK;
  }
  return hc::ctx_fail(g->ctx, HC_ERR_INVALID_ARGUMENT, "not a buffer of hc_group_result_alloc on this group");
}

hc_status hc_group_barrier(hc_group* g) {
  if (!g) return HC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(hc::ctx_mutex(g->ctx));
  DeviceScope dev(hc::ctx_device(g->ctx));
  return enqueue_barrier(g, 1, true, g->timeout_ms);
}

hc_status hc_group_selftest_missing_peer(hc_group* g, int limit_ms) {
  if (!g || limit_ms < 1 || limit_ms > 1000) return HC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(hc::ctx_mutex(g->ctx));
  DeviceScope dev(hc::ctx_device(g->ctx));
  // A barrier in which this rank does not announce itself: its own counter stays behind, exactly
  // what a rank sees whose peer never arrives.  The wait gives up after `limit_ms`.
  hc_status s = enqueue_barrier(g, 1, false, limit_ms);
  if (s != HC_OK) return s;
  // Bring the counter up to date so that the group stays usable (local store, stream-ordered).
  unsigned long long* mine = ((ControlBlock*)g->ctrl.local)->arrived[1] + g->rank;
  HCG_CUDA(g, cudaMemcpyAsync(mine, &g->epoch[1], sizeof(unsigned long long), cudaMemcpyHostToDevice, hc::ctx_stream(g->ctx)));
  HCG_CUDA(g, cudaStreamSynchronize(hc::ctx_stream(g->ctx)));
  return HC_OK;
}

hc_status hc_batched_matmul_sharded(hc_group* g, hc_dtype dtype, int64_t matrix_count, const void* a_shard, int trans_a,
                                    const void* b_shard, int trans_b, int trans_out, int64_t rows, int64_t inner,
                                    int64_t cols, void* out, int gather) {
  if (!g) return HC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(hc::ctx_mutex(g->ctx));
  DeviceScope dev(hc::ctx_device(g->ctx));
  if (matrix_count < 0 || rows < 0 || inner < 0 || cols < 0)
    return hc::ctx_fail(g->ctx, HC_ERR_INVALID_ARGUMENT, "negative dimension");
  if (dtype != HC_F16 && dtype != HC_F32)
    return hc::ctx_fail(g->ctx, HC_ERR_NOT_IMPLEMENTED, "matmul: only float16 and float32 are implemented");
  int64_t count;
  const int64_t begin = shard_begin(matrix_count, g->world, g->rank, &count);
  const int64_t eb = dtype == HC_F16 ? 2 : 4;
  int64_t per_matrix, whole;
  if (__builtin_mul_overflow(rows, cols, &per_matrix) || __builtin_mul_overflow(per_matrix, eb, &per_matrix) ||
      __builtin_mul_overflow(per_matrix, matrix_count, &whole))
    return hc::ctx_fail(g->ctx, HC_ERR_INVALID_ARGUMENT, "operand size overflows int64");
  char* mine = (char*)out + (gather ? begin * per_matrix : 0);
  hc_status s = hc::ctx_run_batched(g->ctx, dtype, count, a_shard, trans_a, b_shard, trans_b, trans_out, rows, inner,
                                    cols, mine);
  if (s != HC_OK || !gather || g->world == 1) return s;
  size_t off[kMaxWorld], len[kMaxWorld];
  for (int r = 0; r < g->world; r++) {
    int64_t c;
    const int64_t b = shard_begin(matrix_count, g->world, r, &c);
    off[r] = (size_t)(b * per_matrix);
    len[r] = (size_t)(c * per_matrix);
  }
  return gather_parts(g, (char*)out, off, len);
}

hc_status hc_matmul_nsplit_allgather(hc_group* g, hc_dtype dtype, const void* a, int trans_a, const void* b,
                                     int trans_b, int64_t rows, int64_t inner, int64_t cols, void* out, int fused) {
  if (!g) return HC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(hc::ctx_mutex(g->ctx));
  DeviceScope dev(hc::ctx_device(g->ctx));
  if (rows < 0 || inner < 0 || cols < 0) return hc::ctx_fail(g->ctx, HC_ERR_INVALID_ARGUMENT, "negative dimension");
  if (dtype != HC_F16 && dtype != HC_F32)
    return hc::ctx_fail(g->ctx, HC_ERR_NOT_IMPLEMENTED, "matmul: only float16 and float32 are implemented");
  const int64_t eb = dtype == HC_F16 ? 2 : 4;
  int64_t total_bytes;
  if (__builtin_mul_overflow(rows, cols, &total_bytes) || __builtin_mul_overflow(total_bytes, eb, &total_bytes))
    return hc::ctx_fail(g->ctx, HC_ERR_INVALID_ARGUMENT, "operand size overflows int64");
  if (rows == 0 || cols == 0) return HC_OK;
  if (!out) return hc::ctx_fail(g->ctx, HC_ERR_INVALID_ARGUMENT, "null operand");
  int64_t begin[kMaxWorld], width[kMaxWorld];
  for (int r = 0; r < g->world; r++) column_block(cols, g->world, r, &begin[r], &width[r]);
  const int me = g->rank;

  if (fused) {
    if (inner == 0) return hc::ctx_fail(g->ctx, HC_ERR_INVALID_ARGUMENT, "the fused exchange needs a non-empty contraction");
    const SharedBuf* sb = nullptr;
    for (const auto& x : g->results)
      if (x.local == out) sb = &x;
    if (!sb || sb->bytes < (size_t)total_bytes)
      return hc::ctx_fail(g->ctx, HC_ERR_INVALID_ARGUMENT,
                          "the fused exchange stores into every rank's result: `out` must come from hc_group_result_alloc and hold rows x cols");
    // Entry barrier: every rank has finished, on its stream, whatever it did with the previous
    // contents of its result before any peer overwrites them.
    hc_status s = enqueue_barrier(g, 0, true, g->timeout_ms);
    if (s != HC_OK) return s;
    void* extra[kMaxWorld];
    int n_extra = 0;
    for (int r = 0; r < g->world; r++)
      if (r != me) extra[n_extra++] = (char*)sb->peer[r] + begin[me] * eb;
    if (width[me] > 0) {
      s = hc::ctx_run_colblock(g->ctx, dtype, a, trans_a, b, trans_b, rows, inner, cols, begin[me], width[me],
                               (char*)out + begin[me] * eb, cols, extra, n_extra);
      if (s != HC_OK) return s;
    }
    // Exit barrier: when it has passed on this rank, every rank's kernel - and with it its stores
    // into this rank's result - has completed.
    return enqueue_barrier(g, 1, true, g->timeout_ms);
  }

  if (g->world == 1)
    return hc::ctx_run_colblock(g->ctx, dtype, a, trans_a, b, trans_b, rows, inner, cols, 0, cols, out, cols, nullptr, 0);

  // Packed blocks, rank after rank: block r is rows x width[r], dense.
  size_t off[kMaxWorld], len[kMaxWorld];
  size_t pos = 0;
  for (int r = 0; r < g->world; r++) {
    off[r] = pos;
    len[r] = (size_t)(rows * width[r] * eb);
    pos += len[r];
  }
  if (pos > g->xbuf_bytes) {
    void* fresh = nullptr;
    hc_status s = hc::ctx_device_alloc(g->ctx, &fresh, pos);
    if (s != HC_OK) return s;
    hc::ctx_device_free(g->ctx, g->xbuf);
    g->xbuf = fresh;
    g->xbuf_bytes = pos;
  }
  char* xb = (char*)g->xbuf;
  if (width[me] > 0) {
    hc_status s = hc::ctx_run_colblock(g->ctx, dtype, a, trans_a, b, trans_b, rows, inner, cols, begin[me], width[me],
                                       xb + off[me], width[me], nullptr, 0);
    if (s != HC_OK) return s;
  }
  hc_status s = gather_parts(g, xb, off, len);
  if (s != HC_OK) return s;
  UnpackJob j;
  memset(&j, 0, sizeof j);
  uintptr_t align_or = (uintptr_t)out | (uintptr_t)(cols * eb);
  for (int r = 0; r < g->world; r++) {
    j.src[r] = xb + off[r];
    j.begin_bytes[r] = begin[r] * eb;
    j.width_bytes[r] = width[r] * eb;
    align_or |= (uintptr_t)j.src[r] | (uintptr_t)j.begin_bytes[r] | (uintptr_t)j.width_bytes[r];
  }
  j.dst = (char*)out; j.dst_pitch_bytes = cols * eb; j.rows = rows;
  const dim3 grid(148 * 4, (unsigned)g->world);
  cudaStream_t st = hc::ctx_stream(g->ctx);
  if ((align_or & 15) == 0) unpack_blocks_kernel<uint4><<<grid, 256, 0, st>>>(j);
  else if ((align_or & 3) == 0) unpack_blocks_kernel<uint32_t><<<grid, 256, 0, st>>>(j);
  else unpack_blocks_kernel<uint16_t><<<grid, 256, 0, st>>>(j);
  hc::ctx_count_launches(g->ctx, 1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(g, e, "unpack launch");
  return HC_OK;
}

}  // extern "C"

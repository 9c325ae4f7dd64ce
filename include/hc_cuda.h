/*
 * hc_cuda.h - C ABI of libhccuda, the sm_100a implementation of Honeycrisp's dense
 * matrix-product hot path (Backend.matmul / Backend.batchedMatmul, float32 and float16).
 *
 * This is the surface a Swift `CUDABackend: Backend` binds through a module map
 * (`module CHCCuda { header "hc_cuda.h" link "hccuda" export * }`), and the surface the
 * ctypes host mirror and the tests call.  Plain C: pointers, sizes, int status codes.
 * No exceptions or aborts cross it, there is no CPU fallback behind it, and nothing in it
 * depends on PyTorch.
 *
 * Conventions shared by all matrix entry points (they are the reference's):
 *   - every operand is dense, row-major and contiguous;
 *   - `rows` x `cols` is the shape of op(a)*op(b), `inner` the contracted length;
 *   - `a` is stored [rows,inner], or [inner,rows] when trans_a; `b` is stored [inner,cols],
 *     or [cols,inner] when trans_b; `out` is [rows,cols], or [cols,rows] when trans_out;
 *   - batched calls hold `matrix_count` such matrices back to back, no padding, equal counts;
 *   - float16 accumulates in float32 and rounds once (nearest-even, overflow -> +-inf).
 * Pointers are device pointers on the context's device unless a function says "host".
 * Work is enqueued on the context's stream and the call returns without waiting; inputs must
 * stay alive until the stream has passed the call (hc_sync / hc_event_wait).
 * All functions are thread-safe; calls on one context are ordered by a mutex, which is the
 * same discipline as the reference backends' single worker thread
 * (Sources/Honeycrisp/BackendCPU.swift:235-248).
 */
#ifndef HC_CUDA_H_
#define HC_CUDA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct hc_ctx hc_ctx;     /* one device, one stream, one allocator pool */
typedef struct hc_event hc_event; /* completion marker on the context's stream */

/* Status codes.  The first three after OK map one-to-one onto the reference's BackendError
 * cases (Sources/Honeycrisp/Backend.swift:6-16): allocationFailed, kernelFailed,
 * notImplemented. */
typedef enum hc_status {
  HC_OK = 0,
  HC_ERR_ALLOCATION_FAILED = 1,
  HC_ERR_KERNEL_FAILED = 2,
  HC_ERR_NOT_IMPLEMENTED = 3,
  HC_ERR_INVALID_ARGUMENT = 4, /* the reference traps these earlier with #alwaysAssert
                                  (Sources/Honeycrisp/Linalg.swift:52-59,90-104) */
  HC_ERR_TIMEOUT = 5,          /* a bounded device-side wait gave up (inside a kernel, or for
                                  another rank of a device group); context stays usable */
  HC_ERR_CUDA = 6              /* any other CUDA runtime/driver error; see hc_last_error */
} hc_status;

/* Tensor.DType subset in scope (Sources/Honeycrisp/Tensor.swift: DType). int64 products are
 * legal on the reference's CPU backend but outside this library: HC_ERR_NOT_IMPLEMENTED. */
typedef enum hc_dtype { HC_F16 = 0, HC_F32 = 1 } hc_dtype;

/* Which kernel serves a product.  AUTO is what a backend uses; the rest exist for tests,
 * benchmarks and as the GPU-side cross-check of the tensor-core paths. */
typedef enum hc_kernel {
  HC_KERNEL_AUTO = 0,
  HC_KERNEL_SIMT = 1,       /* CUDA-core kernel, fused multiply-add, any shape/alignment */
  HC_KERNEL_SIMT_EXACT = 2, /* same, separate multiply and add in k order: bit-identical to
                               the reference CPU loop (BackendCPU.swift:1290-1300) */
  HC_KERNEL_TENSOR = 3      /* tcgen05 path: fp16 direct; fp32 as 3xTF32 split operands.  Operands
                               whose base or row pitch is not 16-byte aligned are repacked into
                               the context's work area first. */
} hc_kernel;

typedef struct hc_launch_info {
  int kernel;          /* hc_kernel actually used (never AUTO) */
  int tile_m, tile_n, tile_k;
  int stages;
  int grid, block;
  int64_t tiles;       /* output tiles over all matrices */
  int64_t flops;       /* 2*matrix_count*rows*inner*cols, the reference's own convention
                          (Sources/Honeycrisp/BackendWrapper.swift:485,499) */
  size_t scratch_bytes;/* global memory used beyond inputs and outputs */
} hc_launch_info;

/* ---- context, memory, ordering ---------------------------------------------------------- */

/* Create a context on CUDA device `device` with its own non-blocking stream.
 * Replaces: `try CUDABackend()` taking the place of MPSBackend.init
 * (Sources/Honeycrisp/BackendMPS.swift:352-375). */
hc_status hc_init(int device, hc_ctx** out);
void hc_destroy(hc_ctx* ctx);

/* Run this context's work on a stream the caller owns (a `cudaStream_t` passed as void*);
 * NULL returns to the context's own stream.  The caller keeps the stream alive.
 * The context's OWN stream is private to the library: record events on it, make other streams
 * wait for it, but launch your own kernels on a stream you pass here.  On its own stream the
 * library lets a product's operand loads start while the product enqueued just before it is
 * still finishing, when that product cannot have written them - which it can only know about
 * kernels it launched itself.  On a caller's stream every product waits for all earlier work. */
hc_status hc_set_stream(hc_ctx* ctx, void* cuda_stream);
void* hc_get_stream(hc_ctx* ctx);
int hc_get_device(hc_ctx* ctx);

/* Stream-ordered allocation; `bytes == 0` allocates one byte, as the reference's GPU backend
 * does (Sources/Honeycrisp/BackendMPS.swift:538-540).
 * Replaces: MPSBackend.allocateBuf (BackendMPS.swift:500-527), CPUBackend.allocate
 * (BackendCPU.swift:250-253).
 * The memory comes from a pool the context owns, which keeps up to 8 GiB of freed memory for
 * reuse (environment HC_POOL_RETAIN_MB at hc_init) instead of returning it to the driver at
 * every synchronisation.  Free buffers before hc_destroy: what is still allocated then stays
 * mapped (kernels in flight may use it) and is reclaimed only when the process ends. */
hc_status hc_alloc(hc_ctx* ctx, size_t bytes, void** dptr);
hc_status hc_free(hc_ctx* ctx, void* dptr);

/* Copies between host and device, ordered on the stream; both return after the copy has
 * been enqueued (h2d from pageable memory has been staged).  hc_d2h needs hc_sync or an
 * event wait before the host reads `dst`.
 * Replaces: Tensor.Data.onCPU / MPSBackend.gpuBuffer staging (BackendMPS.swift:585-620). */
hc_status hc_h2d(hc_ctx* ctx, void* dst_device, const void* src_host, size_t bytes);
hc_status hc_d2h(hc_ctx* ctx, void* dst_host, const void* src_device, size_t bytes);
/* Read a device buffer back to (pinned) host memory without stalling the context's stream: the
 * copy runs on a side stream after everything enqueued so far, later products keep running, and
 * `*done` completes when the bytes are in `dst_host` (hc_event_wait, then hc_event_destroy).  The
 * device buffer must stay alive and unmodified until then.  Mirrors awaiting one result's data
 * while the backend works on the next (Sources/Honeycrisp/Tensor.swift:618-621; the reference's
 * GPU backend completes each command buffer on its own, BackendMPS.swift:2694-2720). */
hc_status hc_d2h_async(hc_ctx* ctx, void* dst_host, const void* src_device, size_t bytes,
                       hc_event** done);
/* The other direction: copy (pinned) host memory into a device buffer on a side stream, ordered
 * after everything enqueued so far (so earlier readers of `dst_device` are done) but not ahead
 * of anything enqueued later: work that reads `dst_device` must be told to wait with
 * hc_enqueue_wait(ctx, *done).  This is how the operands of the next step are brought in while
 * the results of the current one are still being read back (host links are full duplex).
 * Mirrors Backend.collection (Sources/Honeycrisp/Backend.swift:794-800) issued ahead of use. */
hc_status hc_h2d_async(hc_ctx* ctx, void* dst_device, const void* src_host, size_t bytes,
                       hc_event** done);
/* Work enqueued on the context after this call starts only when `ev` has completed; the host
 * does not block.  (The reference expresses the same dependency by awaiting the input Tensor's
 * Task inside the consuming operation, Sources/Honeycrisp/Tensor.swift:618-621.) */
hc_status hc_enqueue_wait(hc_ctx* ctx, hc_event* ev);
hc_status hc_sync(hc_ctx* ctx);

/* Completion markers; they back Tensor.Data.wait() (Sources/Honeycrisp/Tensor.swift:69-85,
 * 618-621), like the command-buffer completion Task of the reference's GPU backend
 * (BackendMPS.swift:2694-2720).  hc_event_wait also reports a device-side timeout or kernel
 * failure recorded before the event. */
hc_status hc_event_record(hc_ctx* ctx, hc_event** out);
hc_status hc_event_wait(hc_event* ev);
/* Milliseconds between two completed events of the same context. */
hc_status hc_event_elapsed_ms(hc_event* start, hc_event* stop, float* ms);
/* A marker may be destroyed after its context (garbage-collected hosts release buffers late);
 * waiting on it or timing with it after hc_destroy is an error of the caller. */
void hc_event_destroy(hc_event* ev);

/* ---- the hot path ------------------------------------------------------------------------ */

/* out = trans_out(op(a) * op(b)).
 * Replaces: Backend.matmul(a:transA:b:transB:transOut:rows:inner:cols:dtype:)
 * (Sources/Honeycrisp/Backend.swift:650-658; CPU body BackendCPU.swift:1222-1232).
 * The products may use the context's work area, a device buffer that only grows (to the
 * largest need seen: the low TF32 halves of float32 operands, float16 operands repacked to an
 * aligned pitch, and at most 256 MiB of float32 partial sums when a long contraction over few
 * outputs is cut into parts); growing it is the only allocation a product makes, and it is
 * stream-ordered from the context's pool (no device-wide synchronisation).  A CUDA graph that
 * captured products is invalid once a later, larger product has grown the work area: run the
 * largest product once before capturing.  The context remembers how it prepared its most recent
 * products (tile plan, tensor maps), so repeating a product on the same buffers costs the host
 * little more than the launch.  Results do not depend on how the work is tiled, cut or
 * scheduled: the same call gives the same bits.  Under HC_KERNEL_AUTO products too small for a
 * tensor-core tile run on the CUDA cores in the reference's own arithmetic (separate multiply and
 * add, k ascending: bit-identical to BackendCPU.swift:1290-1300). */
hc_status hc_matmul(hc_ctx* ctx, hc_dtype dtype, const void* a, int trans_a, const void* b,
                    int trans_b, int trans_out, int64_t rows, int64_t inner, int64_t cols,
                    void* out);

/* The same for `matrix_count` independent products.
 * Replaces: Backend.batchedMatmul(matrixCount:a:transA:b:transB:transOut:rows:inner:cols:dtype:)
 * (Sources/Honeycrisp/Backend.swift:661-669; CPU body BackendCPU.swift:1234-1313). */
hc_status hc_batched_matmul(hc_ctx* ctx, hc_dtype dtype, int64_t matrix_count, const void* a,
                            int trans_a, const void* b, int trans_b, int trans_out,
                            int64_t rows, int64_t inner, int64_t cols, void* out);

/* As hc_batched_matmul with the kernel chosen by the caller. */
hc_status hc_batched_matmul_ex(hc_ctx* ctx, hc_kernel kernel, hc_dtype dtype,
                               int64_t matrix_count, const void* a, int trans_a, const void* b,
                               int trans_b, int trans_out, int64_t rows, int64_t inner,
                               int64_t cols, void* out);

/* Host-buffer form of the batched product: operands and result live in HOST memory; the call
 * stages them to the device, runs the product and copies the result back before returning.
 * This is what a backend does for operands of a foreign Tensor.Data type, which the reference
 * wraps through onCPU (Sources/Honeycrisp/BackendMPS.swift:585-620), followed by the caller
 * reading the result (Tensor.floats()).  Pinned host memory makes the copies asynchronous
 * DMA; pageable memory works but is slower. */
hc_status hc_batched_matmul_host(hc_ctx* ctx, hc_dtype dtype, int64_t matrix_count,
                                 const void* a_host, int trans_a, const void* b_host,
                                 int trans_b, int trans_out, int64_t rows, int64_t inner,
                                 int64_t cols, void* out_host);

/* The same, pipelined: the call enqueues copy-in, product and copy-out on three streams and
 * returns; up to two products are in flight, so the copy-in of one overlaps the product and the
 * copy-out of the one before (host links are full duplex).  `out_host` is valid after hc_host_sync
 * (or after two further _async calls).  Use pinned host memory; pageable memory serialises the
 * copies.  This is the asynchronous form the reference's backends have by construction: a
 * product returns a Tensor whose data is awaited later (Sources/Honeycrisp/Tensor.swift:618-621). */
hc_status hc_batched_matmul_host_async(hc_ctx* ctx, hc_dtype dtype, int64_t matrix_count,
                                       const void* a_host, int trans_a, const void* b_host,
                                       int trans_b, int trans_out, int64_t rows, int64_t inner,
                                       int64_t cols, void* out_host);
hc_status hc_host_sync(hc_ctx* ctx);

/* One column block of a product, for splitting a large GEMM over devices: computes columns
 * [col_begin, col_begin+col_count) of op(a)*op(b) (of its transpose's rows when trans_out) and
 * writes them in place into the FULL-size `out`.  `b` is the full operand; only the block's
 * part of it is read.  Each device of a group calls this with its own block; the blocks are
 * then exchanged (all-gather) by the caller.  No counterpart in the reference, which has no
 * multi-device code; the contract is "equals the same columns of hc_matmul". */
hc_status hc_matmul_colblock(hc_ctx* ctx, hc_kernel kernel, hc_dtype dtype, const void* a,
                             int trans_a, const void* b, int trans_b, int trans_out,
                             int64_t rows, int64_t inner, int64_t cols, int64_t col_begin,
                             int64_t col_count, void* out);

/* ---- around a Linear layer (next to the hot path) ------------------------------------------ */

/* out[rows,out_count] = x[rows,in_count] * weight[in_count,out_count] + bias[out_count], the
 * bias added in the product's epilogue.  `bias` may be NULL.  Numerically this is the
 * reference's two operations: the product rounded to `dtype`, then a broadcast add in `dtype`.
 * Replaces: Linear.callAsFunction (Sources/Honeycrisp/Trainable.swift:530-546) =
 * Tensor.matmul + Backend.binaryOp(.add) (Backend.swift:178-185, CPU body BackendCPU.swift:267-306). */
hc_status hc_linear_forward(hc_ctx* ctx, hc_dtype dtype, const void* x, const void* weight,
                            const void* bias, int64_t rows, int64_t in_count, int64_t out_count,
                            void* out);
/* out[cols] = sum over rows of x[rows,cols]: the bias gradient of a Linear layer.  One float
 * accumulator per column, rows in ascending order, narrowed once.
 * Replaces: Backend.reduce(.sum) over the leading axis as issued by reduceBroadcast
 * (Backend.swift:524-531; CPU body BackendCPU.swift:808-827; use at Tensor.swift:865-868). */
hc_status hc_column_sum(hc_ctx* ctx, hc_dtype dtype, const void* x, int64_t rows, int64_t cols,
                        void* out);
/* Elementwise dtype conversion (Linear's castParams).
 * Replaces: Backend.cast (Backend.swift:489-494). */
hc_status hc_cast(hc_ctx* ctx, hc_dtype from, hc_dtype to, const void* x, int64_t count, void* out);
/* out = a + b on equal shapes: gradient accumulation of a parameter used more than once.
 * Replaces: Backend.binaryOp(.add) without broadcasting (use at Tensor.swift:370-372,
 * Trainable.swift:258-266). */
hc_status hc_add(hc_ctx* ctx, hc_dtype dtype, const void* a, const void* b, int64_t count, void* out);

/* out[0..count) = `value`, narrowed once to `dtype` (round to nearest even for float16): a tensor
 * filled with a constant, created on the device.
 * Replaces: Backend.constant (Backend.swift:787-791; CPU body BackendCPU.swift:1796-1815, which
 * also goes through Float for the float types). */
hc_status hc_constant(hc_ctx* ctx, hc_dtype dtype, float value, int64_t count, void* out);

/* out[cols,rows] = in[rows,cols]^T for `matrix_count` matrices: the materialising `t()` of the
 * reference (a gather through axisPermutation, Sources/Honeycrisp/Index.swift:238-266,359-362;
 * Backend.swift:609-616,803-805).  A backend that keeps its tensors' layouts would instead pass
 * the transpose as a flag of the product; this exists because the reference's benchmark times the
 * two together (Sources/HCMatrixBench/Entrypoint.swift:17). */
hc_status hc_transpose(hc_ctx* ctx, hc_dtype dtype, int64_t matrix_count, const void* in,
                       int64_t rows, int64_t cols, void* out);

/* `count` samples of Honeycrisp's generator, bit-compatible with its CPU backend for the uniform
 * distribution (normal samples go through logf/cosf/sinf and agree to a few ulps): Philox-4x32-10
 * keyed by `seed`, counter starting at `offset`.  `*next_offset` receives the generator's offset
 * after the call (the state is the pair [seed, offset]).  normal == 0: U[0,1]; else N(0,1).
 * Replaces: RandomGenerator._sample (Sources/Honeycrisp/BackendCPU.swift:78-123,177-221), which
 * backs Tensor(rand:) / Tensor(randn:). */
hc_status hc_random(hc_ctx* ctx, int normal, hc_dtype dtype, uint64_t seed, uint64_t offset,
                    int64_t count, void* out, uint64_t* next_offset);

/* hc_matmul_colblock fused with the exchange: every finished tile of the block is stored into
 * `out` AND into the same place of up to 7 other devices' full-size results (`peer_outs`,
 * pointers obtained with hc_ipc_open), from the kernel's epilogue, over NVLink peer stores.
 * When every device of a group has run its call and synchronised, and the group has passed a
 * host-side barrier, every device holds the complete product - no separate all-gather.
 * Tensor-core kernel only; results must be 16-byte aligned with 16-byte row pitch.
 * No counterpart in the reference (single-device). */
hc_status hc_matmul_colblock_push(hc_ctx* ctx, hc_dtype dtype, const void* a, int trans_a,
                                  const void* b, int trans_b, int trans_out, int64_t rows,
                                  int64_t inner, int64_t cols, int64_t col_begin,
                                  int64_t col_count, void* out, void* const* peer_outs,
                                  int n_peers);

/* Device memory that other processes on the box can map (one process per GPU), and the
 * handle exchange for it (CUDA IPC; 64-byte opaque handles travel over any host channel).
 * No counterpart in the reference. */
#define HC_IPC_HANDLE_BYTES 64
hc_status hc_shared_alloc(hc_ctx* ctx, size_t bytes, void** dptr);
hc_status hc_shared_free(hc_ctx* ctx, void* dptr);
hc_status hc_ipc_export(hc_ctx* ctx, void* dptr, void* handle_out);
hc_status hc_ipc_open(hc_ctx* ctx, const void* handle, void** dptr);
hc_status hc_ipc_close(hc_ctx* ctx, void* dptr);

/* ---- products split over the GPUs of one box ------------------------------------------------ */
/* No counterpart in the reference, which has no multi-device code (a Backend holds one device,
 * Sources/Honeycrisp/BackendMPS.swift:352); the contract of every entry point is "equals the
 * single-device result of the same call".  They extend the two primitives of
 * Sources/Honeycrisp/Backend.swift:650-669.
 *
 * A group is one rank's handle on `world` contexts, one per GPU (at most 8).  Ranks are
 * processes (one per GPU) or threads of one process (one host driving several devices); either
 * way every rank creates its own context and calls hc_group_init with the same 128-byte id,
 * which rank 0 makes with hc_group_unique_id and hands to the others over any host channel.
 * The calls marked "collective" must be made by every rank, in the same order.  NCCL is looked
 * up at run time (a copy already loaded into the process, else HC_NCCL_LIB, else libnccl.so.2
 * on the library path); without it groups of one rank still work. */
typedef struct hc_group hc_group;
#define HC_GROUP_ID_BYTES 128
hc_status hc_group_unique_id(void* id_out);
hc_status hc_group_init(hc_ctx* ctx, int world, int rank, const void* id, hc_group** out); /* collective */
void hc_group_destroy(hc_group* g);                                                        /* collective */
int hc_group_rank(hc_group* g);
int hc_group_world(hc_group* g);
/* Limit of every device-side wait for another rank (default 10 000 ms).  When it runs out the
 * waiting kernel returns, and hc_check_device_status / hc_event_wait report HC_ERR_TIMEOUT. */
hc_status hc_group_set_timeout_ms(hc_group* g, int ms);

/* The partitions, as pure host arithmetic (no device, no group): rank `rank` of `world` owns
 * matrices [begin, begin+count) of a batch - contiguous ranges that differ by at most one - and
 * columns [begin, begin+count) of a split product, with block boundaries on multiples of 256
 * columns (the kernel's tile width) while that leaves every rank a block, else on multiples of 8. */
hc_status hc_shard_range(int64_t total, int world, int rank, int64_t* begin, int64_t* count);
hc_status hc_column_block(int64_t cols, int world, int rank, int64_t* begin, int64_t* count);

/* This rank's share of Backend.batchedMatmul over `matrix_count` matrices: `a_shard` and
 * `b_shard` hold the matrices of hc_shard_range(matrix_count, world, rank), back to back.
 * gather == 0: `out` receives the results of those matrices; nothing is exchanged.
 * gather != 0: `out` is the result buffer of the WHOLE batch on every rank; each rank writes its
 * range in place and the ranges are exchanged with one ncclAllGather (one ncclBroadcast per rank
 * when the ranges differ in size) - the batch dimension is contiguous, nothing is re-laid.
 * Collective when gather != 0. */
hc_status hc_batched_matmul_sharded(hc_group* g, hc_dtype dtype, int64_t matrix_count, const void* a_shard,
                                    int trans_a, const void* b_shard, int trans_b, int trans_out,
                                    int64_t rows, int64_t inner, int64_t cols, void* out, int gather);

/* One large Backend.matmul split over the columns of op(a)*op(b); every rank holds all of `a`
 * and `b` (it reads only its column block of `b`) and ends with the complete [rows, cols]
 * product in `out`.  Each block is computed with the tile plan of the whole product, so the
 * result equals hc_batched_matmul_ex(HC_KERNEL_TENSOR) bit for bit.  Collective.
 * fused == 0: blocks are computed into a packed buffer the group owns (it grows to rows*cols
 *   elements), exchanged with ncclAllGather, and one kernel moves them into `out`.
 * fused != 0: there is no collective and no staging: the product kernel's epilogue stores every
 *   finished tile into `out` on EVERY rank (peer stores over NVLink), so the exchange overlaps
 *   the remaining tiles.  `out` must come from hc_group_result_alloc.  The call enqueues a flag
 *   barrier before the product (no rank overwrites a peer's result while work enqueued earlier
 *   on that peer's context may still read it) and one after it (when it has passed on a rank's
 *   stream, every rank's tiles have landed there).  Work that reads the result on another
 *   stream must be ordered against the context's stream by the caller. */
hc_status hc_matmul_nsplit_allgather(hc_group* g, hc_dtype dtype, const void* a, int trans_a, const void* b,
                                     int trans_b, int64_t rows, int64_t inner, int64_t cols, void* out,
                                     int fused);
/* A result buffer of `bytes` on every rank that the other ranks can store into (mapped through
 * CUDA IPC between processes, through peer access inside one process).  Collective, as is the
 * matching free, which waits until no rank can still be storing into the buffer. */
hc_status hc_group_result_alloc(hc_group* g, size_t bytes, void** dptr);
hc_status hc_group_result_free(hc_group* g, void* dptr);
/* Enqueues a flag barrier on the context's stream: work enqueued after it starts when every rank
 * has completed the work it enqueued before its own call.  Returns without waiting.  Collective. */
hc_status hc_group_barrier(hc_group* g);
/* Failure-path self-test that harms nothing: a barrier in which this rank does not announce
 * itself, which is what a rank sees whose peer never arrives.  After `limit_ms` (1..1000) the
 * wait gives up; the next hc_check_device_status reports HC_ERR_TIMEOUT, and the group stays
 * usable.  In a group of more than one rank every rank must call it. */
hc_status hc_group_selftest_missing_peer(hc_group* g, int limit_ms);

/* float32 `transOut(op(a) * op(b))` on the tensor cores WITHOUT allocating: no counterpart in
 * the reference.  It exists for hosts that must not allocate device memory from inside a
 * library call - a framework whose caching allocator already owns the device, or a loop that
 * cannot afford the device-wide synchronisation cudaMalloc implies.  The work area of the
 * 3xTF32 split operands is a fixed array inside the library (hc_static_scratch_capacity()
 * bytes, held by every GPU that loads the library); a product needs about
 * 4 * (rows*inner + inner*cols) bytes of it (twice that for an operand whose address or row
 * pitch is not a multiple of 16 bytes), and a larger one is refused with
 * HC_ERR_INVALID_ARGUMENT (hc_last_error says how much was needed).  The result is, bit for
 * bit, that of hc_batched_matmul_ex(ctx, HC_KERNEL_TENSOR, HC_F32, 1, ...) whenever that call's
 * whole work area fits into the array - including the float32 partial sums of a long contraction
 * over few outputs, which it cuts into parts.  When the operands fit but those partial sums do
 * not, the contraction runs uncut: same tolerance (1e-5), different summation order.
 * The first call on each device looks up the array's device address; make that call outside
 * stream capture.  All calls in the process share the one array: calls that can overlap on
 * the GPU (other streams or contexts on the same device) must be ordered by the caller. */
hc_status hc_matmul_f32_static_scratch(hc_ctx* ctx, const void* a, int trans_a, const void* b,
                                       int trans_b, int trans_out, int64_t rows, int64_t inner,
                                       int64_t cols, void* out);
size_t hc_static_scratch_capacity(void);

/* ---- diagnostics ------------------------------------------------------------------------- */

const char* hc_status_string(hc_status s);
/* Text of the last failure on this context (thread-unsafe snapshot; empty if none). */
const char* hc_last_error(hc_ctx* ctx);
/* The same text copied into `buf` (NUL-terminated, at most `capacity` bytes) under the context's
 * lock, for hosts whose threads call into one context concurrently; returns the length copied. */
size_t hc_copy_last_error(hc_ctx* ctx, char* buf, size_t capacity);
/* Geometry of the most recent product launched on this context. */
hc_status hc_last_launch_info(hc_ctx* ctx, hc_launch_info* out);
/* How the tensor-core path would tile a product on a device with `sm_count` SMs: tile shape,
 * k slabs per pipeline slot, parts the contraction is cut into and the float32 work area those
 * parts need.  Pure host arithmetic (no device, no context): the launch code calls the same
 * routine, so tests can check the choice without a GPU.  No counterpart in the reference, which
 * leaves tiling to MPSGraph / vDSP. */
typedef struct hc_plan_info {
  int tile_m, tile_n;      /* output tile of one CTA or CTA pair */
  int ctas_per_tile;       /* 1, or 2 for a CTA pair (cta_group::2) */
  int slabs_per_slot;      /* 128-byte k slabs per pipeline slot */
  int parts;               /* 1, or the number of parts of a cut contraction */
  int slots_per_part;      /* pipeline slots each part walks */
  int64_t tiles;           /* tiles x parts over all matrices */
  size_t workspace_bytes;  /* float32 partial sums (0 when parts == 1) */
} hc_plan_info;
hc_status hc_plan_product(hc_dtype dtype, int64_t matrix_count, int trans_a, int trans_b,
                          int trans_out, int64_t rows, int64_t inner, int64_t cols, int sm_count,
                          hc_plan_info* out);
/* Kernels launched on this context since creation (each matrix product may launch several). */
int64_t hc_launch_count(hc_ctx* ctx);
/* Reads and clears the device-side status word; HC_ERR_TIMEOUT if a bounded wait expired in
 * a kernel that has completed.  Synchronises the stream. */
hc_status hc_check_device_status(hc_ctx* ctx);
/* Failure-path self-test that harms nothing: enqueues a one-thread kernel that waits, through
 * the same bounded-wait routine as the GEMM kernels, on a barrier nobody signals.  After
 * `limit_ms` (1..1000) the wait gives up, sets the status word and the kernel returns; the next
 * hc_check_device_status / hc_event_wait reports HC_ERR_TIMEOUT and the context stays usable. */
hc_status hc_selftest_bounded_wait(hc_ctx* ctx, int limit_ms);
/* Test hook for the allocation-failure paths: the next `count` device allocations this context
 * makes (results of hc_alloc, growth of a work area or staging buffer) fail as if the device were
 * out of memory.  Whatever the context held before such a failure stays valid. */
hc_status hc_inject_allocation_failures(hc_ctx* ctx, int count);
/* Tracing, off by default: while on, every product is wrapped in an NVTX range
 * ("hc_matmul f16 1x[8192x8192x8192]", visible to Nsight tools; the reference labels its command
 * buffers the same way, Sources/Honeycrisp/BackendMPS.swift:2698) and in a pair of events, from
 * which hc_last_elapsed_ms returns the device time of the most recent product (it waits for it). */
hc_status hc_set_tracing(hc_ctx* ctx, int on);
hc_status hc_last_elapsed_ms(hc_ctx* ctx, float* ms);
/* Library version, "major.minor". */
const char* hc_version(void);

#ifdef __cplusplus
}
#endif
#endif /* HC_CUDA_H_ */

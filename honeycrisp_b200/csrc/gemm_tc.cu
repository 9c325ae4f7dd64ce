// Tensor-core matrix product for sm_100a: tcgen05.mma with the accumulator in tensor memory,
// operands brought into shared memory by TMA through an mbarrier ring, results leaving through
// shared memory and TMA stores.
//
// One persistent CTA per SM walks a list of output tiles.  Inside a CTA:
//   warp 0, one lane : TMA producer of A.  Fills a ring of kStages shared-memory slots with one
//                      or two 128-byte-wide k-slabs of A per slot (128B-swizzled) and announces
//                      the slot's bytes to its barrier.
//   last warp, one lane : TMA producer of B, into the same slots.
//   warp 1, one lane : MMA issuer.  For every filled slot issues the tcgen05.mma instructions
//                      of its slabs into an accumulator buffer in tensor memory, then commits
//                      the slot back to the producers.
//   warps 2..        : epilogue.  Drain a finished accumulator (tcgen05.ld), round, stage the
//                      rows in swizzled shared memory and send them with TMA stores, then hand
//                      the accumulator back, while the issuer already works on the other one.
// Each of these single-thread loops has to stay shorter than the MMAs of one slot execute
// (512 clocks for a 256x256 pair tile and one slab): no division, non-blocking barrier probes
// first, and the copies split over two threads (one tensor copy costs its thread ~115 clocks).
// The issuing lanes are chosen with elect.sync, never by comparing the lane index: only then
// does the compiler keep descriptors in uniform registers, and a tcgen05.mma issues in a few
// cycles instead of ~220.
//
// Tile shapes:
//   128 x 128 / 128 x 256 on one CTA     products of at most 128 rows;
//   256 x 128 / 256 x 64 on a CTA pair   products too small to fill the SMs with larger tiles;
//   256 x 256 on a CTA pair              cta_group::2: the two CTAs of a cluster own the upper and
//                                        lower 128 rows, each loads its own rows of A and its own
//                                        half of the B columns, the leader issues one MMA that
//                                        spans both SMs; two accumulator buffers alternate;
//   256 x 512 on a CTA pair              long float16 contractions: two MMAs per k-step share the
//                                        A slab and fill both accumulator buffers - least operand
//                                        traffic per flop; the drain overlaps only half by half
//                                        (the left half under the last k-steps' right-half MMAs,
//                                        the right half under the next tile's first left-half ones).
// Every copy is an ordinary per-CTA TMA load into the CTA's own shared memory.
// The shape is chosen per launch by a cost model (plan_tc: waves of tiles x clocks per tile).
// When even the smallest shape fills less than one wave and the contraction is long, the
// contraction is cut into parts that run as separate tiles into float32 partial matrices, which
// splitk_reduce_kernel sums in ascending order.
//
// Transposed operands are never moved: a "K-major" operand (contracted index contiguous) and
// an "MN-major" one (row/column index contiguous) differ only in the TMA box shape and in one
// bit of the instruction descriptor.
//
// float32 runs as 3xTF32: x = hi + lo with hi, lo representable in TF32, and
// A*B ~= A_lo*B_hi + A_hi*B_lo + A_hi*B_hi.  hi is the operand itself (the tensor core reads a
// float32 operand truncated to TF32), lo is written to a scratch area by a pre-pass; every
// pipeline slot holds the hi and lo slabs of both operands, loaded once, and the issuer runs
// the three products of the slab from them into the same accumulator.  Tensor-core accumulation
// truncates instead of rounding, so a long contraction is cut into windows: every window
// accumulates in tensor memory, and the epilogue warps add the windows together in registers
// with ordinary float32 adds.
//
// Optional extras of the epilogue: a bias row added to the rounded product (Linear), and up
// to seven more destinations for every result block (other devices' copies of the result,
// written with peer TMA stores).
//
// Every wait in this file is bounded: after a time limit the waiting thread records a bit in
// the context's status word, raises a CTA-wide abort flag and the CTA leaves through the
// normal teardown (tensor memory is freed).  The host reports HC_ERR_TIMEOUT.
#include <cuda.h>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"

extern "C" char** environ;

// The 512-wide tile's MMA issuer leaves its tile loop body early (`continue`), which makes the
// generic k loop behind it unreachable in that one instantiation.
#pragma nv_diag_suppress 128

namespace hc {
namespace {

constexpr int BM = 128;
constexpr unsigned long long kWaitLimitNs = 4000000000ull;  // 4 s

struct TcParams {
  int64_t M, N;
  int num_k_blocks;   // pipeline slots (of one or two k slabs) along the whole contraction
  int splits;         // parts the contraction is cut into (1: none); part z of matrix m is "matrix" m*splits+z
  int kb_per_split;   // slots per part (the last part may be shorter)
  int chunk_kb;       // slabs per accumulation window (== num_k_blocks when not windowed)
  int tiles_m, tiles_n;
  int64_t total_tiles;
  int group_m;
  int a_mn_major, b_mn_major;
  void* C;
  int64_t ldc, strideC;
  unsigned int* status;
  int vec_ok;         // C base and ldc allow 16-byte stores
  int tile_rows;      // 128 per CTA of the group
  int tma_store;      // results leave through shared memory and TMA stores (else direct stores)
  const void* bias;   // optional row vector added to the rounded product (Linear), or null
  int n_out;          // destinations of every result tile: this device's result, then peers' copies
  int skip_input_wait;  // the operands are known not to be written by the kernel launched just before
};

// ---- PTX wrappers ---------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// True in exactly one lane of a fully active warp.  Choosing the issuing lane with elect.sync
// (rather than comparing the lane index) tells the compiler that a single thread runs the
// guarded code, so descriptors and barrier addresses can live in uniform registers.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n"
      ".reg .pred P;\n"
      "elect.sync _|P, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, P;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}
// Address of the same shared-memory location in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
// Programmatic dependent launch: a kernel launched with the stream-serialization attribute may
// start while its predecessor in the stream is still draining.  `pdl_release` lets the successor
// be scheduled as soon as every CTA of this grid has issued it (or exited); `pdl_wait` blocks
// until the predecessor has completed and its memory is visible.  Both are no-ops for an
// ordinary launch.  Everything before pdl_wait must touch no global memory - with one exception
// the host decides: operand loads may run ahead of it when the operands cannot have been written
// by the predecessor (TcParams::skip_input_wait).
// The product kernel releases its successor only AFTER its own wait has returned.  Its successor
// therefore never starts before the product kernel's predecessor has completed, and the only
// kernel a product can race with when it skips its operand wait is the one enqueued immediately
// before it.  The small elementwise kernels around it (operand split, repack, sum of a cut
// contraction's parts) release at entry, so that the kernel behind them is already launched and
// parked at its wait when they finish; a product that follows one of them never skips its wait.
__device__ __forceinline__ void pdl_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Rendezvous without memory ordering: for the teardown, where the CTAs of a pair only have to
// know that the other has stopped signalling (a releasing arrive first waits for the thread's
// outstanding writes to be visible cluster-wide, about 0.5 us at the end of every launch).
// Setup rendezvous of a CTA pair: the thread that initialised the barriers has published them
// with fence.mbarrier_init.release.cluster, so the arrive itself needs no release (which would
// wait for every thread's earlier writes); the wait acquires.
__device__ __forceinline__ void cluster_sync_after_barrier_init() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_rendezvous() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;\nbarrier.cluster.wait.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
// Arrive, without memory ordering, on a barrier given by its cluster-wide address (this CTA's or
// the partner's).  Handing an accumulator buffer back to the MMA issuer orders
// tensor-memory accesses only, which tcgen05.fence does on both sides of the barrier; a releasing
// arrive here waited about 1400 clocks for the epilogue's own stores on every tile.
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t bar) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  False means: gave up (time limit, or another role of this CTA already did).
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                            unsigned long long limit_ns = kWaitLimitNs) {
  const unsigned long long t0 = globaltimer_ns();
#pragma unroll 1
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; i++)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (globaltimer_ns() - t0 > limit_ns) return false;
  }
}
// The non-blocking probe: it answers in about half the time of try_wait (which may suspend
// the thread), so every wait starts with it - in a full pipeline the phase is usually complete.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_test_wait(bar, parity)) return true;
#pragma unroll 1
  for (int i = 0; i < 16; i++)
    if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_flag);
}

// Long waits of a whole warp (the epilogue waits a full main loop for its accumulator): one
// lane polls, sleeping between polls so the spinning does not compete with the issuing warps
// for issue slots and power; when it has seen the phase complete, every lane observes the
// barrier once itself (that returns at once and gives each lane its own acquire).
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag, int lane) {
  bool ok = true;
  if (lane == 0) {
    ok = false;
#pragma unroll 1
    for (int i = 0; i < 32 && !ok; i++) ok = mbar_try_wait(bar, parity);
    if (!ok) {
      const unsigned long long t0 = globaltimer_ns();
#pragma unroll 1
      for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32 && !ok; i++) {
          __nanosleep(100);
          ok = mbar_try_wait(bar, parity);
        }
        if (ok || *abort_flag || globaltimer_ns() - t0 > kWaitLimitNs) break;
      }
    }
  }
  ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
  if (ok) {
    bool mine = false;
#pragma unroll 1
    for (int i = 0; i < 4096 && !mine; i++) mine = mbar_try_wait(bar, parity);
    ok = __all_sync(0xffffffffu, mine);
  }
  return ok;
}

// Tiled TMA load of one box into this CTA's shared memory.  With kCta == 2 the completion
// bytes are counted on a barrier that may live in the partner CTA (the leader's).
template <int kCta>
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2) {
  if (kCta == 2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"((unsigned long long)map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
  } else {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"((unsigned long long)map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
  }
}

// Tiled TMA store of one box from this CTA's shared memory; out-of-range parts are clipped.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
      ::"l"((unsigned long long)map), "r"(src), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Wait until at most kPending of this thread's bulk groups have not finished reading shared memory.
template <int kPending>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrive on `bar` (cluster-wide address) once every MMA issued so far by this thread is done.
template <int kCta>
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  if (kCta == 2) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
  } else {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
  }
}
template <bool kTf32, int kCta>
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                       uint32_t idesc, uint32_t accumulate) {
  if (kTf32 && kCta == 1) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else if (kTf32 && kCta == 2) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else if (kCta == 1) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp gets lane (base+i).
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of tcgen05.mma.
//   bits  0-13 start address >> 4      bits 16-29 leading-dimension byte offset >> 4
//   bits 32-45 stride byte offset >> 4 bits 46-47 descriptor version (1 on sm_100)
//   bits 61-63 swizzle mode: 2 = 128-byte rows permuted in 16-byte units,
//                            1 = 128-byte rows permuted in 32-byte units
// K-major operand : rows are 128-byte k-slabs; 8-row groups are 1024 bytes apart (stride offset).
// MN-major operand: each 128-byte row holds consecutive M (or N) indices for one k; a group of
//                   k-rows (8 rows for 16-bit data; 4 rows for 32-bit data, which only supports
//                   the 32-byte-unit swizzle in this orientation) is one stride offset; the
//                   next run of M/N indices starts one whole box later (leading offset).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint32_t swizzle_mode) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)swizzle_mode << 61;
  return d;
}

// Instruction descriptor of tcgen05.mma kind::f16 / kind::tf32 (dense, fp32 accumulate).
//   bits 4-5 D format (1 = f32)   bits 7-9 A format   bits 10-12 B format (0 = f16, 2 = tf32)
//   bit 15 A is MN-major          bit 16 B is MN-major
//   bits 17-22 N >> 3             bits 24-28 M >> 4
__host__ __device__ constexpr uint32_t make_idesc(bool tf32, int a_mn, int b_mn, int m, int n) {
  return (1u << 4) | ((tf32 ? 2u : 0u) << 7) | ((tf32 ? 2u : 0u) << 10) | ((uint32_t)(a_mn & 1) << 15) |
         ((uint32_t)(b_mn & 1) << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// Linear's `h + bias` on W consecutive columns starting at `col`, as the reference computes it:
// the product is first rounded to the output dtype, then widened, added, and narrowed again by
// the caller (BackendCPU.swift:295-303 after the matmul's own writeBuffer).
template <bool kHalf, int W>
__device__ __forceinline__ void add_bias(const void* bias, int64_t col, int64_t N, float (&x)[W]) {
  if (kHalf) {
    const __half* b = (const __half*)bias + col;
    if (W == 8 && col + 8 <= N && (((uintptr_t)b) & 15) == 0) {
      const uint4 u = __ldg((const uint4*)b);
      const __half2* h2 = (const __half2*)&u;
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const float2 f = __half22float2(h2[i]);
        x[2 * i] = __fadd_rn(__half2float(__float2half_rn(x[2 * i])), f.x);
        x[2 * i + 1] = __fadd_rn(__half2float(__float2half_rn(x[2 * i + 1])), f.y);
      }
    } else {
#pragma unroll
      for (int i = 0; i < W; i++)
        if (col + i < N) x[i] = __fadd_rn(__half2float(__float2half_rn(x[i])), __half2float(__ldg(b + i)));
    }
  } else {
    const float* b = (const float*)bias + col;
    if (W == 4 && col + 4 <= N && (((uintptr_t)b) & 15) == 0) {
      const float4 f = __ldg((const float4*)b);
      x[0] = __fadd_rn(x[0], f.x); x[1] = __fadd_rn(x[1], f.y); x[2] = __fadd_rn(x[2], f.z); x[3] = __fadd_rn(x[3], f.w);
    } else {
#pragma unroll
      for (int i = 0; i < W; i++)
        if (col + i < N) x[i] = __fadd_rn(x[i], __ldg(b + i));
    }
  }
}

template <bool kHalf>
__device__ __forceinline__ void store_row32(void* cbase, int64_t row_off, int64_t gn, int64_t N,
                                            const float (&v)[32], bool vec_ok) {
  if (kHalf) {
    __half* dst = (__half*)cbase + row_off + gn;
    if (vec_ok && gn + 32 <= N) {
#pragma unroll
      for (int q = 0; q < 4; q++) {
        uint4 u;
        __half2 h0 = __floats2half2_rn(v[q * 8 + 0], v[q * 8 + 1]);
        __half2 h1 = __floats2half2_rn(v[q * 8 + 2], v[q * 8 + 3]);
        __half2 h2 = __floats2half2_rn(v[q * 8 + 4], v[q * 8 + 5]);
        __half2 h3 = __floats2half2_rn(v[q * 8 + 6], v[q * 8 + 7]);
        u.x = *(uint32_t*)&h0; u.y = *(uint32_t*)&h1; u.z = *(uint32_t*)&h2; u.w = *(uint32_t*)&h3;
        *(uint4*)(dst + q * 8) = u;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; j++)
        if (gn + j < N) dst[j] = __float2half_rn(v[j]);
    }
  } else {
    float* dst = (float*)cbase + row_off + gn;
    if (vec_ok && gn + 32 <= N) {
#pragma unroll
      for (int q = 0; q < 8; q++)
        *(float4*)(dst + q * 4) = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; j++)
        if (gn + j < N) dst[j] = v[j];
    }
  }
}

// One tensor map per destination of the result: [0] is this device's buffer, the rest are the
// same-shaped buffers of other devices of the box, mapped into this process (plain peer
// stores over NVLink; never a load).
constexpr int kMaxOut = 8;
struct OutMaps { CUtensorMap m[kMaxOut]; };

struct TileCoord { int64_t mat; int tm, tn; };
__device__ __forceinline__ TileCoord decode_tile(int64_t tile, const TcParams& p) {
  const int64_t per_mat = (int64_t)p.tiles_m * p.tiles_n;
  TileCoord t;
  int r;
  if (p.total_tiles <= 0x7fffffffll) {   // the usual case: 32-bit division, a fraction of the 64-bit one's latency
    const uint32_t tl = (uint32_t)tile, pm = (uint32_t)per_mat;
    const uint32_t m = tl / pm;
    t.mat = m;
    r = (int)(tl - m * pm);
  } else {
    t.mat = tile / per_mat;
    r = (int)(tile % per_mat);
  }
  const int per_group = p.group_m * p.tiles_n;
  const int g = r / per_group;
  const int first_m = g * p.group_m;
  const int gsize = min(p.group_m, p.tiles_m - first_m);
  const int rr = r % per_group;
  t.tm = first_m + rr % gsize;
  t.tn = rr / gsize;
  return t;
}

// Store staging buffers (4 KB each) per epilogue warp: two that alternate, or one where shared
// memory is short (the windowed epilogue, and eight epilogue warps next to the 48 KB slots of the
// 512-wide tiles) or where a warp's share of the tile is a single buffer wide.
__host__ __device__ constexpr int staging_bufs(int out_bytes, int bn, int epi_warps, bool windowed, int nsplit) {
  return (windowed || (epi_warps == 8 && nsplit == 2) || (bn * nsplit / (epi_warps / 4)) < 2 * (128 / out_bytes)) ? 1 : 2;
}

// With the contraction cut into parts, tiles are numbered over batch x parts "matrices": the
// operands of matrix v / parts, k slots [kb0, kb0 + count), the result into partial matrix v.
struct KRange { int mat, kb0, count; };
__device__ __forceinline__ KRange k_range(int64_t vmat, const TcParams& p) {
  KRange r;
  if (p.splits <= 1) {
    r.mat = (int)vmat; r.kb0 = 0; r.count = p.num_k_blocks;
  } else {
    r.mat = (int)((uint32_t)vmat / (uint32_t)p.splits);   // batch x parts fits 32 bits (host checks)
    r.kb0 = (int)((uint32_t)vmat - (uint32_t)r.mat * (uint32_t)p.splits) * p.kb_per_split;
    r.count = min(p.kb_per_split, p.num_k_blocks - r.kb0);
  }
  return r;
}

// kElemBytes: 2 (float16 operands) or 4 (float32 operands consumed as TF32).
// kBN       : columns of one tcgen05.mma (and of one accumulator buffer).
// kNSplit   : 1, or 2 for tiles two MMAs wide (512 columns) whose halves take the two accumulator
//             buffers: less operand traffic per flop, but the epilogue no longer overlaps the
//             next tile (used for long contractions only).
// kWindowed : epilogue sums accumulation windows in registers (float32 output only).
// kCta      : 1, or 2 for CTA pairs (cluster of two, 256-row tiles, one MMA over both SMs).
// kSlabs    : 128-byte k slabs per pipeline slot.  Two halve the barrier round trips per k, which
//             is what bounds the small tile shapes (their MMAs are shorter than the issue loop).
// kPartial  : float16 operands, float32 results: the partial sums of a contraction cut into parts.
// One CTA per SM: a kernel that allocates tensor memory (tcgen05.alloc) is never given a second
// resident CTA on an SM, however little shared memory and however few registers it uses (the
// occupancy query answers 1 for any such kernel; measured).  Overlap across the end of one launch
// and the start of the next therefore has to come from programmatic dependent launch alone.
template <int kElemBytes, int kBN, int kStages, int kEpiWarps, bool kWindowed, int kCta, int kNSplit, int kSlabs,
          bool kPartial>
__global__ void __launch_bounds__(96 + 32 * kEpiWarps, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap mapA_hi, const __grid_constant__ CUtensorMap mapA_lo,
               const __grid_constant__ CUtensorMap mapB_hi, const __grid_constant__ CUtensorMap mapB_lo,
               const __grid_constant__ OutMaps mapC, const TcParams p) {
  constexpr bool kTf32 = (kElemBytes == 4);
  constexpr bool kOutHalf = (kElemBytes == 2) && !kPartial;
  constexpr int BK = 128 / kElemBytes;       // elements in one 128-byte slab row
  constexpr int UMMA_K = 32 / kElemBytes;    // k per tcgen05.mma
  constexpr int CH = 128 / kElemBytes;       // M/N indices in one 128-byte row of an MN-major box
  constexpr int BN_LOCAL = kBN / kCta;       // B columns this CTA loads per MMA-wide part of the tile
  constexpr int TILE_N = kBN * kNSplit;
  constexpr int ACC_SLOTS = 2 / kNSplit;     // accumulator buffers that alternate between windows
  // MN-major geometry: 16-bit data uses the 16-byte-unit swizzle with 8-row k groups, 32-bit
  // data the 32-byte-unit swizzle with 4-row k groups.  One MMA consumes UMMA_K 128-byte k-rows.
  constexpr uint32_t MN_SBO = kTf32 ? 512u : 1024u;
  constexpr uint32_t MN_MODE = kTf32 ? 1u : 2u;
  // A pipeline slot: [A (hi) | A lo] [B (hi) | B lo]; the lo slabs exist for float32 only.
  constexpr int PARTS = kTf32 ? 2 : 1;
  constexpr uint32_t A_BYTES = BM * 128, B_PART_BYTES = BN_LOCAL * 128, B_BYTES = kNSplit * B_PART_BYTES,
                     SLAB_BYTES = PARTS * (A_BYTES + B_BYTES), STAGE_BYTES = kSlabs * SLAB_BYTES;
  static_assert(kSlabs == 1 || !kWindowed, "accumulation windows count single slabs");
  constexpr int STG_BUFS = staging_bufs(kOutHalf ? 2 : 4, kBN, kEpiWarps, kWindowed, kNSplit);
  constexpr uint32_t STG_BYTES_PER_WARP = STG_BUFS * 4096u;
  constexpr int TMEM_COLS = (2 * kBN <= 32) ? 32 : 2 * kBN;
  constexpr int COL_SPLIT = kEpiWarps / 4;   // epilogue warps sharing one lane quarter
  constexpr int COLS_PER_THREAD = TILE_N / COL_SPLIT;
  static_assert(kNSplit == 1 || (kNSplit == 2 && !kWindowed && kBN == 256), "wide tiles: plain epilogue only");
  static_assert(kEpiWarps == 4 || kEpiWarps == 8 || kEpiWarps == 16, "epilogue warps come in groups of four");
  static_assert(TMEM_COLS == 64 || TMEM_COLS == 128 || TMEM_COLS == 256 || TMEM_COLS == 512, "power of two");
  static_assert(kCta == 1 || kCta == 2, "one CTA or a pair");

  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * kStages + 4];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = (kCta == 2) ? cluster_ctarank() : 0u;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_full = smem_u32(&bars[0]);
  const uint32_t bar_empty = smem_u32(&bars[kStages]);
  const uint32_t bar_tfull = smem_u32(&bars[2 * kStages]);
  const uint32_t bar_tempty = smem_u32(&bars[2 * kStages + 2]);

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStages; s++) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int s = 0; s < 2; s++) {
      mbar_init(bar_tfull + 8 * s, 1);
      mbar_init(bar_tempty + 8 * s, 32 * kEpiWarps * kCta);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    if (kCta == 2) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                   "r"((uint32_t)TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                   "r"((uint32_t)TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (kCta == 2) cluster_sync_after_barrier_init();   // the partner's barriers are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int* abortp = &abort_flag;
  // Barriers and tensor memory are set up.  Each role that touches global memory (the producer
  // reads operands an earlier kernel in the stream may have produced, the epilogue overwrites
  // results it may have read) waits for that kernel below, after the part of its own setup that
  // only needs the launch parameters: tensor-map prefetch and the first tile's coordinates.

  const int nkb = p.num_k_blocks;
  const int chunk_kb = p.chunk_kb;
  const int64_t tile_first = blockIdx.x / kCta, tile_step = gridDim.x / kCta;

  constexpr int kWarpProducerB = 2 + kEpiWarps;
  if (warp == 0 || warp == kWarpProducerB) {
    // ---------------------------------------------------------------- TMA producers
    // Issuing one tensor copy costs its thread about 115 clocks, and a slot takes two to eight of
    // them (two slabs; two boxes per slab for an MN-major operand): one thread doing all of it
    // is slower than the MMAs of the small tile shapes and of transposed operands.  Warp 0 copies
    // A and announces the slot's bytes, the last warp copies B; both watch the same barriers.
    const bool do_a = (warp == 0), do_b = !do_a;
    if (elect_one()) {
      if (do_a) asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&mapA_hi) : "memory");
      if (do_b) asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&mapB_hi) : "memory");
      if (kTf32) {
        if (do_a) asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&mapA_lo) : "memory");
        if (do_b) asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&mapB_lo) : "memory");
      }
      // Completion bytes of both CTAs of a pair are counted on the leader's barrier.
      const uint32_t full_leader = (kCta == 2) ? map_to_cta(bar_full, 0) : bar_full;
      // (L2 eviction priorities on these loads - the band of A a wave shares with the next one
      // asked to stay, the panels of B to go first - were measured at 8192^3: evict_last changes
      // nothing (897-913 MB read from DRAM either way), evict_first on B doubles the reads.)
      auto load = [&](uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
        tma_load_3d<kCta>(dst, map, bar, c0, c1, c2);
      };
      uint32_t s = 0, ph = 0;
      bool ok = true;
      TileCoord t = decode_tile(tile_first < p.total_tiles ? tile_first : 0, p);
      KRange kr = k_range(t.mat, p);
      // The ring starts empty: the first kStages slots of the first tile need no wait, and their
      // byte counts can be announced before the previous kernel is waited for.
      const int free_slots = (tile_first < p.total_tiles) ? min(kStages, kr.count) : 0;
      if (do_a && rank == 0)
        for (int i = 0; i < free_slots; i++) mbar_expect_tx(bar_full + 8 * i, STAGE_BYTES * kCta);
      if (!p.skip_input_wait) pdl_wait();
      for (int64_t tile = tile_first; ok && tile < p.total_tiles; tile += tile_step) {
        if (tile != tile_first) { t = decode_tile(tile, p); kr = k_range(t.mat, p); }
        const int prearmed = (tile == tile_first) ? free_slots : 0;
        const int m0 = t.tm * (BM * kCta) + (int)rank * BM;
        const int n0 = t.tn * TILE_N + (int)rank * BN_LOCAL;
        const int mat = kr.mat;
        for (int kb = 0; kb < kr.count; kb++) {
          if (kb >= prearmed && !mbar_wait(bar_empty + 8 * s, ph ^ 1, abortp)) {
            atomicOr(p.status, kDevTimeoutProducer);
            abort_flag = 1;
            ok = false;
            break;
          }
          const uint32_t full = full_leader + 8 * s;
          // (copies of B may complete before the bytes are announced: the count goes negative
          // for a moment, and the phase cannot complete before this arrive)
          if (rank == 0 && do_a && kb >= prearmed) mbar_expect_tx(bar_full + 8 * s, STAGE_BYTES * kCta);
          // A slab past the end of K lies outside the tensor and arrives as zeros.
#pragma unroll
          for (int j = 0; j < kSlabs; j++) {
          const int kc = ((kr.kb0 + kb) * kSlabs + j) * BK;
          const uint32_t stage = smem_base + s * STAGE_BYTES + j * SLAB_BYTES;
#pragma unroll
          for (int part = 0; part < PARTS; part++) {   // 0: the operand itself (hi), 1: its lo half
            const CUtensorMap* ma = part ? &mapA_lo : &mapA_hi;
            const CUtensorMap* mb = part ? &mapB_lo : &mapB_hi;
            const uint32_t sa = stage + part * A_BYTES, sb = stage + PARTS * A_BYTES + part * B_BYTES;
            if (do_a) {
              if (!p.a_mn_major) {
                load(sa, ma, full, kc, m0, mat);
              } else {
#pragma unroll
                for (int c = 0; c < BM / CH; c++) load(sa + c * (BK * 128), ma, full, m0 + c * CH, kc, mat);
              }
            }
#pragma unroll
            for (int h = 0; do_b && h < kNSplit; h++) {
              const uint32_t sbh = sb + h * B_PART_BYTES;
              const int n0h = n0 + h * kBN;
              if (!p.b_mn_major) {
                load(sbh, mb, full, kc, n0h, mat);
              } else {
#pragma unroll
                for (int c = 0; c < BN_LOCAL / CH; c++)
                  load(sbh + c * (BK * 128), mb, full, n0h + c * CH, kc, mat);
              }
            }
          }
          }
          if (++s == kStages) { s = 0; ph ^= 1; }
        }
      }
      if (kCta == 2 && ok && do_a) {
        // Drain: every slot's release (an asynchronous arrive from the leader's MMA commits)
        // must have landed in this CTA's barriers before the CTA may exit.
        for (int i = 0; i < kStages; i++) {
          if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abortp)) {
            atomicOr(p.status, kDevTimeoutProducer);
            abort_flag = 1;
            break;
          }
          if (++s == kStages) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (leader CTA)
    if (elect_one() && rank == 0) {
      const uint32_t idesc = make_idesc(kTf32, p.a_mn_major, p.b_mn_major, BM * kCta, kBN);
      // K-major: leading offset unused (1 unit), stride offset = 8 rows * 128 B.
      // MN-major: leading offset = one box (BK rows * 128 B), stride offset = one k-row group.
      const uint32_t a_lbo = p.a_mn_major ? (uint32_t)(BK * 128) : 16u, a_sbo = p.a_mn_major ? MN_SBO : 1024u;
      const uint32_t b_lbo = p.b_mn_major ? (uint32_t)(BK * 128) : 16u, b_sbo = p.b_mn_major ? MN_SBO : 1024u;
      const uint32_t a_mode = p.a_mn_major ? MN_MODE : 2u, b_mode = p.b_mn_major ? MN_MODE : 2u;
      const uint32_t a_kstep = p.a_mn_major ? (uint32_t)(UMMA_K * 128) : 32u;
      const uint32_t b_kstep = p.b_mn_major ? (uint32_t)(UMMA_K * 128) : 32u;
      const uint32_t empty_peer = (kCta == 2) ? map_to_cta(bar_empty, 1) : 0u;
      const uint32_t tfull_peer = (kCta == 2) ? map_to_cta(bar_tfull, 1) : 0u;
      uint32_t s = 0, ph = 0, win = 0, slot = 0;
      bool ok = true;
      for (int64_t tile = tile_first; ok && tile < p.total_tiles; tile += tile_step) {
        // This loop is one thread's serial instruction stream and has to stay shorter than the
        // MMAs of one k block take to execute (512 clocks for a 256x256 pair tile), or the tensor
        // pipe waits for the issuer: no division, no blocking probe on the usual path.
        int in_win = -1;   // position of this k block in its accumulation window
        const int nkb_t = (p.splits > 1) ? k_range(decode_tile(tile, p).mat, p).count : nkb;
        if (kNSplit == 2) {
          // 512-wide tile: both accumulator buffers belong to this tile, half h in buffer h, so
          // the drain cannot hide behind the next tile as a whole - but it can half by half.  The
          // last kHead k blocks first run their left-half MMAs, the left half is published, and
          // its drain overlaps their right-half MMAs; the next tile starts with the left-half MMAs
          // of its first kHead k blocks, which overlap the drain of the previous right half.
          // In between, every k block issues both halves.  `win` counts tiles here.
          constexpr int kHead = 2;
          static_assert(kNSplit == 1 || kStages >= 2 * kHead, "head and tail each hold kHead slots");
          const uint32_t tpar = win & 1;
          const bool staged = nkb_t >= 2 * kHead;
          auto mma_half = [&](uint32_t slot_s, int h, bool fresh) {
#pragma unroll
            for (int j = 0; j < kSlabs; j++) {
              const uint32_t stage = smem_base + slot_s * STAGE_BYTES + j * SLAB_BYTES;
              const uint64_t adesc = make_smem_desc(stage, a_lbo, a_sbo, a_mode);
              const uint64_t bdesc = make_smem_desc(stage + PARTS * A_BYTES + h * B_PART_BYTES, b_lbo, b_sbo, b_mode);
#pragma unroll
              for (int k = 0; k < BK / UMMA_K; k++)
                tc_mma<kTf32, kCta>(tmem_base + h * kBN, adesc + (uint64_t)((k * a_kstep) >> 4),
                                    bdesc + (uint64_t)((k * b_kstep) >> 4), idesc, (fresh && j == 0 && k == 0) ? 0u : 1u);
            }
          };
          auto release = [&](uint32_t slot_s) {
            tc_commit<kCta>(bar_empty + 8 * slot_s);
            if (kCta == 2) tc_commit<kCta>(empty_peer + 8 * slot_s);
          };
          auto fail = [&]() {
            atomicOr(p.status, kDevTimeoutMma);
            abort_flag = 1;
            ok = false;
          };
          int kb = 0;
          if (!mbar_wait(bar_tempty, tpar ^ 1, abortp)) { fail(); break; }
          tc_fence_after();
          if (staged) {
            uint32_t hs[kHead];
#pragma unroll
            for (int i = 0; i < kHead && ok; i++) {
              hs[i] = s;
              if (!mbar_wait(bar_full + 8 * s, ph, abortp)) { fail(); break; }
              tc_fence_after();
              mma_half(s, 0, i == 0);
              if (++s == kStages) { s = 0; ph ^= 1; }
            }
            if (!ok) break;
            if (!mbar_wait(bar_tempty + 8, tpar ^ 1, abortp)) { fail(); break; }
            tc_fence_after();
#pragma unroll
            for (int i = 0; i < kHead; i++) {
              mma_half(hs[i], 1, i == 0);
              release(hs[i]);
            }
            kb = kHead;
          } else {
            if (!mbar_wait(bar_tempty + 8, tpar ^ 1, abortp)) { fail(); break; }
            tc_fence_after();
          }
          const int body_end = staged ? nkb_t - kHead : nkb_t;
          for (; kb < body_end; kb++) {
            if (!mbar_wait(bar_full + 8 * s, ph, abortp)) { fail(); break; }
            tc_fence_after();
            mma_half(s, 0, kb == 0);
            mma_half(s, 1, kb == 0);
            release(s);
            if (++s == kStages) { s = 0; ph ^= 1; }
          }
          if (!ok) break;
          if (staged) {
            uint32_t ts[kHead];
#pragma unroll
            for (int i = 0; i < kHead && ok; i++) {
              ts[i] = s;
              if (!mbar_wait(bar_full + 8 * s, ph, abortp)) { fail(); break; }
              tc_fence_after();
              mma_half(s, 0, false);
              if (++s == kStages) { s = 0; ph ^= 1; }
            }
            if (!ok) break;
            tc_commit<kCta>(bar_tfull);
            if (kCta == 2) tc_commit<kCta>(tfull_peer);
#pragma unroll
            for (int i = 0; i < kHead; i++) {
              mma_half(ts[i], 1, false);
              release(ts[i]);
            }
            tc_commit<kCta>(bar_tfull + 8);
            if (kCta == 2) tc_commit<kCta>(tfull_peer + 8);
          } else {
            tc_commit<kCta>(bar_tfull);
            if (kCta == 2) tc_commit<kCta>(tfull_peer);
            tc_commit<kCta>(bar_tfull + 8);
            if (kCta == 2) tc_commit<kCta>(tfull_peer + 8);
          }
          win++;
          continue;
        }
        for (int kb = 0; kb < nkb_t; kb++) {
          if (++in_win == chunk_kb) in_win = 0;
          if (in_win == 0) {
            slot = win % ACC_SLOTS;
            if (!mbar_wait(bar_tempty + 8 * slot, ((win / ACC_SLOTS) & 1) ^ 1, abortp)) {
              atomicOr(p.status, kDevTimeoutMma);
              abort_flag = 1;
              ok = false;
              break;
            }
            tc_fence_after();
          }
          if (!mbar_wait(bar_full + 8 * s, ph, abortp)) {
            atomicOr(p.status, kDevTimeoutMma);
            abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          // float16: one product per slab.  float32: A_lo*B_hi, A_hi*B_lo, A_hi*B_hi - the two
          // small products first, all into the same accumulator.
          constexpr int PRODUCTS = kTf32 ? 3 : 1;
#pragma unroll
          for (int j = 0; j < kSlabs; j++) {
          const uint32_t stage = smem_base + s * STAGE_BYTES + j * SLAB_BYTES;
#pragma unroll
          for (int pr = 0; pr < PRODUCTS; pr++) {
            const int a_part = (kTf32 && pr == 0) ? 1 : 0, b_part = (kTf32 && pr == 1) ? 1 : 0;
            const uint32_t sa = stage + a_part * A_BYTES, sb = stage + PARTS * A_BYTES + b_part * B_BYTES;
            const uint64_t adesc = make_smem_desc(sa, a_lbo, a_sbo, a_mode);
#pragma unroll
            for (int h = 0; h < kNSplit; h++) {
              const uint64_t bdesc = make_smem_desc(sb + h * B_PART_BYTES, b_lbo, b_sbo, b_mode);
              const uint32_t d = tmem_base + (kNSplit == 2 ? h : slot) * kBN;
#pragma unroll
              for (int k = 0; k < BK / UMMA_K; k++) {
                tc_mma<kTf32, kCta>(d, adesc + (uint64_t)((k * a_kstep) >> 4), bdesc + (uint64_t)((k * b_kstep) >> 4),
                                    idesc, (in_win | j | pr | k) ? 1u : 0u);
              }
            }
          }
          }
          tc_commit<kCta>(bar_empty + 8 * s);
          if (kCta == 2) tc_commit<kCta>(empty_peer + 8 * s);
          if (in_win == chunk_kb - 1 || kb == nkb_t - 1) {
            tc_commit<kCta>(bar_tfull + 8 * slot);
            if (kCta == 2) tc_commit<kCta>(tfull_peer + 8 * slot);
            win++;
          }
          if (++s == kStages) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp < kWarpProducerB) {
    // ---------------------------------------------------------------- epilogue
    const int ew = warp - 2;
    const int quarter = warp & 3;            // tensor-memory lanes this warp may read
    const int col_part = ew / 4;             // which share of the columns
    const int col0 = col_part * COLS_PER_THREAD;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    // Buffers are handed back to the leader's MMA issuer.
    const uint32_t tempty_leader = (kCta == 2) ? map_to_cta(bar_tempty, 0) : bar_tempty;
    // Staging for TMA stores behind the operand ring: per epilogue warp two 4 KB buffers, or one
    // for the windowed epilogue (which stores once per tile).
    const uint32_t stg_base = smem_base + kStages * STAGE_BYTES + (uint32_t)ew * STG_BYTES_PER_WARP;
    const bool store_leader = elect_one();
    uint32_t win = 0;
    bool ok = true;
    if (store_leader && p.tma_store) asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&mapC.m[0]) : "memory");
    TileCoord t = decode_tile(tile_first < p.total_tiles ? tile_first : 0, p);
    pdl_wait();
    if (warp == 2 && store_leader) pdl_release();   // one thread per CTA is enough
    for (int64_t tile = tile_first; ok && tile < p.total_tiles; tile += tile_step) {
      if (tile != tile_first) t = decode_tile(tile, p);
      const int64_t gm = (int64_t)t.tm * (BM * kCta) + rank * BM + quarter * 32 + lane;
      const int64_t n0 = (int64_t)t.tn * TILE_N + col0;
      void* cmat = kOutHalf ? (void*)((__half*)p.C + t.mat * p.strideC) : (void*)((float*)p.C + t.mat * p.strideC);
      const int64_t row_off = gm * p.ldc;
      const int nkb_t = (p.splits > 1) ? k_range(t.mat, p).count : nkb;
      const int nwin = (nkb_t + chunk_kb - 1) / chunk_kb;
      if (!kWindowed) {
        // A 512-wide tile is drained half by half (half h lives in accumulator buffer h and is
        // published on its own, the left one while the right one's last MMAs still run); every
        // epilogue warp takes its share of the columns of each half.
        constexpr int COLS_PER_PART = kBN / COL_SPLIT;
#pragma unroll 1
        for (int h = 0; h < kNSplit && ok; h++) {
        const uint32_t slot = (kNSplit == 2) ? (uint32_t)h : win % ACC_SLOTS;
        const uint32_t par = (kNSplit == 2) ? (win & 1) : ((win / ACC_SLOTS) & 1);
        const bool got = mbar_wait_warp(bar_tfull + 8 * slot, par, abortp, lane);
        if (!got) {
          if (lane == 0) { atomicOr(p.status, kDevTimeoutEpilogue); abort_flag = 1; }
          ok = false;
          break;
        }
        tc_fence_after();
        const int part0 = col_part * COLS_PER_PART;
        const uint32_t tbase = tmem_base + lane_base + slot * kBN + part0;
        const int64_t n0h = (int64_t)t.tn * TILE_N + h * kBN + part0;
        if (p.tma_store) {
          // Each warp rounds its 32 rows x 128 bytes into a swizzled staging buffer and one lane
          // sends it with a TMA store (full 128-byte lines); two buffers per warp alternate.
          constexpr int COLS_PER_BUF = kOutHalf ? 64 : 32;   // columns in one 128-byte staging row
          constexpr int LOADS = STG_BUFS * (kOutHalf ? 2 : 1);   // tcgen05.ld.x32 per pass (all staging buffers)
          static_assert(COLS_PER_PART % (STG_BUFS * COLS_PER_BUF) == 0, "a pass fills every staging buffer");
          const int m_warp = t.tm * (BM * kCta) + (int)rank * BM + quarter * 32;
          const uint32_t row_addr = stg_base + (uint32_t)lane * 128u;
          const uint32_t sw = (uint32_t)(lane & 7);
#pragma unroll 1
          for (int c = 0; c < COLS_PER_PART; c += STG_BUFS * COLS_PER_BUF) {
            uint32_t r[LOADS][32];
#pragma unroll
            for (int l = 0; l < LOADS; l++) tmem_ld_x32(tbase + c + 32 * l, r[l]);
            tmem_ld_wait();
            // The previous pass's stores must have finished reading the buffers; they had the
            // whole tensor-memory load above to do so.
            if (store_leader) bulk_wait_read<0>();
            __syncwarp();
#pragma unroll
            for (int l = 0; l < LOADS; l++) {
              if (kOutHalf) {
                // load l covers columns 32l..32l+31 = 16-byte chunks 4(l&1)..4(l&1)+3 of buffer l>>1
                const uint32_t buf = row_addr + (uint32_t)(l >> 1) * 4096u;
#pragma unroll
                for (int q = 0; q < 4; q++) {
                  float x[8];
#pragma unroll
                  for (int e = 0; e < 8; e++) x[e] = __uint_as_float(r[l][q * 8 + e]);
                  if (p.bias) add_bias<true, 8>(p.bias, n0h + c + 32 * l + q * 8, p.N, x);
                  uint32_t hh[4];
#pragma unroll
                  for (int e = 0; e < 4; e++) {
                    __half2 v2 = __floats2half2_rn(x[2 * e], x[2 * e + 1]);
                    hh[e] = *(uint32_t*)&v2;
                  }
                  st_shared_v4(buf + (((uint32_t)(q + 4 * (l & 1)) ^ sw) << 4), hh[0], hh[1], hh[2], hh[3]);
                }
              } else {
                const uint32_t buf = row_addr + (uint32_t)l * 4096u;
#pragma unroll
                for (int q = 0; q < 8; q++) {
                  float x[4];
#pragma unroll
                  for (int e = 0; e < 4; e++) x[e] = __uint_as_float(r[l][q * 4 + e]);
                  if (p.bias) add_bias<false, 4>(p.bias, n0h + c + 32 * l + q * 4, p.N, x);
                  st_shared_v4(buf + (((uint32_t)q ^ sw) << 4), __float_as_uint(x[0]), __float_as_uint(x[1]),
                               __float_as_uint(x[2]), __float_as_uint(x[3]));
                }
              }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (store_leader && m_warp < p.M) {
#pragma unroll
              for (int b2 = 0; b2 < STG_BUFS; b2++) {
                const int64_t col = n0h + c + b2 * COLS_PER_BUF;
                if (col < p.N) {
                  for (int d = 0; d < p.n_out; d++)
                    tma_store_3d(&mapC.m[d], stg_base + (uint32_t)b2 * 4096u, (int)col, m_warp, (int)t.mat);
                }
              }
              bulk_commit();
            }
          }
        } else {
#pragma unroll 1
          for (int c = 0; c < COLS_PER_PART; c += 32) {
            uint32_t r[32];
            tmem_ld_x32(tbase + c, r);
            tmem_ld_wait();
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] = __uint_as_float(r[j]);
            if (p.bias) add_bias<kOutHalf, 32>(p.bias, n0h + c, p.N, v);
            if (gm < p.M && n0h + c < p.N) store_row32<kOutHalf>(cmat, row_off, n0h + c, p.N, v, p.vec_ok != 0);
          }
        }
        tc_fence_before();
        mbar_arrive_cluster_relaxed(tempty_leader + 8 * slot);
        }
        win++;
      } else {
        float acc[COLS_PER_THREAD];
        for (int w = 0; w < nwin && ok; w++) {
          const uint32_t slot = win & 1;
          const bool got = mbar_wait_warp(bar_tfull + 8 * slot, (win >> 1) & 1, abortp, lane);
          if (!got) {
            if (lane == 0) { atomicOr(p.status, kDevTimeoutEpilogue); abort_flag = 1; }
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t tbase = tmem_base + lane_base + slot * kBN + col0;
#pragma unroll
          for (int c = 0; c < COLS_PER_THREAD; c += 32) {
            uint32_t r[32];
            tmem_ld_x32(tbase + c, r);
            tmem_ld_wait();
            if (w == 0) {
#pragma unroll
              for (int j = 0; j < 32; j++) acc[c + j] = __uint_as_float(r[j]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; j++) acc[c + j] = __fadd_rn(acc[c + j], __uint_as_float(r[j]));
            }
          }
          tc_fence_before();
          mbar_arrive_cluster_relaxed(tempty_leader + 8 * slot);
          win++;
        }
        if (ok && p.tma_store) {
          // Same staging as above, fed from the register accumulators: one buffer, 32 columns per pass.
          const int m_warp = t.tm * (BM * kCta) + (int)rank * BM + quarter * 32;
          const uint32_t row_addr = stg_base + (uint32_t)lane * 128u;
          const uint32_t sw = (uint32_t)(lane & 7);
#pragma unroll
          for (int c = 0; c < COLS_PER_THREAD; c += 32) {
            if (store_leader) bulk_wait_read<0>();
            __syncwarp();
#pragma unroll
            for (int q = 0; q < 8; q++) {
              float x[4];
#pragma unroll
              for (int e = 0; e < 4; e++) x[e] = acc[c + q * 4 + e];
              if (p.bias) add_bias<false, 4>(p.bias, n0 + c + q * 4, p.N, x);
              st_shared_v4(row_addr + (((uint32_t)q ^ sw) << 4), __float_as_uint(x[0]), __float_as_uint(x[1]),
                           __float_as_uint(x[2]), __float_as_uint(x[3]));
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (store_leader && m_warp < p.M && n0 + c < p.N) {
              for (int d = 0; d < p.n_out; d++) tma_store_3d(&mapC.m[d], stg_base, (int)(n0 + c), m_warp, (int)t.mat);
              bulk_commit();
            }
          }
        } else if (ok && gm < p.M) {
#pragma unroll
          for (int c = 0; c < COLS_PER_THREAD; c += 32) {
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] = acc[c + j];
            if (p.bias) add_bias<kOutHalf, 32>(p.bias, n0 + c, p.N, v);
            if (n0 + c < p.N) store_row32<kOutHalf>(cmat, row_off, n0 + c, p.N, v, p.vec_ok != 0);
          }
        }
      }
    }
  }

  if (warp >= 2 && warp < kWarpProducerB) {
    // Shared memory must outlive the TMA stores that read it.  Their writes to this device are
    // complete when the grid is (no wait needed: about 450 clocks saved at the end of every
    // launch); stores into other devices' memory are waited for in full.
    __syncwarp();
    if (elect_one()) {
      if (p.n_out > 1) bulk_wait_all();
      else bulk_wait_read<0>();
    }
  }
  // ---------------------------------------------------------------- teardown
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (kCta == 2) cluster_rendezvous();   // neither CTA leaves while the other may still signal it
  tc_fence_after();
  if (abort_flag) {
    // Give copies and MMAs that were already issued time to land before the CTA's
    // shared and tensor memory are handed to another CTA.
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) { __nanosleep(1000); }
    __syncthreads();
  }
  if (warp == 1) {
    if (kCta == 2) {
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                   : "memory");
    } else {
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                   : "memory");
    }
  }
}

// Self-test of the bounded wait: one thread waits on a barrier that nothing will ever arrive
// on, with a short limit, through the same wait routine the GEMM kernel uses.  The wait gives
// up, the status word gets its bit, and the kernel returns normally.
__global__ void wait_probe_kernel(unsigned int* status, unsigned long long limit_ns) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!mbar_wait_slow(smem_u32(&bar), 0, &abort_flag, limit_ns)) atomicOr(status, kDevTimeoutSelfTest);
  }
}

// Second half of a cut contraction: result = round(sum over parts, ascending, of the float32
// partial matrices) (+ bias, as a second rounded operation for float16, exactly like the
// epilogue of the uncut kernel).  Four columns per thread; the partial matrices have a row pitch
// that is a multiple of four floats, so every load is one aligned float4.
struct ReduceJob {
  const float* ws;
  void* C;
  const void* bias;
  int64_t M, N, ws_ld, batch, ldc, strideC;
  int parts, vec_ok;
};

template <bool kHalf>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const ReduceJob j) {
  pdl_release();
  pdl_wait();
  const int64_t groups = j.ws_ld / 4;
  const int64_t total = j.batch * j.M * groups;
  const int64_t part_stride = j.M * j.ws_ld;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t g = i % groups, row = (i / groups) % j.M, mat = i / (groups * j.M);
    const int64_t n = g * 4;
    const float* src = j.ws + (mat * j.parts) * part_stride + row * j.ws_ld + n;
    float4 acc = __ldg((const float4*)src);
    for (int z = 1; z < j.parts; z++) {
      const float4 v = __ldg((const float4*)(src + z * part_stride));
      acc.x = __fadd_rn(acc.x, v.x); acc.y = __fadd_rn(acc.y, v.y);
      acc.z = __fadd_rn(acc.z, v.z); acc.w = __fadd_rn(acc.w, v.w);
    }
    float x[4] = {acc.x, acc.y, acc.z, acc.w};
    const int valid = (int)min((int64_t)4, j.N - n);
    if (kHalf) {
      __half h[4];
#pragma unroll
      for (int e = 0; e < 4; e++) {
        h[e] = __float2half_rn(x[e]);
        if (j.bias && e < valid)
          h[e] = __float2half_rn(__fadd_rn(__half2float(h[e]), __half2float(__ldg((const __half*)j.bias + n + e))));
      }
      __half* dst = (__half*)j.C + mat * j.strideC + row * j.ldc + n;
      if (valid == 4 && j.vec_ok) {
        *(uint2*)dst = *(const uint2*)h;
      } else {
        for (int e = 0; e < valid; e++) dst[e] = h[e];
      }
    } else {
      if (j.bias)
#pragma unroll
        for (int e = 0; e < 4; e++)
          if (e < valid) x[e] = __fadd_rn(x[e], __ldg((const float*)j.bias + n + e));
      float* dst = (float*)j.C + mat * j.strideC + row * j.ldc + n;
      if (valid == 4 && j.vec_ok) {
        *(float4*)dst = make_float4(x[0], x[1], x[2], x[3]);
      } else {
        for (int e = 0; e < valid; e++) dst[e] = x[e];
      }
    }
  }
}

// float32 as two TF32 operands: x = hi + lo with hi = x truncated to TF32's 10 mantissa bits and
// lo = nearest TF32 of (x - hi), which is exact in float32.  hi is never computed: kind::tf32
// reads a float32 operand by dropping its low 13 mantissa bits (measured on both operands: the
// MMA of 1 + 2^-11 + 2^-12 by 1 gives 1, not the 1 + 2^-10 rounding would give), so the operand
// itself serves as hi and only lo is written.  Non-finite x: lo = 0, so infinities and NaNs
// propagate through the hi*hi product only.
struct SplitJob {
  const float* src;
  float *hi, *lo;     // hi: null, or where to put a TMA-addressable copy of src
  int64_t rows, width, ld_src, ld_dst, stride_src, stride_dst, batch;
  int vec4;   // rows, pitches and bases allow 16-byte accesses
};

__device__ __forceinline__ float split_lo(float x) {
  if (!isfinite(x)) return 0.0f;
  const float d = x - __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
  uint32_t lbits;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lbits) : "f"(d));
  return __uint_as_float(lbits & 0xFFFFE000u);
}

// One launch splits both operands: the first `blocks_a` blocks work on A, the rest on B.
__global__ void __launch_bounds__(256) split_tf32_kernel(const SplitJob ja, const SplitJob jb, int blocks_a) {
  pdl_release();
  pdl_wait();
  const bool is_a = (int)blockIdx.x < blocks_a;
  const SplitJob& j = is_a ? ja : jb;
  const int64_t bid = is_a ? blockIdx.x : blockIdx.x - blocks_a;
  const int64_t nblk = is_a ? blocks_a : (int64_t)gridDim.x - blocks_a;
  if (j.vec4) {
    const int64_t w4 = j.width / 4, total = j.batch * j.rows * w4;
    for (int64_t i = bid * blockDim.x + threadIdx.x; i < total; i += nblk * blockDim.x) {
      const int64_t c = (i % w4) * 4, r = (i / w4) % j.rows, b = i / (w4 * j.rows);
      const float4 x = *(const float4*)(j.src + b * j.stride_src + r * j.ld_src + c);
      if (j.hi) *(float4*)(j.hi + b * j.stride_dst + r * j.ld_dst + c) = x;
      *(float4*)(j.lo + b * j.stride_dst + r * j.ld_dst + c) =
          make_float4(split_lo(x.x), split_lo(x.y), split_lo(x.z), split_lo(x.w));
    }
  } else {
    const int64_t total = j.batch * j.rows * j.width;
    for (int64_t i = bid * blockDim.x + threadIdx.x; i < total; i += nblk * blockDim.x) {
      const int64_t c = i % j.width, r = (i / j.width) % j.rows, b = i / (j.width * j.rows);
      const float x = j.src[b * j.stride_src + r * j.ld_src + c];
      if (j.hi) j.hi[b * j.stride_dst + r * j.ld_dst + c] = x;
      j.lo[b * j.stride_dst + r * j.ld_dst + c] = split_lo(x);
    }
  }
}

// float16 operands whose base or pitches TMA cannot address are copied once into a packed,
// 16-byte aligned area (same values, leading dimension rounded up to eight elements).
struct RepackJob {
  const __half* src;
  __half* dst;
  int64_t rows, width, ld_src, ld_dst, stride_src, stride_dst, batch;
};
__global__ void __launch_bounds__(256) repack_f16_kernel(const RepackJob ja, const RepackJob jb, int blocks_a) {
  pdl_release();
  pdl_wait();
  const bool is_a = (int)blockIdx.x < blocks_a;
  const RepackJob& j = is_a ? ja : jb;
  const int64_t bid = is_a ? blockIdx.x : blockIdx.x - blocks_a;
  const int64_t nblk = is_a ? blocks_a : (int64_t)gridDim.x - blocks_a;
  const int64_t total = j.batch * j.rows * j.width;
  for (int64_t i = bid * blockDim.x + threadIdx.x; i < total; i += nblk * blockDim.x) {
    const int64_t c = i % j.width, r = (i / j.width) % j.rows, b = i / (j.width * j.rows);
    j.dst[b * j.stride_dst + r * j.ld_dst + c] = j.src[b * j.stride_src + r * j.ld_src + c];
  }
}

// ---- host side ------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

// One operand as a rank-3 tensor {contiguous index, other index, matrix}.
// `box_rows` is the number of M (or N) indices one load brings in for a K-major operand; an
// MN-major operand is always loaded in boxes of one 128-byte row of indices by one k-slab.
bool make_operand_map(CUtensorMap* map, const void* base, int elem_bytes, bool mn_major, int64_t mn, int64_t k,
                      int64_t ld, int64_t stride_mat, int64_t batch, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const int per_row = 128 / elem_bytes;
  cuuint64_t dims[3] = {(cuuint64_t)(mn_major ? mn : k), (cuuint64_t)(mn_major ? k : mn), (cuuint64_t)batch};
  cuuint64_t mat_bytes = (cuuint64_t)stride_mat * elem_bytes;
  if (batch == 1) mat_bytes = (cuuint64_t)ld * elem_bytes * dims[1];
  cuuint64_t strides[2] = {(cuuint64_t)ld * elem_bytes, mat_bytes};
  cuuint32_t box[3] = {(cuuint32_t)per_row, (cuuint32_t)(mn_major ? per_row : box_rows), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  // 32-bit MN-major operands must use the swizzle that permutes 32-byte units (the only one
  // tcgen05.mma accepts for them); everything else the usual 16-byte-unit 128B swizzle.
  const CUtensorMapSwizzle swz =
      (mn_major && elem_bytes == 4) ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B;
  CUresult r = fn(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// The result as a rank-3 tensor {column, row, matrix}; one store moves 32 rows x 128 bytes.
bool make_output_map(CUtensorMap* map, void* base, int elem_bytes, int64_t n, int64_t m, int64_t ldc,
                     int64_t stride_mat, int64_t batch) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {(cuuint64_t)n, (cuuint64_t)m, (cuuint64_t)batch};
  cuuint64_t mat_bytes = (cuuint64_t)stride_mat * elem_bytes;
  if (batch == 1) mat_bytes = (cuuint64_t)ldc * elem_bytes * dims[1];
  cuuint64_t strides[2] = {(cuuint64_t)ldc * elem_bytes, mat_bytes};
  cuuint32_t box[3] = {(cuuint32_t)(128 / elem_bytes), 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, base,
                  dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

bool operand_ok(const void* base, int elem_bytes, int64_t ld, int64_t stride_mat, int64_t batch, int64_t d0,
                int64_t d1) {
  if (((uintptr_t)base & 15) != 0) return false;
  if ((ld * elem_bytes) % 16 != 0) return false;
  if (batch > 1 && (stride_mat * elem_bytes) % 16 != 0) return false;
  if (d0 >= (1ll << 31) || d1 >= (1ll << 31) || batch >= (1ll << 31)) return false;
  if (ld * elem_bytes >= (1ll << 40) || stride_mat * elem_bytes >= (1ll << 40)) return false;
  return true;
}

// Thresholds of the tile-shape model.  In the shipped library they are constants.  A library
// built with -DHC_DIAGNOSTICS (the test-suite's second build) can move them, force a tile shape
// or a cut of the contraction from the environment, read at every launch, so that small test
// products reach every code path; none of the switches changes what a product computes.
struct Tunables {
  int wide_min_kb = 32;   // HC_TC_WIDE_MIN_KB: k blocks from which the 256x512 tile is considered
  int shape = 0;          // HC_TC_SHAPE: force a tile shape (1..6)
  int splits = 0;         // HC_TC_SPLITS: 1 never cut the contraction, n > 1 cut into n parts
  int short_k = 8;        // HC_TC_SHORT_K: slabs up to which the eight-warp epilogue config is used
  int group_m = 0;        // HC_TC_GROUP_M: tile rows sharing a sweep over the columns (0: default)
  int wide_epi8 = 1;      // HC_TC_WIDE_EPI8: eight epilogue warps on the 256x512 tile
};
#ifdef HC_DIAGNOSTICS
Tunables read_tunables() {
  Tunables t;
  for (char** e = environ; e && *e; e++) {
    const char* s = *e;
    if (s[0] != 'H' || strncmp(s, "HC_TC_", 6) != 0) continue;
    const char* eq = strchr(s, '=');
    if (!eq) continue;
    const char* k = s + 6;
    const size_t n = (size_t)(eq - k);
    const int v = atoi(eq + 1);
    if (n == 5 && !strncmp(k, "SHAPE", 5)) t.shape = v;
    else if (n == 6 && !strncmp(k, "SPLITS", 6)) t.splits = v;
    else if (n == 11 && !strncmp(k, "WIDE_MIN_KB", 11)) t.wide_min_kb = v;
    else if (n == 7 && !strncmp(k, "SHORT_K", 7)) t.short_k = v;
    else if (n == 7 && !strncmp(k, "GROUP_M", 7)) t.group_m = v;
    else if (n == 9 && !strncmp(k, "WIDE_EPI8", 9)) t.wide_epi8 = v;
  }
  return t;
}
int env_int(const char* name, int fallback) {
  const char* e = getenv(name);
  return e ? atoi(e) : fallback;
}
// HC_TC_DEBUG bits: 2 = no accumulation windows, 4 = never pair CTAs, 128 = direct stores instead
// of TMA stores
int debug_flags() {
  static int v = env_int("HC_TC_DEBUG", 0);
  return v;
}
// Slabs of the original contraction per accumulation window of a float32 product.
int window_slabs() {
  static int v = env_int("HC_TC_WINDOW_SLABS", 4);
  return v < 1 ? 1 : v;
}
// HC_TC_PDL=0 launches without programmatic dependent launch.
bool overlap_launches() {
  static int v = env_int("HC_TC_PDL", 1);
  return v != 0;
}
constexpr bool kPlanCacheEnabled = false;   // the switches are read per launch
#else
inline Tunables read_tunables() { return Tunables(); }
constexpr int debug_flags() { return 0; }
constexpr int window_slabs() { return 4; }
// Successive kernels of this library in one stream overlap their prologue with the
// predecessor's tail (programmatic dependent launch).
constexpr bool overlap_launches() { return true; }
constexpr bool kPlanCacheEnabled = true;
#endif

template <int kElemBytes, int kBN, int kStages, int kEpiWarps, bool kWindowed, int kCta, int kNSplit = 1, int kSlabs = 1,
          bool kPartial = false>
struct TcConfig {
  // operand ring (float32 slots also hold the lo slabs) + store staging + alignment slack
  static constexpr size_t smem = (size_t)kStages * kSlabs * (kElemBytes == 4 ? 2 : 1) * (BM * 128 + kNSplit * (kBN / kCta) * 128) +
                                 (size_t)kEpiWarps * staging_bufs((kElemBytes == 2 && !kPartial) ? 2 : 4, kBN, kEpiWarps, kWindowed, kNSplit) * 4096 + 1024;
  static_assert(smem <= 232448, "more shared memory than one CTA can have on sm_100");
  static constexpr int block = 96 + 32 * kEpiWarps;   // producers A and B, MMA issuer, epilogue warps
  static auto kernel() { return tc_gemm_kernel<kElemBytes, kBN, kStages, kEpiWarps, kWindowed, kCta, kNSplit, kSlabs, kPartial>; }

  static cudaError_t configure() {
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !configured[dev]) {
      cudaError_t e = cudaFuncSetAttribute(kernel(), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
      // All of the SM's configurable memory as shared memory: nothing here uses the L1 cache.
      e = cudaFuncSetAttribute(kernel(), cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
      if (e != cudaSuccess) cudaGetLastError();
      if (kCta == 2) {
        e = cudaFuncSetAttribute(kernel(), cudaFuncAttributeNonPortableClusterSizeAllowed, 0);
        if (e != cudaSuccess) cudaGetLastError();
      }
      configured[dev] = true;
    }
    return cudaSuccess;
  }

  // CTA pairs that can be resident at once (pairs need two free SMs of one cluster-capable
  // group; on some parts that leaves a few SMs unpaired).
  static int max_pairs(int sm_count) {
    static int cached[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && cached[dev]) return cached[dev];
    configure();   // the answer depends on the shared-memory attributes
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(sm_count * 4));   // more than can be resident: the answer is the limit
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel(), &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sm_count / 2;
    }
    if (dev < 64) cached[dev] = n;
    return n;
  }

  static cudaError_t launch(const CUtensorMap maps[4], const OutMaps& outs, const TcParams& p, int sm_count,
                            cudaStream_t stream, LaunchRecord* rec) {
    cudaError_t e = configure();
    if (e != cudaSuccess) return e;
    int64_t groups = (kCta == 2) ? max_pairs(sm_count) : sm_count;
    if (p.total_tiles < groups) groups = p.total_tiles;
    const int grid = (int)groups * kCta;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kCta; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap_launches() ? 2 : 1;
    e = cudaLaunchKernelEx(&cfg, kernel(), maps[0], maps[1], maps[2], maps[3], outs, p);
    if (rec) {
      rec->tile_m = BM * kCta; rec->tile_n = kBN * kNSplit; rec->tile_k = kSlabs * 128 / kElemBytes; rec->stages = kStages;
      rec->grid = grid; rec->block = block; rec->launches++;
    }
    // cudaLaunchKernelEx reports this launch's own failure; the thread's sticky-less "last error"
    // may hold another library's earlier error and is not this launch's to report.
    return e;
  }
};

}  // namespace

cudaError_t launch_wait_probe(cudaStream_t stream, unsigned int* status_word, unsigned long long limit_ns) {
  wait_probe_kernel<<<1, 32, 0, stream>>>(status_word, limit_ns);
  return cudaGetLastError();
}

// Any product of sane size runs on the tensor cores: operands TMA cannot address directly
// (unaligned base, pitches that are not 16-byte multiples) are repacked into the work area first
// - the float32 split does that anyway - and a result TMA cannot address is stored from registers.
bool tc_supported(const GemmProblem& p) {
  if (p.M <= 0 || p.N <= 0 || p.K <= 0 || p.batch <= 0) return false;
  if (p.M >= (1ll << 31) - 256 || p.N >= (1ll << 31) - 256 || p.K >= (1ll << 31) - 256 || p.batch >= (1ll << 31))
    return false;
  return encode_fn() != nullptr;
}

// float32 products: the lo halves of both operands are stored compactly, with the leading
// dimension rounded up to four elements so TMA can address them.  The hi half is the operand
// where it lies; only an operand TMA cannot address (base or pitches not multiples of 16 bytes)
// is also copied, into the same compact layout.
static inline int64_t round4(int64_t x) { return (x + 3) & ~3ll; }
struct SplitLayout {
  int64_t a_rows, a_width, a_ld, a_mat, b_rows, b_width, b_ld, b_mat;
  size_t a_bytes, b_bytes;   // of one compact array
  bool a_copy, b_copy;       // the operand needs a TMA-addressable copy as its hi half
};
static SplitLayout split_layout(const GemmProblem& p) {
  SplitLayout s;
  s.a_rows = p.a_mn_major ? p.K : p.M; s.a_width = p.a_mn_major ? p.M : p.K;
  s.b_rows = p.b_mn_major ? p.K : p.N; s.b_width = p.b_mn_major ? p.N : p.K;
  s.a_ld = round4(s.a_width); s.b_ld = round4(s.b_width);
  s.a_mat = s.a_rows * s.a_ld; s.b_mat = s.b_rows * s.b_ld;
  s.a_bytes = ((size_t)(s.a_mat * p.batch) * 4 + 255) & ~(size_t)255;
  s.b_bytes = ((size_t)(s.b_mat * p.batch) * 4 + 255) & ~(size_t)255;
  s.a_copy = !operand_ok(p.A, 4, p.lda, p.strideA, p.batch, p.M, p.K);
  s.b_copy = !operand_ok(p.B, 4, p.ldb, p.strideB, p.batch, p.N, p.K);
  return s;
}

// float16 operands that need repacking: packed copy with the leading dimension rounded to 8.
struct RepackLayout {
  bool a, b;
  int64_t a_rows, a_width, a_ld, a_mat, b_rows, b_width, b_ld, b_mat;
  size_t a_bytes, b_bytes;
};
static RepackLayout repack_layout(const GemmProblem& p) {
  RepackLayout r;
  r.a = !operand_ok(p.A, 2, p.lda, p.strideA, p.batch, p.M, p.K);
  r.b = !operand_ok(p.B, 2, p.ldb, p.strideB, p.batch, p.N, p.K);
  r.a_rows = p.a_mn_major ? p.K : p.M; r.a_width = p.a_mn_major ? p.M : p.K;
  r.b_rows = p.b_mn_major ? p.K : p.N; r.b_width = p.b_mn_major ? p.N : p.K;
  r.a_ld = (r.a_width + 7) & ~7ll; r.b_ld = (r.b_width + 7) & ~7ll;
  r.a_mat = r.a_rows * r.a_ld; r.b_mat = r.b_rows * r.b_ld;
  r.a_bytes = r.a ? (((size_t)(r.a_mat * p.batch) * 2 + 255) & ~(size_t)255) : 0;
  r.b_bytes = r.b ? (((size_t)(r.b_mat * p.batch) * 2 + 255) & ~(size_t)255) : 0;
  return r;
}

// ---- choice of tile shape and of a cut of the contraction ------------------------------------
enum Shape { SHAPE_AUTO = 0, SHAPE_WIDE, SHAPE_PAIR, SHAPE_C1_256, SHAPE_C1_128, SHAPE_PAIR_128, SHAPE_PAIR_64,
             SHAPE_COUNT };

struct TcPlan {
  int shape = SHAPE_PAIR;
  int slabs = 1;            // k slabs per pipeline slot
  int splits = 1;           // parts of the contraction (1: none)
  int kb_per_split = 0;     // slots per part
  int64_t ws_ld = 0;        // row pitch (floats) of one partial matrix
  size_t ws_bytes = 0;      // float32 partial sums: splits x batch x M x ws_ld
};

constexpr size_t kMaxSplitWorkspace = 256ull << 20;

// The cost model.  A shape costs (waves of tiles over the SMs) x (clocks per tile); the clocks
// per 64-wide k block of each float16 shape are measured on large products (relative to 600 for
// the 256x256 pair), plus a fixed cost per tile for refilling the pipeline.  Large tiles move the
// fewest operand bytes per flop and win whenever there are enough tiles to fill the SMs; for small
// products the small pair shapes spread the work over more SMs, which shortens the one wave there
// is.  Only the 256x512 shape cannot hide the result drain behind the next tile.
// When even the smallest shape leaves most SMs idle and the contraction is long (the weight
// gradient of a small Linear layer: few outputs, many tokens), the contraction is cut into up to
// 16 parts that run as separate tiles into float32 partial matrices, summed in ascending part
// order by a second kernel (splitk_reduce_kernel): deterministic, and float16 still rounds once.
// float32 (3xTF32, 12 MMAs per 32-wide slab) goes through the same model with its own clocks.
TcPlan plan_tc(const GemmProblem& p, int sm_count, bool may_split, const Tunables& tun) {
  const bool f32 = p.dtype == HC_F32;
  const int BK = f32 ? 32 : 64;
  const int dbg = debug_flags();
  const int kslabs = (int)((p.K + BK - 1) / BK);
  // A block of a larger product is planned as the whole product.
  const int64_t M = p.plan_M > 0 ? p.plan_M : p.M, N = p.plan_N > 0 ? p.plan_N : p.N;
  const bool pairs_ok = M > BM && !(dbg & 4);
  struct Cand { int shape; bool ok; int rows, cols, slots, slabs; double clk_per_slab, drain_per_tile; bool splittable; };
  const double drain = 2400.0, refill = 300.0;
  const int pair_slots = sm_count / 2;
  Cand cands[SHAPE_COUNT - 1];
  int n_cands = 0;
  if (!f32) {
    const bool wide_ok = pairs_ok && N >= 1024 && kslabs >= tun.wide_min_kb;
    cands[n_cands++] = {SHAPE_WIDE, wide_ok, 256, 512, pair_slots, 1, 1140.0, drain, false};
    cands[n_cands++] = {SHAPE_PAIR, pairs_ok && N > 128, 256, 256, pair_slots, 1, 600.0, 0.0, true};
    cands[n_cands++] = {SHAPE_C1_256, N > 128, 128, 256, sm_count, 1, 680.0, 0.0, false};
    cands[n_cands++] = {SHAPE_C1_128, true, 128, 128, sm_count, 2, 410.0, 0.0, true};
    cands[n_cands++] = {SHAPE_PAIR_128, pairs_ok && N > 64, 256, 128, pair_slots, 2, 340.0, 0.0, true};
    // 32 columns of B per CTA: half a 128-byte row of an MN-major box, which the copy cannot split
    cands[n_cands++] = {SHAPE_PAIR_64, pairs_ok && !p.b_mn_major, 256, 64, pair_slots, 2, 265.0, 0.0, true};
  } else {
    // float32 (3xTF32): 12 MMAs per 32-wide slab; clocks per slab measured the same way.  The small
    // pair shapes need the windowed epilogue (they are not built for the no-window debug mode).
    const bool small_ok = pairs_ok && !(dbg & 2);
    cands[n_cands++] = {SHAPE_WIDE, false, 256, 512, pair_slots, 1, 0.0, 0.0, false};
    cands[n_cands++] = {SHAPE_PAIR, pairs_ok && N > 128, 256, 256, pair_slots, 1, 1700.0, 0.0, true};
    cands[n_cands++] = {SHAPE_C1_256, N > 128, 128, 256, sm_count, 1, 1900.0, 0.0, true};
    cands[n_cands++] = {SHAPE_C1_128, true, 128, 128, sm_count, 1, 1130.0, 0.0, true};
    cands[n_cands++] = {SHAPE_PAIR_128, small_ok && N > 64, 256, 128, pair_slots, 1, 950.0, 0.0, true};
    cands[n_cands++] = {SHAPE_PAIR_64, small_ok, 256, 64, pair_slots, 1, 615.0, 0.0, true};
  }
  const int forced = tun.shape;
  const int forced_splits = tun.splits;   // 1: never cut; n > 1: cut into n where possible
  int choices[8] = {1, 2, 3, 4, 6, 8, 12, 16};
  int n_choices = 8;
  if (forced_splits > 1) { choices[0] = forced_splits > 64 ? 64 : forced_splits; n_choices = 1; }
  TcPlan best;
  double best_cost = -1.0;
  for (int ci = 0; ci < n_cands; ci++) {
    const Cand& c = cands[ci];
    if (!c.ok || c.slots < 1) continue;
    if (forced >= 1 && forced < SHAPE_COUNT && cands[forced - 1].ok && c.shape != forced) continue;
    const int64_t tiles = ((M + c.rows - 1) / c.rows) * ((N + c.cols - 1) / c.cols) * p.batch;
    const int kslots = (kslabs + c.slabs - 1) / c.slabs;
    const int64_t ws_ld = (p.N + 3) & ~3ll;   // of this block
    // (matrix index x parts must stay a 32-bit tensor-map coordinate)
    const bool can_split = may_split && c.splittable && !p.no_split && forced_splits != 1 && p.batch < (1ll << 24);
    for (int i = 0; i < n_choices; i++) {
      int want = can_split ? choices[i] : 1;
      if (want > kslots) want = kslots;
      if (want < 1) want = 1;
      int per = (kslots + want - 1) / want;
      if (want > 1 && forced_splits <= 1 && per * c.slabs < 8) break;   // at least 8 slabs per part
      if (want > 1 && forced_splits <= 1 && tiles >= c.slots) break;    // a full wave needs no cut
      const int parts = (kslots + per - 1) / per;
      const size_t ws = parts > 1 ? (size_t)parts * p.batch * p.M * ws_ld * 4 : 0;
      // the limit applies to the whole product, so that a block of it is cut like the whole
      if (parts > 1 && (size_t)parts * p.batch * M * ((N + 3) & ~3ll) * 4 > kMaxSplitWorkspace) break;
      const int64_t units = tiles * parts;
      const int64_t waves = (units + c.slots - 1) / c.slots;
      double cost = (double)waves * ((double)per * c.slabs * c.clk_per_slab + c.drain_per_tile + refill) +
                    (c.drain_per_tile > 0 ? 0.0 : drain);
      if (parts > 1) cost += 2500.0 + (double)ws / 3000.0;   // the second launch and its traffic
      if (best_cost < 0 || cost < best_cost) {
        best_cost = cost;
        best.shape = c.shape; best.slabs = c.slabs; best.splits = parts; best.kb_per_split = per;
        best.ws_ld = ws_ld; best.ws_bytes = ws;
      }
      if (!can_split) break;
    }
  }
  return best;
}

static size_t operand_scratch_bytes(const GemmProblem& p) {
  if (p.dtype != HC_F32) {
    const RepackLayout r = repack_layout(p);
    return r.a_bytes + r.b_bytes;
  }
  const SplitLayout s = split_layout(p);
  return (s.a_copy ? 2 : 1) * s.a_bytes + (s.b_copy ? 2 : 1) * s.b_bytes;
}

// Work area of one product: re-laid operands (float32 hi/lo parts, repacked float16), then,
// 256-byte aligned, the partial matrices of a cut contraction.
size_t tc_scratch_bytes(const GemmProblem& p, int sm_count) {
  const size_t ops = operand_scratch_bytes(p);
  const TcPlan plan = plan_tc(p, sm_count, true, read_tunables());
  return plan.ws_bytes ? ((ops + 255) & ~(size_t)255) + plan.ws_bytes : ops;
}

PlanSummary tc_describe_plan(const GemmProblem& p, int sm_count) {
  const TcPlan plan = plan_tc(p, sm_count, true, read_tunables());
  static const int kRows[SHAPE_COUNT] = {0, 256, 256, 128, 128, 256, 256};
  static const int kCols[SHAPE_COUNT] = {0, 512, 256, 256, 128, 128, 64};
  PlanSummary r;
  r.tile_m = kRows[plan.shape]; r.tile_n = kCols[plan.shape];
  r.ctas = r.tile_m / BM;
  r.slabs = plan.slabs; r.parts = plan.splits;
  const int BK = p.dtype == HC_F32 ? 32 : 64;
  const int kslots = (int)(((p.K + BK - 1) / BK + plan.slabs - 1) / plan.slabs);
  r.slots_per_part = plan.splits > 1 ? plan.kb_per_split : kslots;
  r.tiles = ((p.M + r.tile_m - 1) / r.tile_m) * ((p.N + r.tile_n - 1) / r.tile_n) * p.batch * plan.splits;
  r.ws_bytes = plan.ws_bytes;
  return r;
}

// ---- a product, prepared once and issued many times ------------------------------------------
// Planning a product (tile shape, cut, tensor maps: four driver calls) costs the host several
// microseconds, which is as long as the kernel of a small product runs.  A training loop issues
// the same products - same buffers, same shapes - step after step, so the context keeps the
// prepared launches of the products it has seen most recently and a repeat costs one lookup.
namespace {

typedef cudaError_t (*TcLaunchFn)(const CUtensorMap maps[4], const OutMaps& outs, const TcParams& p, int sm_count,
                                  cudaStream_t stream, LaunchRecord* rec);

struct TcPrepared {
  int pre = 0;                       // pre-pass: 0 none, 1 repack float16 operands, 2 split float32 operands
  RepackJob rja, rjb;
  SplitJob sja, sjb;
  int pre_blocks_a = 0, pre_blocks_b = 0;
  CUtensorMap maps[4];
  OutMaps outs;
  TcParams tp;
  TcLaunchFn fn = nullptr;
  bool cut = false;                  // second kernel sums the parts of a cut contraction
  bool reduce_half = false;
  ReduceJob job;
  int reduce_blocks = 0;
  size_t scratch_used = 0;           // bytes of the work area this product touches
  // Address ranges the main kernel reads (operands, bias) and this device's range it writes.
  uintptr_t in_lo[3] = {0, 0, 0}, in_hi[3] = {0, 0, 0};
  uintptr_t out_lo = 0, out_hi = 0;
  bool trackable = false;            // one kernel, no pre-pass, no second kernel: the ranges say it all
};

// What the tensor-core kernel most recently launched on a stream wrote.  Consulted only for
// streams the library owns (nobody else enqueues kernels there), where it decides whether the
// next kernel's operand loads may run ahead of the wait for its predecessor.
struct StreamTrack {
  cudaStream_t stream = nullptr;
  bool used = false, known = false;
  uintptr_t lo = 0, hi = 0;
  uint64_t stamp = 0;
};
std::mutex g_track_mu;
StreamTrack g_track[16];
uint64_t g_track_clock = 0;

StreamTrack* track_entry(cudaStream_t stream, bool create) {
  StreamTrack* victim = &g_track[0];
  for (auto& t : g_track) {
    if (t.used && t.stream == stream) return &t;
    if (!t.used ? victim->used : (victim->used && t.stamp < victim->stamp)) victim = &t;
  }
  if (!create) return nullptr;
  *victim = StreamTrack();
  victim->stream = stream;
  victim->used = true;
  return victim;
}


struct TcKey {
  int dtype, a_mn, b_mn, no_split, n_extra, may_split;
  int64_t batch, M, N, K, lda, ldb, ldc, sA, sB, sC, plan_M, plan_N;
  const void *A, *B, *C, *bias, *scratch, *status;
  const void* extra[kMaxOut - 1];
};

TcKey make_key(const GemmProblem& p, const void* scratch, const void* status, void* const* extra_out, int n_extra) {
  TcKey k;
  memset(&k, 0, sizeof k);
  k.dtype = (int)p.dtype; k.a_mn = p.a_mn_major; k.b_mn = p.b_mn_major; k.no_split = p.no_split ? 1 : 0;
  k.n_extra = n_extra; k.may_split = n_extra == 0;
  k.batch = p.batch; k.M = p.M; k.N = p.N; k.K = p.K; k.lda = p.lda; k.ldb = p.ldb; k.ldc = p.ldc;
  k.sA = p.strideA; k.sB = p.strideB; k.sC = p.strideC; k.plan_M = p.plan_M; k.plan_N = p.plan_N;
  k.A = p.A; k.B = p.B; k.C = p.C; k.bias = p.bias; k.scratch = scratch; k.status = status;
  for (int i = 0; i < n_extra && i < kMaxOut - 1; i++) k.extra[i] = extra_out[i];
  return k;
}

}  // namespace

struct TcCache {
  static constexpr int kEntries = 32;
  struct Entry {
    bool used = false;
    uint64_t stamp = 0;
    TcKey key;
    TcPrepared prep;
  };
  Entry e[kEntries];
  uint64_t clock = 0;
};

TcCache* tc_cache_create() { return new (std::nothrow) TcCache(); }
void tc_cache_destroy(TcCache* c) { delete c; }
void tc_cache_clear(TcCache* c) {
  if (c) for (auto& x : c->e) x.used = false;
}

namespace {

cudaError_t launch_elementwise(const void* fn, void** args, int blocks, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)blocks);
  cfg.blockDim = dim3(256);
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = overlap_launches() ? 1 : 0;
  return cudaLaunchKernelExC(&cfg, fn, args);
}

// Everything about a product that does not depend on the stream: pre-pass jobs, tensor maps,
// kernel parameters, which kernel.  `*scratch_needed` receives the work-area bytes the product
// needs; when the area given is smaller, nothing else is filled in and cudaErrorInvalidValue
// comes back, so that the caller can grow the area and ask again.
cudaError_t prepare_tc(const GemmProblem& p, unsigned int* status_word, void* scratch, size_t scratch_bytes,
                       int sm_count, void* const* extra_out, int n_extra, TcPrepared* out, size_t* scratch_needed) {
  TcPrepared& pp = *out;
  const bool f32 = p.dtype == HC_F32;
  const int eb = f32 ? 4 : 2;
  const int BK = 128 / eb;
  const Tunables tun = read_tunables();
  const TcPlan plan = plan_tc(p, sm_count, n_extra == 0, tun);
  const size_t ops_bytes = operand_scratch_bytes(p);
  const size_t need = plan.ws_bytes ? ((ops_bytes + 255) & ~(size_t)255) + plan.ws_bytes : ops_bytes;
  if (scratch_needed) *scratch_needed = need;
  if (need > 0 && (!scratch || scratch_bytes < need)) return cudaErrorInvalidValue;
  pp.scratch_used = need;

  const void *a_hi = p.A, *a_lo = p.A, *b_hi = p.B, *b_lo = p.B;
  int64_t lda = p.lda, ldb = p.ldb, sa = p.strideA, sb = p.strideB;
  int64_t lda_lo = 0, ldb_lo = 0, sa_lo = 0, sb_lo = 0;   // float32: layout of the lo arrays
  pp.pre = 0;
  if (!f32) {
    const RepackLayout r = repack_layout(p);
    if (r.a || r.b) {
      __half* ra = (__half*)scratch;
      __half* rb = (__half*)((char*)scratch + r.a_bytes);
      pp.rja = RepackJob{(const __half*)p.A, ra, r.a_rows, r.a_width, p.lda, r.a_ld, p.strideA, r.a_mat, r.a ? p.batch : 0};
      pp.rjb = RepackJob{(const __half*)p.B, rb, r.b_rows, r.b_width, p.ldb, r.b_ld, p.strideB, r.b_mat, r.b ? p.batch : 0};
      auto blocks = [&](const RepackJob& j) {
        const int64_t work = j.batch * j.rows * j.width;
        int64_t b = (work + 255) / 256;
        return (int)(b > 148 * 8 ? 148 * 8 : b);   // zero blocks for an operand that stays in place
      };
      pp.pre_blocks_a = blocks(pp.rja); pp.pre_blocks_b = blocks(pp.rjb);
      pp.pre = 1;
      if (r.a) { a_hi = a_lo = ra; lda = r.a_ld; sa = r.a_mat; }
      if (r.b) { b_hi = b_lo = rb; ldb = r.b_ld; sb = r.b_mat; }
    }
  } else {
    const SplitLayout s = split_layout(p);
    // Work area: [A lo][A copy, if needed][B lo][B copy, if needed]
    char* at = (char*)scratch;
    float* al = (float*)at; at += s.a_bytes;
    float* ah = nullptr;
    if (s.a_copy) { ah = (float*)at; at += s.a_bytes; }
    float* bl = (float*)at; at += s.b_bytes;
    float* bh = nullptr;
    if (s.b_copy) { bh = (float*)at; at += s.b_bytes; }
    auto vec_ok4 = [](const void* src, int64_t width, int64_t ld, int64_t stride, int64_t batch) {
      return (int)(width % 4 == 0 && ld % 4 == 0 && ((uintptr_t)src & 15) == 0 && (batch == 1 || stride % 4 == 0));
    };
    pp.sja = SplitJob{(const float*)p.A, ah, al, s.a_rows, s.a_width, p.lda, s.a_ld, p.strideA, s.a_mat, p.batch,
                      vec_ok4(p.A, s.a_width, p.lda, p.strideA, p.batch)};
    pp.sjb = SplitJob{(const float*)p.B, bh, bl, s.b_rows, s.b_width, p.ldb, s.b_ld, p.strideB, s.b_mat, p.batch,
                      vec_ok4(p.B, s.b_width, p.ldb, p.strideB, p.batch)};
    auto blocks = [&](const SplitJob& j) {
      const int64_t work = j.batch * j.rows * (j.vec4 ? j.width / 4 : j.width);
      int64_t b = (work + 255) / 256;
      return (int)(b > 148 * 8 ? 148 * 8 : (b < 1 ? 1 : b));
    };
    pp.pre_blocks_a = blocks(pp.sja); pp.pre_blocks_b = blocks(pp.sjb);
    pp.pre = 2;
    a_lo = al; b_lo = bl;
    lda_lo = s.a_ld; ldb_lo = s.b_ld; sa_lo = s.a_mat; sb_lo = s.b_mat;
    if (s.a_copy) { a_hi = ah; lda = s.a_ld; sa = s.a_mat; }
    if (s.b_copy) { b_hi = bh; ldb = s.b_ld; sb = s.b_mat; }
  }

  const int dbg = debug_flags();
  const int kslabs = (int)((p.K + BK - 1) / BK);
  const int shape = plan.shape;
  const int bn = (shape == SHAPE_C1_128 || shape == SHAPE_PAIR_128) ? 128 : shape == SHAPE_PAIR_64 ? 64 : 256;
  const int cta = (shape == SHAPE_C1_256 || shape == SHAPE_C1_128) ? 1 : 2;
  const int b_box = bn / cta;
  memset(pp.maps, 0, sizeof pp.maps);
  memset(&pp.outs, 0, sizeof pp.outs);
  if (!make_operand_map(&pp.maps[0], a_hi, eb, p.a_mn_major, p.M, p.K, lda, sa, p.batch, BM) ||
      !make_operand_map(&pp.maps[2], b_hi, eb, p.b_mn_major, p.N, p.K, ldb, sb, p.batch, b_box))
    return cudaErrorNotSupported;
  if (f32) {
    if (!make_operand_map(&pp.maps[1], a_lo, eb, p.a_mn_major, p.M, p.K, lda_lo, sa_lo, p.batch, BM) ||
        !make_operand_map(&pp.maps[3], b_lo, eb, p.b_mn_major, p.N, p.K, ldb_lo, sb_lo, p.batch, b_box))
      return cudaErrorNotSupported;
  } else {
    pp.maps[1] = pp.maps[0];   // float16 has no lo parts; the kernel never reads these two
    pp.maps[3] = pp.maps[2];
  }

  TcParams& tp = pp.tp;
  tp.M = p.M; tp.N = p.N;
  // Short contractions are bound by draining results, not by the MMA: they get more epilogue
  // warps (eight up to 8 slabs, sixteen up to 2: each warp's drain is a serial chain of tensor-
  // memory load, conversion, proxy fence and TMA store, and more chains in flight hide more of
  // it - measured +8 % at K = 128, nothing at K = 256, -3 % at K = 512) and fewer operand stages.
  const bool short_k = kslabs <= tun.short_k;
  const int slabs = plan.slabs;   // pipeline slots of the small float16 shapes hold two k slabs
  tp.num_k_blocks = (kslabs + slabs - 1) / slabs;
  const bool cut = plan.splits > 1;
  tp.splits = plan.splits;
  tp.kb_per_split = cut ? plan.kb_per_split : tp.num_k_blocks;
  // float32: a window bounds the number of truncating tensor-core accumulations that feed one
  // correctly rounded float32 add in the epilogue.
  const bool windowed = f32 && !(dbg & 2);
  tp.chunk_kb = windowed ? window_slabs() : tp.num_k_blocks;
  if (tp.chunk_kb > tp.num_k_blocks) tp.chunk_kb = tp.num_k_blocks;
  const bool wide = shape == SHAPE_WIDE;
  const int tile_n = wide ? 2 * bn : bn;
  tp.tile_rows = BM * cta;
  tp.tiles_m = (int)((p.M + tp.tile_rows - 1) / tp.tile_rows);
  tp.tiles_n = (int)((p.N + tile_n - 1) / tile_n);
  tp.total_tiles = (int64_t)tp.tiles_m * tp.tiles_n * p.batch * plan.splits;
  // Tile rows that share a sweep over the columns.  A wave of CTA pairs then touches g tile rows
  // of A and (pairs / g) tile columns of B; the bytes are least near g = sqrt(pairs x tile_n / tile_m):
  // 8 for 256x256 pairs, 12-16 for 256x512 (measured at 16384^3: 6.51 ms with 8, 6.35 with 16).
  tp.group_m = tun.group_m > 0 ? tun.group_m : wide ? 16 : 16 / cta;
  tp.a_mn_major = p.a_mn_major; tp.b_mn_major = p.b_mn_major;
  tp.status = status_word;
  tp.skip_input_wait = 0;
  // Where the tiles go: the result itself, or - for a cut contraction - float32 partial matrices
  // in the work area (part z of matrix m at index m * parts + z), which a second kernel sums.
  void* out_base = p.C;
  int out_bytes = eb;
  int64_t out_ld = p.ldc, out_stride = p.strideC, out_mats = p.batch;
  tp.bias = p.bias;
  if (cut) {
    const size_t off = (ops_bytes + 255) & ~(size_t)255;
    out_base = (char*)scratch + off;
    out_bytes = 4;
    out_ld = plan.ws_ld; out_stride = p.M * plan.ws_ld; out_mats = p.batch * plan.splits;
    tp.bias = nullptr;
  }
  tp.C = out_base; tp.ldc = out_ld; tp.strideC = out_stride;
  tp.vec_ok = (((uintptr_t)out_base & 15) == 0 && (out_ld * out_bytes) % 16 == 0 && (out_stride * out_bytes) % 16 == 0) ? 1 : 0;
  // Results leave through TMA stores when the result can be described to TMA (16-byte aligned
  // base and pitches); otherwise from registers.
  tp.tma_store = 0;
  tp.n_out = 1;
  if (tp.vec_ok && !(dbg & 128) && p.M < (1ll << 31) && p.N < (1ll << 31) && out_ld * out_bytes < (1ll << 40) &&
      make_output_map(&pp.outs.m[0], out_base, out_bytes, p.N, p.M, out_ld, out_stride, out_mats))
    tp.tma_store = 1;
  if (n_extra > 0) {
    // Extra destinations only exist on the TMA-store path.
    if (!tp.tma_store || cut) return cudaErrorNotSupported;
    for (int i = 0; i < n_extra; i++) {
      if (((uintptr_t)extra_out[i] & 15) != 0 ||
          !make_output_map(&pp.outs.m[1 + i], extra_out[i], eb, p.N, p.M, p.ldc, p.strideC, p.batch))
        return cudaErrorNotSupported;
    }
    tp.n_out = 1 + n_extra;
  }

  {
    auto span = [&](const void* base, int64_t rows_, int64_t ld, int64_t stride, int64_t batch, int idx) {
      const int64_t per = rows_ * ld;
      const int64_t elems = (batch - 1) * (stride > per ? stride : per) + per;
      pp.in_lo[idx] = (uintptr_t)base;
      pp.in_hi[idx] = (uintptr_t)base + (uintptr_t)(elems * eb);
    };
    span(p.A, p.a_mn_major ? p.K : p.M, p.lda, p.strideA, p.batch, 0);
    span(p.B, p.b_mn_major ? p.K : p.N, p.ldb, p.strideB, p.batch, 1);
    pp.in_lo[2] = (uintptr_t)p.bias;
    pp.in_hi[2] = p.bias ? (uintptr_t)p.bias + (uintptr_t)(p.N * eb) : 0;
    const int64_t per_c = p.M * p.ldc;
    pp.out_lo = (uintptr_t)p.C;
    pp.out_hi = (uintptr_t)p.C + (uintptr_t)(((p.batch - 1) * (p.strideC > per_c ? p.strideC : per_c) + per_c) * eb);
    pp.trackable = (pp.pre == 0 && !cut);
  }

  TcLaunchFn fn = nullptr;
  if (!f32 && cut) {
    if (shape == SHAPE_PAIR_128) fn = TcConfig<2, 128, 4, 4, false, 2, 1, 2, true>::launch;
    else if (shape == SHAPE_PAIR_64) fn = TcConfig<2, 64, 4, 4, false, 2, 1, 2, true>::launch;
    else if (shape == SHAPE_PAIR) fn = TcConfig<2, 256, 6, 4, false, 2, 1, 1, true>::launch;
    else if (shape == SHAPE_C1_128) fn = TcConfig<2, 128, 3, 4, false, 1, 1, 2, true>::launch;
    else return cudaErrorInvalidValue;
  } else if (!f32) {
    if (wide && tun.wide_epi8) fn = TcConfig<2, 256, 4, 8, false, 2, 2>::launch;
    else if (wide) fn = TcConfig<2, 256, 4, 4, false, 2, 2>::launch;
    else if (shape == SHAPE_PAIR_128) fn = TcConfig<2, 128, 4, 4, false, 2, 1, 2>::launch;
    else if (shape == SHAPE_PAIR_64) fn = TcConfig<2, 64, 4, 4, false, 2, 1, 2>::launch;
    else if (cta == 2 && short_k && kslabs <= 2) fn = TcConfig<2, 256, 4, 16, false, 2>::launch;
    else if (cta == 2 && short_k) fn = TcConfig<2, 256, 4, 8, false, 2>::launch;
    else if (cta == 2) fn = TcConfig<2, 256, 6, 4, false, 2>::launch;
    else if (bn == 256) fn = TcConfig<2, 256, 4, 4, false, 1>::launch;
    else fn = TcConfig<2, 128, 3, 4, false, 1, 1, 2>::launch;
  } else if (windowed) {
    if (shape == SHAPE_PAIR_128) fn = TcConfig<4, 128, 3, 4, true, 2>::launch;
    else if (shape == SHAPE_PAIR_64) fn = TcConfig<4, 64, 4, 4, true, 2>::launch;
    else if (cta == 2) fn = TcConfig<4, 256, 3, 8, true, 2>::launch;
    else if (bn == 256) fn = TcConfig<4, 256, 2, 8, true, 1>::launch;
    else fn = TcConfig<4, 128, 3, 4, true, 1>::launch;
  } else {
#ifdef HC_DIAGNOSTICS
    if (cta == 2) fn = TcConfig<4, 256, 3, 4, false, 2>::launch;
    else if (bn == 256) fn = TcConfig<4, 256, 2, 4, false, 1>::launch;
    else fn = TcConfig<4, 128, 3, 4, false, 1>::launch;
#else
    return cudaErrorInvalidValue;   // float32 always runs windowed in the shipped library
#endif
  }
  pp.fn = fn;
  pp.cut = cut;
  if (cut) {
    // Sum the parts in ascending order, add the bias, round once, store the result.
    ReduceJob& job = pp.job;
    job.ws = (const float*)out_base; job.C = p.C; job.bias = p.bias;
    job.M = p.M; job.N = p.N; job.ws_ld = plan.ws_ld; job.batch = p.batch; job.parts = plan.splits;
    job.ldc = p.ldc; job.strideC = p.strideC;
    const int out_align = f32 ? 15 : 7;   // four results per thread: 16 bytes of float32, 8 of float16
    job.vec_ok = (((uintptr_t)p.C & out_align) == 0 && p.ldc % 4 == 0 && p.strideC % 4 == 0) ? 1 : 0;
    const int64_t work = p.batch * p.M * (plan.ws_ld / 4);
    int64_t blocks = (work + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    pp.reduce_blocks = (int)blocks;
    pp.reduce_half = !f32;
  }
  return cudaSuccess;
}

cudaError_t issue_tc(const TcPrepared& pp, int sm_count, cudaStream_t stream, LaunchRecord* rec, bool private_stream) {
  if (rec) { *rec = LaunchRecord(); rec->kernel = HC_KERNEL_TENSOR; rec->scratch_bytes = pp.scratch_used; }
  if (pp.pre == 1) {
    int blocks_a = pp.pre_blocks_a;
    void* args[3] = {(void*)&pp.rja, (void*)&pp.rjb, (void*)&blocks_a};
    cudaError_t e = launch_elementwise((const void*)repack_f16_kernel, args, pp.pre_blocks_a + pp.pre_blocks_b, stream);
    if (e != cudaSuccess) return e;
    if (rec) rec->launches += 1;
  } else if (pp.pre == 2) {
    int blocks_a = pp.pre_blocks_a;
    void* args[3] = {(void*)&pp.sja, (void*)&pp.sjb, (void*)&blocks_a};
    cudaError_t e = launch_elementwise((const void*)split_tf32_kernel, args, pp.pre_blocks_a + pp.pre_blocks_b, stream);
    if (e != cudaSuccess) return e;
    if (rec) rec->launches += 1;
  }
  if (rec) rec->tiles = pp.tp.total_tiles;
  // May the operand loads run ahead of the wait for the previous kernel?  Only on a stream no one
  // else launches kernels on, only against a predecessor whose written range is known, and only
  // when that range and this product's operands are disjoint.  (Anything else enqueued on the
  // stream in between - copies, ordinary kernels, event waits - completes before this kernel
  // starts at all.)
  bool skip = false;
  if (private_stream && overlap_launches()) {
    std::lock_guard<std::mutex> lock(g_track_mu);
    StreamTrack* t = track_entry(stream, true);
    if (t->known && pp.trackable) {
      skip = true;
      for (int i = 0; i < 3; i++)
        if (pp.in_hi[i] > pp.in_lo[i] && pp.in_lo[i] < t->hi && t->lo < pp.in_hi[i]) skip = false;
    }
    t->known = pp.trackable;
    t->lo = pp.out_lo;
    t->hi = pp.out_hi;
    t->stamp = ++g_track_clock;
  }
  // cudaLaunchKernelEx reports this launch's own failure; the thread's sticky-less "last error"
  // may hold another library's earlier error and is not this launch's to report.
  cudaError_t ge;
  if (skip) {
    TcParams tp = pp.tp;
    tp.skip_input_wait = 1;
    ge = pp.fn(pp.maps, pp.outs, tp, sm_count, stream, rec);
  } else {
    ge = pp.fn(pp.maps, pp.outs, pp.tp, sm_count, stream, rec);
  }
  if (ge != cudaSuccess || !pp.cut) return ge;
  void* args[1] = {(void*)&pp.job};
  cudaError_t re = launch_elementwise(pp.reduce_half ? (const void*)splitk_reduce_kernel<true>
                                                     : (const void*)splitk_reduce_kernel<false>,
                                      args, pp.reduce_blocks, stream);
  if (re != cudaSuccess) return re;
  if (rec) rec->launches += 1;
  return cudaSuccess;
}

}  // namespace

cudaError_t launch_tc(const GemmProblem& p, cudaStream_t stream, unsigned int* status_word, void* scratch,
                      size_t scratch_bytes, int sm_count, LaunchRecord* rec, void* const* extra_out, int n_extra,
                      TcCache* cache, size_t* scratch_needed, bool private_stream) {
  if (scratch_needed) *scratch_needed = 0;
  if (!tc_supported(p)) return cudaErrorNotSupported;
  if (n_extra < 0 || n_extra > kMaxOut - 1 || (n_extra > 0 && !extra_out)) return cudaErrorInvalidValue;
  if (cache && kPlanCacheEnabled) {
    const TcKey key = make_key(p, scratch, status_word, extra_out, n_extra);
    TcCache::Entry* victim = &cache->e[0];
    for (auto& x : cache->e) {
      if (x.used && memcmp(&x.key, &key, sizeof key) == 0) {
        x.stamp = ++cache->clock;
        return issue_tc(x.prep, sm_count, stream, rec, private_stream);
      }
      if (!x.used ? victim->used : (victim->used && x.stamp < victim->stamp)) victim = &x;
    }
    victim->used = false;
    cudaError_t e = prepare_tc(p, status_word, scratch, scratch_bytes, sm_count, extra_out, n_extra, &victim->prep,
                               scratch_needed);
    if (e != cudaSuccess) return e;
    victim->key = key;
    victim->stamp = ++cache->clock;
    victim->used = true;
    return issue_tc(victim->prep, sm_count, stream, rec, private_stream);
  }
  TcPrepared prep;
  cudaError_t e = prepare_tc(p, status_word, scratch, scratch_bytes, sm_count, extra_out, n_extra, &prep, scratch_needed);
  if (e != cudaSuccess) return e;
  return issue_tc(prep, sm_count, stream, rec, private_stream);
}

}  // namespace hc

// The two instructions of the library that deliver to several CTAs of a cluster at once.  They
// are kept in a file of their own, included only when the library is built with
// -DHC_CLUSTER_MULTICAST (libhccuda_mc.so): that build is for hosts that run one GPU per process
// on operands in that GPU's own memory, which the host code checks for every product before it
// chooses a kernel that uses them.  A load of this kind must never read another GPU's memory.
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace hc {
namespace {

constexpr bool kClusterMulticastBuilt = true;

// Tiled TMA load of one box into the same shared-memory offset of every CTA in `cta_mask`
// (bit i = cluster rank i).  The completion bytes are counted, for each destination CTA, on the
// barrier at `bar`'s offset in the even CTA of that destination's pair (`bar` is given with the
// pair bit clear).
__device__ __forceinline__ void tma_load_3d_shared(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1,
                                                   int c2, uint16_t cta_mask) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.multicast::cluster "
      "[%0], [%1, {%3, %4, %5}], [%2], %6;"
      ::"r"(dst), "l"((unsigned long long)map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "h"(cta_mask)
      : "memory");
}

// Arrive on the barrier at `bar`'s offset in every CTA of `cta_mask` once every MMA issued so far
// by this thread is done.
__device__ __forceinline__ void tc_commit_shared(uint32_t bar, uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(cta_mask)
               : "memory");
}

}  // namespace
}  // namespace hc

// A host with no Python and no PyTorch driving several GPUs through the C ABI alone: the ranks
// are threads of this process, one context and one group per device.  Every rank computes its
// share of a batched product (Backend.batchedMatmul, Sources/Honeycrisp/Backend.swift:661-669,
// split over the batch) and of one large product (Backend.matmul, :650-658, split over columns,
// exchanged by NCCL and by the fused epilogue), and compares with the single-device result of the
// same call, bit for bit.  Uses as many devices as are visible, up to `argv[1]` (default 8);
// with one device it runs a group of one.  Prints "group conformance ok (N ranks)" and exits 0.
#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

#include "hc_cuda.h"

namespace {

std::atomic<int> failures{0};

#define CHECK(cond)                                                                 \
  do {                                                                              \
    if (!(cond)) {                                                                  \
      std::printf("FAILED rank %d %s:%d: %s (%s)\n", rank, __FILE__, __LINE__, #cond, \
                  ctx ? hc_last_error(ctx) : "");                                   \
      failures++;                                                                   \
      return;                                                                       \
    }                                                                               \
  } while (0)

// Deterministic values in [-1, 1), the same on every rank.
std::vector<float> values(size_t n, uint32_t seed) {
  std::vector<float> v(n);
  uint32_t s = seed * 2654435761u + 12345u;
  for (size_t i = 0; i < n; i++) {
    s = s * 1664525u + 1013904223u;
    v[i] = (float)((s >> 8) & 0xffff) / 32768.0f - 1.0f;
  }
  return v;
}

void* upload(hc_ctx* ctx, const std::vector<float>& v) {
  void* d = nullptr;
  if (hc_alloc(ctx, v.size() * 4, &d) != HC_OK) return nullptr;
  if (hc_h2d(ctx, d, v.data(), v.size() * 4) != HC_OK || hc_sync(ctx) != HC_OK) return nullptr;
  return d;
}

std::vector<float> download(hc_ctx* ctx, const void* d, size_t n) {
  std::vector<float> v(n);
  hc_d2h(ctx, v.data(), d, n * 4);
  hc_sync(ctx);
  return v;
}

void run_rank(int rank, int world, const unsigned char* id) {
  hc_ctx* ctx = nullptr;
  CHECK(hc_init(rank, &ctx) == HC_OK);
  hc_group* grp = nullptr;
  CHECK(hc_group_init(ctx, world, rank, world > 1 ? id : nullptr, &grp) == HC_OK);
  CHECK(hc_group_rank(grp) == rank && hc_group_world(grp) == world);

  // --- batched: 11 matrices [96,64]x[64,80] split over the ranks, gathered in place
  const int64_t cnt = 11, rows = 96, inner = 64, cols = 80;
  const std::vector<float> a = values(cnt * rows * inner, 1), b = values(cnt * inner * cols, 2);
  void *da = upload(ctx, a), *db = upload(ctx, b), *full = nullptr, *gathered = nullptr;
  CHECK(da && db);
  CHECK(hc_alloc(ctx, cnt * rows * cols * 4, &full) == HC_OK && hc_alloc(ctx, cnt * rows * cols * 4, &gathered) == HC_OK);
  CHECK(hc_batched_matmul(ctx, HC_F32, cnt, da, 0, db, 0, 0, rows, inner, cols, full) == HC_OK);
  int64_t begin = 0, count = 0;
  CHECK(hc_shard_range(cnt, world, rank, &begin, &count) == HC_OK);
  CHECK(hc_batched_matmul_sharded(grp, HC_F32, cnt, (const float*)da + begin * rows * inner, 0,
                                  (const float*)db + begin * inner * cols, 0, 0, rows, inner, cols, gathered, 1) == HC_OK);
  CHECK(download(ctx, full, cnt * rows * cols) == download(ctx, gathered, cnt * rows * cols));

  // --- one product [520,264]x[264,1096] split over columns: NCCL form, then the fused form twice
  const int64_t M = 520, K = 264, N = 1096;
  void *A = nullptr, *B = nullptr, *one = nullptr, *split = nullptr, *shared = nullptr;
  CHECK(hc_alloc(ctx, M * N * 4, &one) == HC_OK && hc_alloc(ctx, M * N * 4, &split) == HC_OK);
  CHECK(hc_group_result_alloc(grp, M * N * 4, &shared) == HC_OK);
  for (int trial = 0; trial < 2; trial++) {
    const std::vector<float> av = values(M * K, 10 + trial), bv = values(K * N, 20 + trial);
    A = upload(ctx, av); B = upload(ctx, bv);
    CHECK(A && B);
    CHECK(hc_batched_matmul_ex(ctx, HC_KERNEL_TENSOR, HC_F32, 1, A, 0, B, 0, 0, M, K, N, one) == HC_OK);
    const std::vector<float> want = download(ctx, one, M * N);
    CHECK(hc_matmul_nsplit_allgather(grp, HC_F32, A, 0, B, 0, M, K, N, split, 0) == HC_OK);
    CHECK(download(ctx, split, M * N) == want);
    CHECK(hc_matmul_nsplit_allgather(grp, HC_F32, A, 0, B, 0, M, K, N, shared, 1) == HC_OK);
    CHECK(download(ctx, shared, M * N) == want);   // read before the next trial's call overwrites it
    hc_free(ctx, A); hc_free(ctx, B);
  }
  CHECK(hc_matmul_nsplit_allgather(grp, HC_F32, da, 0, db, 0, M, K, N, split, 1) == HC_ERR_INVALID_ARGUMENT);
  CHECK(hc_check_device_status(ctx) == HC_OK);
  CHECK(hc_group_result_free(grp, shared) == HC_OK);
  hc_free(ctx, da); hc_free(ctx, db); hc_free(ctx, full); hc_free(ctx, gathered); hc_free(ctx, one); hc_free(ctx, split);
  hc_group_destroy(grp);
  hc_destroy(ctx);
}

}  // namespace

int main(int argc, char** argv) {
  int want = argc > 1 ? std::atoi(argv[1]) : 8;
  int world = 0;
  for (; world < want && world < 8; world++) {   // count the devices hc_init accepts
    hc_ctx* probe = nullptr;
    if (hc_init(world, &probe) != HC_OK) break;
    hc_destroy(probe);
  }
  if (world == 0) {
    std::printf("no usable device\n");
    return 2;
  }
  unsigned char id[HC_GROUP_ID_BYTES] = {0};
  if (world > 1 && hc_group_unique_id(id) != HC_OK) {
    std::printf("no NCCL library: running a group of one\n");
    world = 1;
  }
  std::vector<std::thread> threads;
  for (int r = 0; r < world; r++) threads.emplace_back(run_rank, r, world, id);
  for (auto& t : threads) t.join();
  if (failures.load()) return 1;
  std::printf("group conformance ok (%d ranks)\n", world);
  return 0;
}

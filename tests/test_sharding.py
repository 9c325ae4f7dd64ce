"""Host-side sharding logic on CPU: partition arithmetic, and a world_size-2 gloo run in which
the per-rank arithmetic is done by the CPU oracle (injected; the shipped default is the CUDA
backend)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from honeycrisp_b200.sharding import batchedMatmulSharded, columnBlock, matmulColumnSplit, shardBatch
from oracle import reference_cpu as ref


@pytest.mark.parametrize("n,world", [(64, 1), (64, 2), (64, 8), (7, 4), (3, 8), (0, 2)])
def test_shard_batch_covers_everything_once(n, world):
    pos = 0
    sizes = []
    for r in range(world):
        b, c = shardBatch(n, r, world)
        assert b == pos
        pos += c
        sizes.append(c)
    assert pos == n and max(sizes) - min(sizes) <= 1


@pytest.mark.parametrize("cols,world", [(16384, 8), (16384, 2), (1000, 4), (520, 8), (5, 8), (256, 1)])
def test_column_blocks_cover_and_align(cols, world):
    pos = 0
    for r in range(world):
        b, c = columnBlock(cols, r, world)
        assert b == pos and c >= 0
        if c and cols >= 8 * world:
            assert b % 8 == 0  # 16-byte aligned first element for float16
        pos += c
    assert pos == cols
    if cols % (256 * world) == 0:
        assert all(columnBlock(cols, r, world)[1] == cols // world for r in range(world))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _oracle_batched(count, a, ta, b, tb, to, rows, inner, cols, dt, out):
    res = ref.batched_matmul(count, a.numpy(), ta, b.numpy(), tb, to, rows, inner, cols, library_fast_path=False)
    out.copy_(torch.from_numpy(res))


def _oracle_colblock(a, ta, b, tb, rows, inner, cols, begin, count, dt, out):
    A, B = ref.logical_operands(1, a.numpy(), ta, b.numpy(), tb, rows, inner, cols)
    blk = np.ascontiguousarray(B[0][:, begin:begin + count])
    res = ref.matmul(np.ascontiguousarray(A[0]), False, blk, False, False, rows, inner, count, library_fast_path=False)
    out[:, begin:begin + count] = torch.from_numpy(res.reshape(rows, count))


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(5)
        # batched: 5 matrices [6,7]x[7,4]^T over 2 ranks, no collective on the data path
        a = torch.from_numpy(rng.standard_normal((5, 6, 7)).astype(np.float32))
        b = torch.from_numpy(rng.standard_normal((5, 4, 7)).astype(np.float32))
        shard, (begin, count) = batchedMatmulSharded(None, rank, world, 5, a, False, b, True, False, 6, 7, 4,
                                                     np.float32, compute=_oracle_batched)
        full = ref.batched_matmul(5, a.numpy(), False, b.numpy(), True, False, 6, 7, 4).reshape(5, -1)
        ok1 = np.array_equal(shard.numpy().reshape(count, -1), full[begin:begin + count])
        # column split of [9,11]x[11,21] with all-gather
        a2 = torch.from_numpy(rng.standard_normal((9, 11)).astype(np.float32))
        b2 = torch.from_numpy(rng.standard_normal((11, 21)).astype(np.float32))
        c = matmulColumnSplit(None, rank, world, a2, False, b2, False, 9, 11, 21, np.float32, gather=True,
                              compute=_oracle_colblock)
        full2 = ref.matmul(a2.numpy(), False, b2.numpy(), False, False, 9, 11, 21, library_fast_path=False)
        ok2 = np.array_equal(c.numpy().reshape(-1), full2)
        ret[rank] = (ok1, ok2)
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_sharding_equals_single_device_result():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert dict(ret) == {0: (True, True), 1: (True, True)}

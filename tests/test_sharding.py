"""Host-side sharding logic on CPU.

The partitions are host arithmetic inside the C library (hc_shard_range, hc_column_block), so
they are checked here without a GPU.  The world_size-2 run uses gloo ranks in which the per-rank
arithmetic is the CPU oracle's and the exchange is gloo's, laid out exactly as the library lays it
out on GPUs (blocks packed rank after rank, all-gathered, then moved into the row-major result);
it pins the claim the GPU path rests on: sharded = single-device result, bit for bit.
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from honeycrisp_b200.sharding import columnBlock, shardBatch
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


def test_bad_requests_are_rejected():
    for bad in ((4, 2, 2), (4, -1, 2), (-1, 0, 2), (4, 0, 0)):
        with pytest.raises(ValueError):
            shardBatch(*bad)
        with pytest.raises(ValueError):
            columnBlock(*bad)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(5)
        # batched: 5 matrices [6,7]x[7,4]^T over 2 ranks; each rank holds only its shard of the
        # operands; the ranges (3 and 2 matrices) are then exchanged, one broadcast per rank
        a = rng.standard_normal((5, 6, 7)).astype(np.float32)
        b = rng.standard_normal((5, 4, 7)).astype(np.float32)
        begin, count = shardBatch(5, rank, world)
        mine = ref.batched_matmul(count, a[begin:begin + count], False, b[begin:begin + count], True, False, 6, 7, 4,
                                  library_fast_path=False).reshape(count, -1)
        full = ref.batched_matmul(5, a, False, b, True, False, 6, 7, 4).reshape(5, -1)
        ok1 = np.array_equal(mine, full[begin:begin + count])
        whole = torch.zeros((5, 24))
        whole[begin:begin + count] = torch.from_numpy(mine)
        for r in range(world):
            rb, rc = shardBatch(5, r, world)
            part = whole[rb:rb + rc].contiguous()
            dist.broadcast(part, src=r)
            whole[rb:rb + rc] = part
        ok2 = np.array_equal(whole.numpy(), full)
        # column split of [9,11]x[11,21]: blocks computed on their own, packed rank after rank,
        # gathered, moved into the row-major result
        a2 = rng.standard_normal((9, 11)).astype(np.float32)
        b2 = rng.standard_normal((11, 21)).astype(np.float32)
        widths = [columnBlock(21, r, world)[1] for r in range(world)]
        begins = [columnBlock(21, r, world)[0] for r in range(world)]
        blk = np.ascontiguousarray(b2[:, begins[rank]:begins[rank] + widths[rank]])
        block = ref.matmul(a2, False, blk, False, False, 9, 11, widths[rank], library_fast_path=False)
        packed = [torch.zeros(9 * w) for w in widths]
        packed[rank] = torch.from_numpy(block.reshape(-1).copy())
        for r in range(world):
            dist.broadcast(packed[r], src=r)
        out = np.zeros((9, 21), dtype=np.float32)
        for r in range(world):
            out[:, begins[r]:begins[r] + widths[r]] = packed[r].numpy().reshape(9, widths[r])
        full2 = ref.matmul(a2, False, b2, False, False, 9, 11, 21, library_fast_path=False)
        ok3 = np.array_equal(out.reshape(-1), full2)
        ret[rank] = (ok1, ok2, ok3)
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_sharding_equals_single_device_result():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert dict(ret) == {0: (True, True, True), 1: (True, True, True)}

"""Two ranks on two GPUs (NCCL): sharded products equal the one-device product.  Skipped when
fewer than two GPUs are visible.  NVLS is switched off: nothing here needs it."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    import torch
    import torch.distributed as dist

    from honeycrisp_b200 import CUDABackend, _lib
    from honeycrisp_b200.sharding import batchedMatmulSharded, matmulColumnSplit

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        be = CUDABackend(rank)
        g = torch.Generator(device="cuda").manual_seed(2)           # same operands on every rank
        # batched Q K^T, 8 matrices over 2 ranks, no collective on the data path
        q = torch.randn((8, 512, 128), generator=g, device="cuda").half()
        k = torch.randn((8, 384, 128), generator=g, device="cuda").half()
        torch.cuda.synchronize()
        shard, (begin, count) = batchedMatmulSharded(be, rank, world, 8, q, False, k, True, False, 512, 128, 384,
                                                     np.float16)
        full = torch.empty(8 * 512 * 384, device="cuda", dtype=torch.float16)
        fd = be.wrap(full.data_ptr(), full.numel() * 2, full)
        be.batchedMatmul(8, q, False, k, True, False, 512, 128, 384, np.float16, out=fd)
        be.sync()
        ok1 = bool(torch.equal(shard.view(count, -1), full.view(8, -1)[begin:begin + count]))
        # float32 product split over columns, blocks all-gathered
        a = torch.rand((512, 256), generator=g, device="cuda") * 2 - 1
        b = torch.rand((256, 1024), generator=g, device="cuda") * 2 - 1
        torch.cuda.synchronize()
        c = matmulColumnSplit(be, rank, world, a, False, b, False, 512, 256, 1024, np.float32, gather=True)
        one = torch.empty((512, 1024), device="cuda")
        od = be.wrap(one.data_ptr(), one.numel() * 4, one)
        be.matmul(a, False, b, False, False, 512, 256, 1024, np.float32, out=od, kernel=_lib.HC_KERNEL_TENSOR)
        be.sync()
        torch.cuda.synchronize()
        ok2 = bool(torch.equal(c, one))
        # the same split with the exchange fused into the epilogue (peer stores, no collective)
        from honeycrisp_b200.sharding import FusedColumnSplit
        fused = FusedColumnSplit(be, rank, world, 512, 1024, np.float32)
        fused.matmul(a, False, b, False, 256)
        ok3 = bool(torch.equal(fused.out.asTorch((512, 1024), torch.float32), one))
        fused.close()
        ah = torch.randn((768, 320), generator=g, device="cuda").half()
        bh = torch.randn((1536, 320), generator=g, device="cuda").half()     # stored [cols, inner]
        torch.cuda.synchronize()
        oneh = torch.empty((768, 1536), device="cuda", dtype=torch.float16)
        be.matmul(ah, False, bh, True, False, 768, 320, 1536, np.float16,
                  out=be.wrap(oneh.data_ptr(), oneh.numel() * 2, oneh), kernel=_lib.HC_KERNEL_TENSOR)
        be.sync()
        fusedh = FusedColumnSplit(be, rank, world, 768, 1536, np.float16)
        fusedh.matmul(ah, False, bh, True, 320)
        ok4 = bool(torch.equal(fusedh.out.asTorch((768, 1536), torch.float16), oneh))
        fusedh.close()
        be.checkDeviceStatus()
        ret[rank] = (ok1, ok2, ok3, ok4)
        be.close()
    finally:
        dist.destroy_process_group()


def test_two_ranks_equal_one_device():
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert dict(ret) == {0: (True, True, True, True), 1: (True, True, True, True)}

"""Two ranks on two GPUs through the group entry points of the C ABI: sharded products equal the
one-device product, as processes (one per GPU) and as threads of one process.  Skipped when
fewer than two GPUs are visible.  NVLS is switched off: nothing here needs it."""
import os
import socket
import threading

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _checks(be, grp, rank, world):
    """The body both layouts share; returns a tuple of booleans."""
    import torch

    from honeycrisp_b200 import _lib

    dev = torch.device("cuda", be.device)
    g = torch.Generator(device=dev).manual_seed(2)           # same operands on every rank
    res = []
    # batched Q K^T, 9 matrices over 2 ranks (5 + 4): no exchange, then with the ranges gathered
    q = torch.randn((9, 512, 128), generator=g, device=dev).half()
    k = torch.randn((9, 384, 128), generator=g, device=dev).half()
    torch.cuda.synchronize(dev)
    begin, count = grp.shard(9)
    full = torch.empty((9, 512 * 384), device=dev, dtype=torch.float16)
    be.batchedMatmul(9, q, False, k, True, False, 512, 128, 384, np.float16, out=be.wrap(full.data_ptr(), full.numel() * 2, full))
    shard = torch.empty((count, 512 * 384), device=dev, dtype=torch.float16)
    grp.batchedMatmulSharded(9, q[begin:begin + count], False, k[begin:begin + count], True, False, 512, 128, 384,
                             np.float16, shard)
    gathered = torch.zeros((9, 512 * 384), device=dev, dtype=torch.float16)
    grp.batchedMatmulSharded(9, q[begin:begin + count], False, k[begin:begin + count], True, False, 512, 128, 384,
                             np.float16, gathered, gather=True)
    be.sync()
    res.append(bool(torch.equal(shard, full[begin:begin + count])))
    res.append(bool(torch.equal(gathered, full)))
    # float32 product split over columns: NCCL form, equal blocks and ragged blocks
    for (M, K, N) in ((512, 256, 1024), (264, 96, 328)):
        a = torch.rand((M, K), generator=g, device=dev) * 2 - 1
        b = torch.rand((K, N), generator=g, device=dev) * 2 - 1
        torch.cuda.synchronize(dev)
        one = torch.empty((M, N), device=dev)
        be.matmul(a, False, b, False, False, M, K, N, np.float32, out=be.wrap(one.data_ptr(), one.numel() * 4, one),
                  kernel=_lib.HC_KERNEL_TENSOR)
        c = torch.zeros((M, N), device=dev)
        grp.matmulColumnSplit(a, False, b, False, M, K, N, np.float32, c)
        be.sync()
        res.append(bool(torch.equal(c, one)))
    # the fused form, called twice on the same result buffer with different operands: the second
    # call may not overwrite a peer's result before that peer has read the first one
    M, K, N = 512, 256, 1024
    out = grp.resultAllocate(M * N * 4)
    view = out.asTorch((M, N), torch.float32)
    keep = torch.empty((M, N), device=dev)
    be.sync()
    shared_stream = torch.cuda.Stream(device=dev)       # a stream of the host's, lent to the backend
    be.useStream(shared_stream.cuda_stream)
    for trial in range(2):
        a = torch.rand((M, K), generator=g, device=dev) * 2 - 1
        b = torch.rand((K, N), generator=g, device=dev) * 2 - 1
        torch.cuda.synchronize(dev)
        one = torch.empty((M, N), device=dev)
        be.matmul(a, False, b, False, False, M, K, N, np.float32, out=be.wrap(one.data_ptr(), one.numel() * 4, one),
                  kernel=_lib.HC_KERNEL_TENSOR)
        grp.matmulColumnSplit(a, False, b, False, M, K, N, np.float32, out, fused=True)
        # the consumer of this result, enqueued on the stream the backend works on before the next call
        with torch.cuda.stream(shared_stream):
            keep.copy_(view)
        be.sync()
        res.append(bool(torch.equal(keep, one)))
    grp.resultFree(out)
    be.sync()
    be.useStream(None)
    # float16, transposed B, fused
    ah = torch.randn((768, 320), generator=g, device=dev).half()
    bh = torch.randn((1536, 320), generator=g, device=dev).half()     # stored [cols, inner]
    torch.cuda.synchronize(dev)
    oneh = torch.empty((768, 1536), device=dev, dtype=torch.float16)
    be.matmul(ah, False, bh, True, False, 768, 320, 1536, np.float16,
              out=be.wrap(oneh.data_ptr(), oneh.numel() * 2, oneh), kernel=_lib.HC_KERNEL_TENSOR)
    outh = grp.resultAllocate(768 * 1536 * 2)
    grp.matmulColumnSplit(ah, False, bh, True, 768, 320, 1536, np.float16, outh, fused=True)
    be.sync()
    res.append(bool(torch.equal(outh.asTorch((768, 1536), torch.float16), oneh)))
    # a result that is not a group buffer is refused for the fused form
    try:
        grp.matmulColumnSplit(ah, False, bh, True, 768, 320, 1536, np.float16, oneh, fused=True)
        res.append(False)
    except ValueError:
        res.append(True)
    grp.resultFree(outh)
    be.checkDeviceStatus()
    return tuple(res)


def _missing_peer(be, grp, rank):
    """Rank 1 stays away from a barrier (a host-made failure, between steps): rank 0's bounded wait
    runs out and reports it; nothing hangs and the context keeps working."""
    from honeycrisp_b200 import DeviceTimeout
    grp.setTimeout(200)
    if rank == 0:
        grp.barrier()
        try:
            be.checkDeviceStatus()
            return False
        except DeviceTimeout:
            pass
        x = np.ones((64, 64), dtype=np.float32)
        y = be.matmul(x, False, x, False, False, 64, 64, 64, np.float32).onCPU(np.float32)
        be.checkDeviceStatus()
        return bool(np.all(y == 64.0))
    return True


def _process_worker(rank, world, port, ret):
    import torch
    import torch.distributed as dist

    from honeycrisp_b200 import CUDABackend
    from honeycrisp_b200.sharding import DeviceGroup

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)    # a host channel for the id, nothing else
    try:
        be = CUDABackend(rank)
        grp = DeviceGroup.fromTorchDistributed(be)
        checks = _checks(be, grp, rank, world)
        dist.barrier()
        late = _missing_peer(be, grp, rank)
        ret[rank] = checks + (late,)
        dist.barrier()
        # the group's counters are out of step after the deliberate no-show: it is dropped, not reused
        be.sync()
    finally:
        dist.destroy_process_group()


def test_two_processes_equal_one_device():
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_process_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert dict(ret) == {0: (True,) * 9, 1: (True,) * 9}


def test_two_threads_of_one_process_equal_one_device():
    """One host process driving two devices: the ranks are threads, buffers are shared through
    peer access instead of IPC handles."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from honeycrisp_b200 import CUDABackend
    from honeycrisp_b200.sharding import DeviceGroup
    uid = DeviceGroup.uniqueId()
    ret, errs = {}, []

    def run(rank):
        try:
            be = CUDABackend(rank)
            grp = DeviceGroup(be, rank, 2, uid)
            ret[rank] = _checks(be, grp, rank, 2)
            grp.close()
            be.close()
        except Exception as e:  # noqa: BLE001
            errs.append((rank, repr(e)))

    threads = [threading.Thread(target=run, args=(r,)) for r in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(300)
    assert not errs, errs
    assert ret == {0: (True,) * 8, 1: (True,) * 8}

"""Splitting matrix products over the GPUs of one box: a thin layer over the group entry points
of the C ABI (`hc_group_*`, `hc_batched_matmul_sharded`, `hc_matmul_nsplit_allgather`).

The reference has no multi-device code (a `Backend` holds one device,
Sources/Honeycrisp/BackendMPS.swift:352), so the contract of everything here is "equals the
single-device result of the same call":

* `batchedMatmul` partitions over `matrixCount` - the matrices are independent
  (Sources/Honeycrisp/BackendCPU.swift:1290 loops over them), so each rank multiplies a
  contiguous range of them and nothing is exchanged unless the caller asks for it;
* one large `matmul` partitions over the columns of op(a)*op(b); each rank computes its column
  block with the tile plan of the whole product, and the blocks are exchanged either by NCCL
  (all-gather of packed blocks + one unpack kernel) or by the product kernel itself, whose
  epilogue stores every finished tile into every rank's result over NVLink.

Partitioning, the NCCL communicator, the buffers the ranks share and the barriers all live in the
library; this module converts arguments.  Everything is enqueued on the backend's stream: make
that the stream your other work uses (`backend.useStream(...)`) or call `backend.sync()` before
touching a result from elsewhere.  A host channel is needed once, to hand rank 0's 128-byte group
id to the other ranks; `DeviceGroup.fromTorchDistributed` uses a torch.distributed process group
for that and for nothing else.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

from . import _lib as L
from .backend import CUDABackend, CUDAData, DType, NotImplementedByBackend, _HC_DTYPE, _as_dtype


def shardBatch(matrixCount: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous range (begin, count) of the matrices rank `rank` of `world` multiplies.
    Ranges differ in size by at most one and cover [0, matrixCount) in rank order."""
    b, c = ctypes.c_int64(), ctypes.c_int64()
    if L.load().hc_shard_range(int(matrixCount), int(world), int(rank), ctypes.byref(b), ctypes.byref(c)) != L.HC_OK:
        raise ValueError("bad shard request")
    return b.value, c.value


def columnBlock(cols: int, rank: int, world: int) -> Tuple[int, int]:
    """Column range (begin, count) of rank `rank`.  Boundaries fall on multiples of 256 (the
    kernel's tile width, which also keeps every block's first element 16-byte aligned) as long
    as that leaves every rank a block; otherwise on multiples of 8."""
    b, c = ctypes.c_int64(), ctypes.c_int64()
    if L.load().hc_column_block(int(cols), int(world), int(rank), ctypes.byref(b), ctypes.byref(c)) != L.HC_OK:
        raise ValueError("bad column-block request")
    return b.value, c.value


def _ptr(x) -> int:
    """Device address of a CUDAData, a CUDA torch tensor or a raw integer address."""
    if isinstance(x, int):
        return x
    if isinstance(x, CUDAData):
        return x.ptr
    if hasattr(x, "data_ptr"):
        if not x.is_cuda or not x.is_contiguous():
            raise ValueError("torch operands must be contiguous CUDA tensors")
        return x.data_ptr()
    raise TypeError(f"unsupported operand type {type(x)!r}")


class DeviceGroup:
    """One rank of a group of `world` backends, one per GPU (processes, or threads of one process)."""

    def __init__(self, backend: CUDABackend, rank: int, world: int, uniqueId: Optional[bytes] = None):
        self.backend, self.rank, self.world = backend, int(rank), int(world)
        self._lib = backend._lib
        g = ctypes.c_void_p()
        if world > 1 and (uniqueId is None or len(uniqueId) != 128):
            raise ValueError("a group of more than one rank needs rank 0's 128-byte id")
        backend._check(self._lib.hc_group_init(backend._ctx, self.world, self.rank,
                                               ctypes.c_char_p(uniqueId) if uniqueId else None, ctypes.byref(g)))
        self._g = g.value

    @staticmethod
    def uniqueId() -> bytes:
        """Rank 0 calls this and sends the bytes to the other ranks over any host channel."""
        buf = ctypes.create_string_buffer(128)
        st = L.load().hc_group_unique_id(buf)
        if st != L.HC_OK:
            raise NotImplementedByBackend("no usable NCCL library: " + L.load().hc_status_string(st).decode())
        return bytes(buf.raw)

    @classmethod
    def fromTorchDistributed(cls, backend: CUDABackend, group=None) -> "DeviceGroup":
        """Rank and world size of an initialised torch.distributed group; the id travels through it."""
        import torch.distributed as dist
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        box = [cls.uniqueId() if rank == 0 and world > 1 else None]
        if world > 1:
            dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        return cls(backend, rank, world, box[0])

    # -- plumbing ----------------------------------------------------------------------------

    def close(self):
        """Collective: every rank's close meets in the communicator's teardown."""
        if getattr(self, "_g", None):
            self._lib.hc_group_destroy(self._g)
            self._g = None

    def __del__(self):
        # Not closed here: destruction is collective and must not happen at an arbitrary moment.
        pass

    def setTimeout(self, milliseconds: int):
        self.backend._check(self._lib.hc_group_set_timeout_ms(self._g, int(milliseconds)))

    def barrier(self):
        """Enqueue a flag barrier on the backend's stream (returns without waiting)."""
        self.backend._check(self._lib.hc_group_barrier(self._g))

    def selftestMissingPeer(self, limit_ms: int = 50):
        self.backend._check(self._lib.hc_group_selftest_missing_peer(self._g, int(limit_ms)))

    def resultAllocate(self, byteCount: int) -> CUDAData:
        """Collective: a result buffer on every rank that the other ranks can store into."""
        ptr = ctypes.c_void_p()
        self.backend._check(self._lib.hc_group_result_alloc(self._g, int(byteCount), ctypes.byref(ptr)))
        d = CUDAData(self.backend, ptr.value, int(byteCount), owns=False)
        d._kind = "group"
        d._group = self
        return d

    def resultFree(self, data: CUDAData):
        """Collective."""
        if data.ptr and self._g:
            self.backend._check(self._lib.hc_group_result_free(self._g, data.ptr))
        data.ptr = 0

    # -- the products ------------------------------------------------------------------------

    def shard(self, matrixCount: int) -> Tuple[int, int]:
        return shardBatch(matrixCount, self.rank, self.world)

    def batchedMatmulSharded(self, matrixCount: int, aShard, transA: bool, bShard, transB: bool, transOut: bool,
                             rows: int, inner: int, cols: int, dtype, out, gather: bool = False):
        """This rank's share of `batchedMatmul` over `matrixCount` matrices.  `aShard`/`bShard`
        hold the matrices of `self.shard(matrixCount)`.  Without `gather`, `out` receives those
        matrices' results and nothing is exchanged; with it, `out` is the whole batch's result
        buffer on every rank and the ranges are all-gathered in place (collective)."""
        dt = dtype if isinstance(dtype, DType) else _as_dtype(dtype)
        st = self._lib.hc_batched_matmul_sharded(self._g, _HC_DTYPE[dt], matrixCount, _ptr(aShard), 1 if transA else 0,
                                                 _ptr(bShard), 1 if transB else 0, 1 if transOut else 0, rows, inner,
                                                 cols, _ptr(out), 1 if gather else 0)
        if st != L.HC_OK:
            self.backend._check(st)
        return out

    def matmulColumnSplit(self, a, transA: bool, b, transB: bool, rows: int, inner: int, cols: int, dtype, out,
                          fused: bool = False):
        """op(a)*op(b) with the columns split over the ranks; collective.  Every rank holds all of
        `a` and `b` and ends with the complete [rows, cols] product in `out`.  `fused` moves the
        exchange into the product kernel's epilogue (peer stores); `out` must then come from
        `resultAllocate`."""
        dt = dtype if isinstance(dtype, DType) else _as_dtype(dtype)
        st = self._lib.hc_matmul_nsplit_allgather(self._g, _HC_DTYPE[dt], _ptr(a), 1 if transA else 0, _ptr(b),
                                                  1 if transB else 0, rows, inner, cols, _ptr(out), 1 if fused else 0)
        if st != L.HC_OK:
            self.backend._check(st)
        return out

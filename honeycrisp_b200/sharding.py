"""Splitting matrix products over the GPUs of one box: one process per GPU.

The reference has no multi-device code (a `Backend` holds one device,
Sources/Honeycrisp/BackendMPS.swift:352), so the contract of everything here is "equals the
single-device result of the same call":

* `batchedMatmul` partitions over `matrixCount` - the matrices are independent
  (Sources/Honeycrisp/BackendCPU.swift:1290 loops over them), so each rank multiplies a
  contiguous range of them and nothing is exchanged;
* one large `matmul` partitions over the columns of op(a)*op(b); each rank computes its column
  block with the same tile decomposition of the contraction as the full product, and the
  blocks are exchanged with one all-gather (NCCL through torch.distributed) only when the
  caller wants the whole result on every device.

torch supplies device memory and the process group; the arithmetic is libhccuda's.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

from .backend import CUDABackend, DType, _as_dtype


def shardBatch(matrixCount: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous range (begin, count) of the matrices rank `rank` of `world` multiplies.
    Ranges differ in size by at most one and cover [0, matrixCount) in rank order."""
    if world < 1 or not (0 <= rank < world) or matrixCount < 0:
        raise ValueError("bad shard request")
    base, extra = divmod(matrixCount, world)
    begin = rank * base + min(rank, extra)
    return begin, base + (1 if rank < extra else 0)


def columnBlock(cols: int, rank: int, world: int, align: int = 256) -> Tuple[int, int]:
    """Column range (begin, count) of rank `rank`.  Boundaries fall on multiples of `align`
    (the kernel's tile width, which also keeps every block's first element 16-byte aligned
    for TMA) as long as that leaves every rank a block; otherwise on multiples of 8."""
    if world < 1 or not (0 <= rank < world) or cols < 0:
        raise ValueError("bad column-block request")
    for unit in (align, 8, 1):
        units = -(-cols // unit)
        if units >= world or unit == 1:
            b, c = shardBatch(units, rank, world)
            begin = min(b * unit, cols)
            end = min((b + c) * unit, cols)
            return begin, end - begin
    raise AssertionError


def batchedMatmulSharded(backend: Optional[CUDABackend], rank: int, world: int, matrixCount: int,
                         a: torch.Tensor, transA: bool, b: torch.Tensor, transB: bool, transOut: bool,
                         rows: int, inner: int, cols: int, dtype, out: Optional[torch.Tensor] = None,
                         compute: Optional[Callable] = None) -> Tuple[torch.Tensor, Tuple[int, int]]:
    """This rank's share of a batched product.  `a`, `b` hold ALL matrices (or at least this
    rank's range at its global position); the result holds only this rank's matrices.
    No collective.  Returns (out_shard, (begin, count))."""
    dt = _as_dtype(dtype)
    begin, count = shardBatch(matrixCount, rank, world)
    a3 = a.reshape(matrixCount, -1)
    b3 = b.reshape(matrixCount, -1)
    a_sh = a3[begin:begin + count]
    b_sh = b3[begin:begin + count]
    if out is None:
        out = torch.empty(count * rows * cols, dtype=a.dtype, device=a.device)
    if count:
        if compute is not None:
            compute(count, a_sh, transA, b_sh, transB, transOut, rows, inner, cols, dt, out)
        else:
            od = backend.wrap(out.data_ptr(), out.numel() * out.element_size(), out)
            backend.batchedMatmul(count, a_sh, transA, b_sh, transB, transOut, rows, inner, cols, dt, out=od,
                                  mark=False)
    return out, (begin, count)


def matmulColumnSplit(backend: Optional[CUDABackend], rank: int, world: int, a: torch.Tensor, transA: bool,
                      b: torch.Tensor, transB: bool, rows: int, inner: int, cols: int, dtype,
                      gather: bool = True, group=None, compute: Optional[Callable] = None) -> torch.Tensor:
    """op(a)*op(b) with the columns split over `world` ranks; every rank holds all of `a` and
    `b` (only its column block of `b` is read).

    Each rank writes its block in place into a full-size row-major result.  With `gather`, the
    blocks are then exchanged: packed to a contiguous [rows, block] buffer, all-gathered, and
    unpacked, so that every rank ends with the complete product.  Returns the [rows, cols]
    result (complete if `gather`, otherwise valid only in this rank's columns).
    """
    dt = _as_dtype(dtype)
    out = torch.empty((rows, cols), dtype=a.dtype, device=a.device)
    begin, count = columnBlock(cols, rank, world)
    if count:
        if compute is not None:
            compute(a, transA, b, transB, rows, inner, cols, begin, count, dt, out)
        else:
            od = backend.wrap(out.data_ptr(), out.numel() * out.element_size(), out)
            backend.matmulColumnBlock(a, transA, b, transB, False, rows, inner, cols, begin, count, dt, out=od)
    if not gather or world == 1:
        return out
    if backend is not None:
        # The product was enqueued on the backend's stream; the collective runs on torch's.
        backend.sync()
    widths = [columnBlock(cols, r, world)[1] for r in range(world)]
    wmax = max(widths)
    send = torch.zeros((rows, wmax), dtype=a.dtype, device=a.device)
    send[:, :count] = out[:, begin:begin + count]
    recv_flat = torch.empty((world * rows, wmax), dtype=a.dtype, device=a.device)
    dist.all_gather_into_tensor(recv_flat, send, group=group)
    recv = recv_flat.view(world, rows, wmax)
    for r in range(world):
        if r == rank or widths[r] == 0:
            continue
        rb = columnBlock(cols, r, world)[0]
        out[:, rb:rb + widths[r]] = recv[r, :, :widths[r]]
    return out


class FusedColumnSplit:
    """A product split over columns whose exchange is fused into the kernel's epilogue.

    Every rank owns a full-size result buffer that the other ranks map (CUDA IPC).  Each rank
    computes its column block and its epilogue stores every finished tile into all `world`
    buffers (peer stores over NVLink), so after the ranks have synchronised and passed a
    barrier each of them holds the complete product - there is no all-gather, no packing, and
    the transfer overlaps the remaining tiles' arithmetic.  Set up once per shape, reuse per call.
    """

    def __init__(self, backend: CUDABackend, rank: int, world: int, rows: int, cols: int, dtype, group=None):
        self.backend, self.rank, self.world, self.group = backend, rank, world, group
        self.rows, self.cols, self.dtype = rows, cols, _as_dtype(dtype)
        nbytes = rows * cols * self.dtype.byteSize
        self.out = backend.sharedAllocate(nbytes)
        handle = backend.ipcExport(self.out)
        handles = [None] * world
        if world > 1:
            dist.all_gather_object(handles, handle, group=group)
        self.peers = [backend.ipcOpen(h, nbytes) for r, h in enumerate(handles) if r != rank and h is not None]

    def matmul(self, a, transA: bool, b, transB: bool, inner: int, wait: bool = True):
        """Enqueue this rank's block (and its pushes).  With `wait`, also synchronise and pass
        the group barrier, after which `self.out` holds the complete product on every rank."""
        begin, count = columnBlock(self.cols, self.rank, self.world)
        if count:
            self.backend.matmulColumnBlockPush(a, transA, b, transB, False, self.rows, inner, self.cols, begin,
                                               count, self.dtype, self.out, self.peers)
        if wait:
            self.finish()
        return self.out

    def finish(self):
        self.backend.sync()
        if self.world > 1:
            dist.barrier(group=self.group)

    def close(self):
        self.backend.sync()
        if self.world > 1:
            dist.barrier(group=self.group)   # nobody unmaps while a peer may still be storing
        for p in self.peers:
            p.free()
        self.peers = []
        if self.world > 1:
            dist.barrier(group=self.group)   # nobody frees while a peer still has it mapped
        self.out.free()

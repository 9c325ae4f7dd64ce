"""Host-side mirror of the part of Honeycrisp's `Backend` interface that libhccuda serves.

The reference's host language is Swift, for which this image has no toolchain; this module is
the same surface in Python over the same C ABI, so the tests can read like the reference's own
(Sources/HCTestUtils/BackendTests.swift:684-783).  Names and argument meaning follow

* `Backend.matmul(a:transA:b:transB:transOut:rows:inner:cols:dtype:)`
  (Sources/Honeycrisp/Backend.swift:650-658),
* `Backend.batchedMatmul(matrixCount:a:transA:b:transB:transOut:rows:inner:cols:dtype:)`
  (Backend.swift:661-669),
* `Tensor.Data` (Sources/Honeycrisp/Tensor.swift:69-85): `byteCount`, `wait()`, `onCPU`,
* `BackendError` (Backend.swift:6-16): allocationFailed / kernelFailed / notImplemented.

Everything is computed by the CUDA library; nothing here has a CPU path.
"""
from __future__ import annotations

import ctypes
import enum
from typing import Optional

import numpy as np

from . import _lib as L


class BackendError(Exception):
    """Base of the errors a backend call can throw (Backend.swift:6-16)."""


class AllocationFailed(BackendError):
    pass


class KernelFailed(BackendError):
    pass


class NotImplementedByBackend(BackendError):
    pass


class DeviceTimeout(KernelFailed):
    """A bounded device-side wait expired; the context is still usable."""


class DType(enum.Enum):
    float16 = "float16"
    float32 = "float32"
    int64 = "int64"  # legal in the reference's CPU backend; this backend throws notImplemented

    @property
    def byteSize(self) -> int:
        return {"float16": 2, "float32": 4, "int64": 8}[self.value]

    @property
    def numpy(self):
        return {"float16": np.float16, "float32": np.float32, "int64": np.int64}[self.value]


_DTYPE_OF = {}


def _as_dtype(dtype) -> DType:
    if isinstance(dtype, DType):
        return dtype
    try:
        return _DTYPE_OF[dtype]
    except (KeyError, TypeError):
        pass
    dt = DType(np.dtype(dtype).name)
    try:
        _DTYPE_OF[dtype] = dt
    except TypeError:
        pass
    return dt


_HC_DTYPE = {DType.float16: L.HC_F16, DType.float32: L.HC_F32}


class ReadBack:
    """An asynchronous device-to-host copy in flight (CUDAData.readInto)."""

    def __init__(self, source: "CUDAData", host_array: np.ndarray, event: int):
        self._source, self.array, self._event = source, host_array, event   # keeps the source alive

    def wait(self) -> np.ndarray:
        if self._event:
            lib = self._source.backend._lib
            st = lib.hc_event_wait(self._event)
            lib.hc_event_destroy(self._event)
            self._event = None
            self._source.backend._check(st)
        return self.array

    def __del__(self):
        try:
            if self._event:
                self._source.backend._lib.hc_event_destroy(self._event)
        except Exception:
            pass


class Marker:
    """A completion marker on the backend's stream (hc_event_record): wait for it, or measure the
    device time between two of them."""

    def __init__(self, backend: "CUDABackend"):
        self.backend = backend
        ev = ctypes.c_void_p()
        backend._check(backend._lib.hc_event_record(backend._ctx, ctypes.byref(ev)))
        self._event = ev.value

    def wait(self):
        self.backend._check(self.backend._lib.hc_event_wait(self._event))

    def elapsedMs(self, later: "Marker") -> float:
        """Milliseconds from this marker to `later` (both must have completed)."""
        ms = ctypes.c_float()
        self.backend._check(self.backend._lib.hc_event_elapsed_ms(self._event, later._event, ctypes.byref(ms)))
        return float(ms.value)

    def __del__(self):
        try:
            if self._event:
                self.backend._lib.hc_event_destroy(self._event)
                self._event = None
        except Exception:
            pass


class Upload(ReadBack):
    """An asynchronous host-to-device copy in flight (CUDAData.writeFrom)."""


class CUDAData:
    """Device buffer handle: the `Tensor.Data` of this backend.

    Either owns stream-ordered memory from the library's allocator, or borrows a device
    pointer (for example a torch tensor's) and keeps `owner` alive for as long as it lives.
    """

    def __init__(self, backend: "CUDABackend", ptr: int, byteCount: int, owns: bool, owner=None):
        self.backend = backend
        self.ptr = int(ptr) if ptr else 0
        self.byteCount = int(byteCount)
        self._owns = owns
        self._owner = owner
        self._event: Optional[int] = None

    def _mark(self):
        """Record a completion marker after the work that produces this buffer."""
        lib = self.backend._lib
        if self._event:
            lib.hc_event_destroy(self._event)
            self._event = None
        ev = ctypes.c_void_p()
        self.backend._check(lib.hc_event_record(self.backend._ctx, ctypes.byref(ev)))
        self._event = ev.value

    def wait(self) -> None:
        """Tensor.Data.wait(): block until the buffer's producer has run; rethrow its failure."""
        if not self.backend._ctx:
            raise KernelFailed("wait() on a buffer whose backend has been closed")
        if self._event:
            self.backend._check(self.backend._lib.hc_event_wait(self._event))
        else:
            self.backend.sync()

    def onCPU(self, dtype=np.uint8) -> np.ndarray:
        """Tensor.Data.onCPU: the buffer's bytes on the host, viewed as `dtype`."""
        out = np.empty(self.byteCount, dtype=np.uint8)
        if self.byteCount:
            lib = self.backend._lib
            self.backend._check(lib.hc_d2h(self.backend._ctx, out.ctypes.data, self.ptr, self.byteCount))
        self.backend.sync()
        if self._event:
            self.backend._check(self.backend._lib.hc_event_wait(self._event))
        return out.view(dtype)

    def writeFrom(self, host_array: np.ndarray) -> "Upload":
        """Start copying `host_array` (pinned memory for a true DMA) into this buffer on a side
        stream, after the work enqueued so far.  Work that reads the buffer must be ordered
        behind the copy with backend.enqueueWait(upload) - or upload.wait() on the host."""
        if not host_array.flags["C_CONTIGUOUS"] or host_array.nbytes > self.byteCount:
            raise ValueError("writeFrom: need a contiguous host array no larger than the buffer")
        ev = ctypes.c_void_p()
        self.backend._check(self.backend._lib.hc_h2d_async(self.backend._ctx, self.ptr, host_array.ctypes.data,
                                                  host_array.nbytes, ctypes.byref(ev)))
        return Upload(self, host_array, ev.value)

    def readInto(self, host_array: np.ndarray) -> "ReadBack":
        """Start copying this buffer into `host_array` (pinned memory for a true DMA) on a side
        stream, ordered after the work enqueued so far; later products keep running.  The
        returned handle's wait() blocks until the bytes have arrived."""
        if not host_array.flags["C_CONTIGUOUS"] or host_array.nbytes > self.byteCount:
            raise ValueError("readInto: need a contiguous host array no larger than the buffer")
        ev = ctypes.c_void_p()
        self.backend._check(self.backend._lib.hc_d2h_async(self.backend._ctx, host_array.ctypes.data, self.ptr,
                                                  host_array.nbytes, ctypes.byref(ev)))
        return ReadBack(self, host_array, ev.value)

    def asTorch(self, shape, torch_dtype):
        """The buffer as a torch tensor that aliases it (no copy); the tensor keeps this handle alive."""
        import torch
        typestr = {torch.float16: "<f2", torch.float32: "<f4"}[torch_dtype]

        class _View:
            pass

        v = _View()
        v.__cuda_array_interface__ = {"shape": tuple(int(x) for x in shape), "typestr": typestr,
                                      "data": (self.ptr, False), "version": 3}
        v._keep = self
        t = torch.as_tensor(v, device=torch.device("cuda", self.backend.device))
        t._hc_owner = self
        return t

    def free(self) -> None:
        if self._event:
            self.backend._lib.hc_event_destroy(self._event)
            self._event = None
        if self.ptr and self.backend._ctx:
            kind = getattr(self, "_kind", None)
            if kind == "shared":
                self.backend._lib.hc_shared_free(self.backend._ctx, self.ptr)
            elif kind == "ipc":
                self.backend._lib.hc_ipc_close(self.backend._ctx, self.ptr)
            elif self._owns:
                self.backend._lib.hc_free(self.backend._ctx, self.ptr)
        self.ptr = 0
        self._owner = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class CUDABackend:
    """`Backend` subclass counterpart: one CUDA device, one stream, matmul and batchedMatmul.

    Methods of `Backend` outside the matrix-product path are not provided; asking for them
    raises NotImplementedByBackend, the reference's convention for partial backends
    (Backend.swift: every primitive defaults to `throw BackendError.notImplemented`).
    """

    def __init__(self, device: int = 0, diagnostics: bool = False):
        """`diagnostics` binds the context to the diagnostics build of the library (planner choices
        forced through HC_TC_* environment variables); the test-suite's use only."""
        lib = self._lib = L.load(diagnostics)
        ctx = ctypes.c_void_p()
        st = lib.hc_init(int(device), ctypes.byref(ctx))
        if st != L.HC_OK:
            raise KernelFailed(f"hc_init(device={device}) failed: {lib.hc_status_string(st).decode()}")
        self._ctx = ctx.value
        self.device = int(device)

    # -- plumbing ------------------------------------------------------------------------

    def close(self):
        if getattr(self, "_ctx", None):
            self._lib.hc_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, status: int):
        if status == L.HC_OK:
            return
        lib = self._lib
        msg = lib.hc_last_error(self._ctx).decode() or lib.hc_status_string(status).decode()
        if status == L.HC_ERR_ALLOCATION_FAILED:
            raise AllocationFailed(msg)
        if status == L.HC_ERR_NOT_IMPLEMENTED:
            raise NotImplementedByBackend(msg)
        if status == L.HC_ERR_TIMEOUT:
            raise DeviceTimeout(msg)
        if status == L.HC_ERR_INVALID_ARGUMENT:
            # The reference traps these with #alwaysAssert before the backend is reached.
            raise ValueError(msg)
        raise KernelFailed(msg)

    def useStream(self, cuda_stream_ptr: Optional[int]):
        """Enqueue this backend's work on a stream owned by the caller (None: its own)."""
        self._check(self._lib.hc_set_stream(self._ctx, cuda_stream_ptr or None))

    def enqueueWait(self, transfer: "ReadBack"):
        """Work enqueued after this call starts only when `transfer` (an Upload or ReadBack) has
        completed; the host does not block."""
        if transfer._event:
            self._check(self._lib.hc_enqueue_wait(self._ctx, transfer._event))

    def sync(self):
        self._check(self._lib.hc_sync(self._ctx))

    def marker(self) -> Marker:
        """Record a completion marker after everything enqueued so far."""
        return Marker(self)

    def stream(self) -> int:
        """The CUDA stream (a `cudaStream_t` as an integer) this backend enqueues on."""
        return int(self._lib.hc_get_stream(self._ctx) or 0)

    def checkDeviceStatus(self):
        self._check(self._lib.hc_check_device_status(self._ctx))

    def launchCount(self) -> int:
        return int(self._lib.hc_launch_count(self._ctx))

    def lastLaunchInfo(self) -> dict:
        info = L.LaunchInfo()
        self._check(self._lib.hc_last_launch_info(self._ctx, ctypes.byref(info)))
        return {name: getattr(info, name) for name, _ in L.LaunchInfo._fields_}

    # -- buffers -------------------------------------------------------------------------

    def allocate(self, byteCount: int) -> CUDAData:
        ptr = ctypes.c_void_p()
        self._check(self._lib.hc_alloc(self._ctx, int(byteCount), ctypes.byref(ptr)))
        return CUDAData(self, ptr.value, int(byteCount), owns=True)

    def collection(self, values, dtype) -> CUDAData:
        """Backend.collection (Backend.swift:794-800): host values -> device buffer."""
        dt = _as_dtype(dtype)
        arr = np.ascontiguousarray(np.asarray(values).astype(dt.numpy, copy=False)).reshape(-1)
        data = self.allocate(arr.nbytes)
        if arr.nbytes:
            self._check(self._lib.hc_h2d(self._ctx, data.ptr, arr.ctypes.data, arr.nbytes))
            self.sync()  # the host array may be a temporary
        return data

    def sharedAllocate(self, byteCount: int) -> CUDAData:
        """Memory that the other processes of the box (one per GPU) can map with ipcOpen."""
        ptr = ctypes.c_void_p()
        self._check(self._lib.hc_shared_alloc(self._ctx, int(byteCount), ctypes.byref(ptr)))
        d = CUDAData(self, ptr.value, int(byteCount), owns=False)
        d._kind = "shared"
        return d

    def ipcExport(self, data: CUDAData) -> bytes:
        """Opaque 64-byte handle of a sharedAllocate buffer, to send to the other processes."""
        buf = ctypes.create_string_buffer(64)
        self._check(self._lib.hc_ipc_export(self._ctx, data.ptr, buf))
        return bytes(buf.raw)

    def ipcOpen(self, handle: bytes, byteCount: int) -> CUDAData:
        """Map another process's sharedAllocate buffer into this one (peer access over NVLink)."""
        ptr = ctypes.c_void_p()
        self._check(self._lib.hc_ipc_open(self._ctx, ctypes.c_char_p(handle), ctypes.byref(ptr)))
        d = CUDAData(self, ptr.value, int(byteCount), owns=False)
        d._kind = "ipc"
        return d

    def matmulColumnBlockPush(self, a, transA: bool, b, transB: bool, transOut: bool, rows: int, inner: int,
                              cols: int, colBegin: int, colCount: int, dtype, out: CUDAData, peerOuts) -> CUDAData:
        """matmulColumnBlock whose epilogue also stores every tile into the peers' results."""
        dt = _as_dtype(dtype)
        if dt not in _HC_DTYPE:
            raise NotImplementedByBackend(f"matmul for dtype {dt.value}")
        a_d = self._device_operand(a, dt)
        b_d = self._device_operand(b, dt)
        need = rows * cols * dt.byteSize
        if out.byteCount < need or any(p.byteCount < need for p in peerOuts):
            raise ValueError("matmulColumnBlockPush: every result must be the full rows x cols buffer")
        arr = (ctypes.c_void_p * max(1, len(peerOuts)))(*[p.ptr for p in peerOuts])
        st = self._lib.hc_matmul_colblock_push(self._ctx, _HC_DTYPE[dt], a_d.ptr, int(bool(transA)), b_d.ptr,
                                              int(bool(transB)), int(bool(transOut)), int(rows), int(inner),
                                              int(cols), int(colBegin), int(colCount), out.ptr, arr, len(peerOuts))
        self._check(st)
        out._mark()
        out._inputs = (a_d, b_d)
        return out

    def wrap(self, device_ptr: int, byteCount: int, owner=None) -> CUDAData:
        """Borrow device memory allocated elsewhere (e.g. `t.data_ptr()` of a CUDA torch tensor)."""
        return CUDAData(self, device_ptr, byteCount, owns=False, owner=owner)

    def _device_operand(self, x, dt: DType):
        """Operands of a foreign Data type are staged to the device, as the reference's GPU
        backend does through onCPU (Sources/Honeycrisp/BackendMPS.swift:585-620)."""
        if isinstance(x, CUDAData):
            return x
        if isinstance(x, np.ndarray):
            return self.collection(x, dt)
        if hasattr(x, "data_ptr") and hasattr(x, "element_size"):  # a CUDA torch tensor
            if not x.is_cuda or not x.is_contiguous():
                raise ValueError("torch operands must be contiguous CUDA tensors")
            return self.wrap(x.data_ptr(), x.numel() * x.element_size(), owner=x)
        raise TypeError(f"unsupported operand type {type(x)!r}")

    def _operand(self, x, dt: DType):
        """(device address, bytes, object to keep alive) of an operand, without building a handle
        for device memory that already has an owner: the per-call cost matters for products that
        run for a few microseconds."""
        if isinstance(x, CUDAData):
            return x.ptr, x.byteCount, x
        if hasattr(x, "data_ptr"):  # a CUDA torch tensor
            if not x.is_cuda or not x.is_contiguous():
                raise ValueError("torch operands must be contiguous CUDA tensors")
            return x.data_ptr(), x.numel() * x.element_size(), x
        d = self._device_operand(x, dt)
        return d.ptr, d.byteCount, d

    # -- the hot path --------------------------------------------------------------------

    def matmul(self, a, transA: bool, b, transB: bool, transOut: bool, rows: int, inner: int, cols: int,
               dtype, kernel: int = L.HC_KERNEL_AUTO, out: Optional[CUDAData] = None, mark: bool = True) -> CUDAData:
        """`transOut(op(a) * op(b))`; rows x cols is the shape of op(a)*op(b) (Backend.swift:650-658)."""
        return self.batchedMatmul(1, a, transA, b, transB, transOut, rows, inner, cols, dtype, kernel=kernel,
                                  out=out, mark=mark)

    def batchedMatmul(self, matrixCount: int, a, transA: bool, b, transB: bool, transOut: bool, rows: int,
                      inner: int, cols: int, dtype, kernel: int = L.HC_KERNEL_AUTO,
                      out: Optional[CUDAData] = None, mark: bool = True) -> CUDAData:
        """matrixCount independent products, operands packed back to back (Backend.swift:661-669).

        `mark=False` skips the per-result completion marker (wait() then synchronises the whole
        stream instead); launch-bound loops and CUDA-graph capture use it."""
        dt = _as_dtype(dtype)
        hdt = _HC_DTYPE.get(dt)
        if hdt is None:
            raise NotImplementedByBackend(f"matmul for dtype {dt.value}")
        a_p, a_n, a_keep = self._operand(a, dt)
        b_p, b_n, b_keep = self._operand(b, dt)
        eb = 2 if hdt == L.HC_F16 else 4
        n_out = matrixCount * rows * cols * eb
        # Same size checks the reference's GPU backend makes before encoding
        # (Sources/Honeycrisp/BackendMPS.swift:2221-2230).
        if a_n < matrixCount * rows * inner * eb:
            raise ValueError("matmul: operand a is smaller than matrixCount*rows*inner elements")
        if b_n < matrixCount * inner * cols * eb:
            raise ValueError("matmul: operand b is smaller than matrixCount*inner*cols elements")
        if out is None:
            out = self.allocate(n_out)
        elif out.byteCount < n_out:
            raise ValueError("matmul: output buffer too small")
        st = self._lib.hc_batched_matmul_ex(self._ctx, kernel, hdt, matrixCount, a_p, 1 if transA else 0, b_p,
                                            1 if transB else 0, 1 if transOut else 0, rows, inner, cols, out.ptr)
        if st != L.HC_OK:
            self._check(st)
        if mark:
            out._mark()
        out._inputs = (a_keep, b_keep)  # keep operands alive until the result is collected
        return out

    def matmulColumnBlock(self, a, transA: bool, b, transB: bool, transOut: bool, rows: int, inner: int,
                          cols: int, colBegin: int, colCount: int, dtype, out: CUDAData,
                          kernel: int = L.HC_KERNEL_AUTO) -> CUDAData:
        """Columns [colBegin, colBegin+colCount) of op(a)*op(b), written in place into the
        full-size `out`.  One device's share of a product split over devices."""
        dt = _as_dtype(dtype)
        if dt not in _HC_DTYPE:
            raise NotImplementedByBackend(f"matmul for dtype {dt.value}")
        a_d = self._device_operand(a, dt)
        b_d = self._device_operand(b, dt)
        if out.byteCount < rows * cols * dt.byteSize:
            raise ValueError("matmulColumnBlock: output must be the full rows x cols buffer")
        st = self._lib.hc_matmul_colblock(self._ctx, int(kernel), _HC_DTYPE[dt], a_d.ptr, int(bool(transA)), b_d.ptr,
                                         int(bool(transB)), int(bool(transOut)), int(rows), int(inner), int(cols),
                                         int(colBegin), int(colCount), out.ptr)
        self._check(st)
        out._mark()
        out._inputs = (a_d, b_d)
        return out

    def batchedMatmulHost(self, matrixCount: int, a: np.ndarray, transA: bool, b: np.ndarray, transB: bool,
                          transOut: bool, rows: int, inner: int, cols: int, dtype,
                          out: Optional[np.ndarray] = None, asynchronous: bool = False) -> np.ndarray:
        """Host arrays in, host array out: stage, multiply, read back, in one library call.

        With `asynchronous`, the call only enqueues (copy-in, product and copy-out overlap with
        the neighbouring calls' stages); `out` is valid after hostSync()."""
        dt = _as_dtype(dtype)
        if dt not in _HC_DTYPE:
            raise NotImplementedByBackend(f"matmul for dtype {dt.value}")
        if a.dtype != dt.numpy or b.dtype != dt.numpy or not a.flags.c_contiguous or not b.flags.c_contiguous:
            raise ValueError("host operands must be contiguous arrays of the stated dtype")
        if a.size < matrixCount * rows * inner or b.size < matrixCount * inner * cols:
            raise ValueError("host operand smaller than its stated shape")
        if out is None:
            out = np.empty(matrixCount * rows * cols, dtype=dt.numpy)
        elif out.dtype != dt.numpy or out.size < matrixCount * rows * cols or not out.flags.c_contiguous:
            raise ValueError("bad host output array")
        fn = self._lib.hc_batched_matmul_host_async if asynchronous else self._lib.hc_batched_matmul_host
        st = fn(self._ctx, _HC_DTYPE[dt], int(matrixCount), a.ctypes.data, int(bool(transA)), b.ctypes.data,
                int(bool(transB)), int(bool(transOut)), int(rows), int(inner), int(cols), out.ctypes.data)
        self._check(st)
        return out

    # -- around a Linear layer ---------------------------------------------------------------

    def linearForward(self, x, weight, bias, rows: int, inCount: int, outCount: int, dtype,
                      out: Optional[CUDAData] = None) -> CUDAData:
        """x[rows,in] * weight[in,out] + bias[out] with the add fused into the product's epilogue
        (Linear.callAsFunction, Trainable.swift:530-546).  `bias` may be None."""
        dt = _as_dtype(dtype)
        if dt not in _HC_DTYPE:
            raise NotImplementedByBackend(f"linear for dtype {dt.value}")
        x_d, w_d = self._device_operand(x, dt), self._device_operand(weight, dt)
        b_d = self._device_operand(bias, dt) if bias is not None else None
        if out is None:
            out = self.allocate(rows * outCount * dt.byteSize)
        self._check(self._lib.hc_linear_forward(self._ctx, _HC_DTYPE[dt], x_d.ptr, w_d.ptr, b_d.ptr if b_d else None,
                                               int(rows), int(inCount), int(outCount), out.ptr))
        out._mark()
        out._inputs = (x_d, w_d, b_d)
        return out

    def columnSum(self, x, rows: int, cols: int, dtype) -> CUDAData:
        """Sum over the rows of x[rows,cols] (reduce(.sum) over the leading axis, Backend.swift:524-531)."""
        dt = _as_dtype(dtype)
        x_d = self._device_operand(x, dt)
        out = self.allocate(cols * dt.byteSize)
        self._check(self._lib.hc_column_sum(self._ctx, _HC_DTYPE[dt], x_d.ptr, int(rows), int(cols), out.ptr))
        out._mark()
        out._inputs = (x_d,)
        return out

    def cast(self, x, count: int, inType, outType) -> CUDAData:
        """Backend.cast (Backend.swift:489-494) between float16 and float32."""
        di, do = _as_dtype(inType), _as_dtype(outType)
        if di not in _HC_DTYPE or do not in _HC_DTYPE:
            raise NotImplementedByBackend(f"cast {di.value} -> {do.value}")
        x_d = self._device_operand(x, di)
        out = self.allocate(count * do.byteSize)
        self._check(self._lib.hc_cast(self._ctx, _HC_DTYPE[di], _HC_DTYPE[do], x_d.ptr, int(count), out.ptr))
        out._mark()
        out._inputs = (x_d,)
        return out

    def add(self, a, b, count: int, dtype) -> CUDAData:
        """binaryOp(.add) on equal shapes (gradient accumulation, Tensor.swift:370-372)."""
        dt = _as_dtype(dtype)
        a_d, b_d = self._device_operand(a, dt), self._device_operand(b, dt)
        out = self.allocate(count * dt.byteSize)
        self._check(self._lib.hc_add(self._ctx, _HC_DTYPE[dt], a_d.ptr, b_d.ptr, int(count), out.ptr))
        out._mark()
        out._inputs = (a_d, b_d)
        return out

    def constant(self, value: float, count: int, dtype) -> CUDAData:
        """Backend.constant (Backend.swift:787-791): `count` elements equal to `value`."""
        dt = _as_dtype(dtype)
        if dt not in _HC_DTYPE:
            raise NotImplementedByBackend(f"constant for dtype {dt.value}")
        out = self.allocate(count * dt.byteSize)
        self._check(self._lib.hc_constant(self._ctx, _HC_DTYPE[dt], float(value), int(count), out.ptr))
        out._mark()
        return out

    def transpose(self, x, matrixCount: int, rows: int, cols: int, dtype) -> CUDAData:
        """The materialised `t()` of the last two axes (Index.swift:359-362)."""
        dt = _as_dtype(dtype)
        x_d = self._device_operand(x, dt)
        out = self.allocate(matrixCount * rows * cols * dt.byteSize)
        self._check(self._lib.hc_transpose(self._ctx, _HC_DTYPE[dt], int(matrixCount), x_d.ptr, int(rows), int(cols),
                                          out.ptr))
        out._mark()
        out._inputs = (x_d,)
        return out

    def seed(self, x: int):
        """RandomGenerator.seed (Sources/Honeycrisp/Random.swift:57-64): state = [seed, 0]."""
        self._rng_state = [int(x) & 0xFFFFFFFFFFFFFFFF, 0]

    def sample(self, count: int, dist: str, dtype) -> CUDAData:
        """RandomGenerator.sample(count:dist:dtype:): `dist` is "uniform" or "normal"; advances
        the generator state exactly as the reference's CPU generator does."""
        dt = _as_dtype(dtype)
        if dt not in _HC_DTYPE:
            raise NotImplementedByBackend(f"random for dtype {dt.value}")
        if not hasattr(self, "_rng_state"):
            self.seed(0)
        out = self.allocate(count * dt.byteSize)
        nxt = ctypes.c_uint64()
        self._check(self._lib.hc_random(self._ctx, 1 if dist == "normal" else 0, _HC_DTYPE[dt], self._rng_state[0],
                                       self._rng_state[1], int(count), out.ptr, ctypes.byref(nxt)))
        self._rng_state[1] = nxt.value
        out._mark()
        return out

    def hostSync(self):
        """Wait for every asynchronous host-buffer product enqueued so far."""
        self._check(self._lib.hc_host_sync(self._ctx))

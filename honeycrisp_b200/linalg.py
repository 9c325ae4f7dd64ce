"""Tensor-level matmul with the reference's autodiff flag algebra.

Mirrors Sources/Honeycrisp/Linalg.swift:45-137: shape checks, output shape, the backend call
with post-transpose logical dimensions, and the two backward products

    dA = matmul(a: grad, transA: transOut, b: B, transB: !transB, transOut: transA)   (:75)
    dB = matmul(a: A, transA: !transA, b: grad, transB: transOut, transOut: transB)   (:78)

so that the reference's gradient known-answer tests can be replayed against the CUDA backend.
Only what those products need is here; there is no general autodiff engine.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import numpy as np

from .backend import CUDABackend, CUDAData, DType, _as_dtype


class Tensor:
    """A dense, contiguous, row-major tensor on a CUDABackend (Tensor.swift:21: shape, dtype, data)."""

    def __init__(self, backend: CUDABackend, data: CUDAData, shape: Sequence[int], dtype,
                 backward: Optional[Callable[["Tensor"], None]] = None):
        self.backend = backend
        self.data = data
        self.shape = list(int(s) for s in shape)
        self.dtype = _as_dtype(dtype)
        self._backward = backward
        self.grad: Optional["Tensor"] = None
        self.needsGrad = False

    @staticmethod
    def fromHost(backend: CUDABackend, values, shape: Sequence[int], dtype) -> "Tensor":
        dt = _as_dtype(dtype)
        arr = np.asarray(values, dtype=dt.numpy).reshape(shape)
        return Tensor(backend, backend.collection(arr, dt), shape, dt)

    def onGrad(self) -> "Tensor":
        """Leaf that records the gradient reaching it (Tensor.onGradUnsafe in the reference's tests)."""
        leaf = Tensor(self.backend, self.data, self.shape, self.dtype)
        leaf.needsGrad = True
        return leaf

    def numpy(self) -> np.ndarray:
        n = int(np.prod(self.shape)) if self.shape else 1
        return self.data.onCPU(self.dtype.numpy)[:n].reshape(self.shape)

    def backward(self, grad: "Tensor") -> None:
        if self._backward is not None:
            self._backward(grad)
        elif self.needsGrad:
            self.grad = grad


def _product(xs) -> int:
    out = 1
    for x in xs:
        out *= int(x)
    return out


def matmul(a: Tensor, transA: bool, b: Tensor, transB: bool, transOut: bool, kernel: int = 0) -> Tensor:
    """Tensor.matmul(a:transA:b:transB:transOut:) (Linalg.swift:45-82)."""
    assert len(a.shape) == 2 and len(b.shape) == 2, f"invalid shapes for matmul: {a.shape}, {b.shape}"
    assert a.dtype == b.dtype, f"mismatched dtypes for matmul: {a.dtype} and {b.dtype}"
    aShape = [a.shape[1], a.shape[0]] if transA else list(a.shape)
    bShape = [b.shape[1], b.shape[0]] if transB else list(b.shape)
    assert aShape[1] == bShape[0], f"shape mismatch for matmul (with transposes): {aShape}, {bShape}"
    outShape = [bShape[1], aShape[0]] if transOut else [aShape[0], bShape[1]]
    backend = a.backend
    data = backend.matmul(a.data, transA, b.data, transB, transOut, aShape[0], aShape[1], bShape[1], a.dtype,
                          kernel=kernel)
    if not (a.needsGrad or a._backward or b.needsGrad or b._backward):
        return Tensor(backend, data, outShape, a.dtype)

    def backward(grad: Tensor) -> None:
        a.backward(matmul(grad, transOut, _detached(b), not transB, transA, kernel=kernel))
        b.backward(matmul(_detached(a), not transA, grad, transOut, transB, kernel=kernel))

    return Tensor(backend, data, outShape, a.dtype, backward=backward)


def batchedMatmul(a: Tensor, transA: bool, b: Tensor, transB: bool, transOut: bool, kernel: int = 0) -> Tensor:
    """Tensor.batchedMatmul(a:transA:b:transB:transOut:) (Linalg.swift:84-129)."""
    assert len(a.shape) > 2 and len(b.shape) > 2 and a.shape[:-2] == b.shape[:-2], \
        f"invalid shapes for batched matmul: {a.shape}, {b.shape}"
    assert a.dtype == b.dtype, f"mismatched dtypes for batched matmul: {a.dtype} and {b.dtype}"
    batchShape: List[int] = list(a.shape[:-2])
    aShape = [a.shape[-1], a.shape[-2]] if transA else [a.shape[-2], a.shape[-1]]
    bShape = [b.shape[-1], b.shape[-2]] if transB else [b.shape[-2], b.shape[-1]]
    assert aShape[1] == bShape[0], f"shape mismatch for batched matmul: {a.shape} (trans={transA}), {b.shape} (trans={transB})"
    outShape = batchShape + ([bShape[1], aShape[0]] if transOut else [aShape[0], bShape[1]])
    backend = a.backend
    data = backend.batchedMatmul(_product(batchShape), a.data, transA, b.data, transB, transOut, aShape[0],
                                 aShape[1], bShape[1], a.dtype, kernel=kernel)
    if not (a.needsGrad or a._backward or b.needsGrad or b._backward):
        return Tensor(backend, data, outShape, a.dtype)

    def backward(grad: Tensor) -> None:
        a.backward(batchedMatmul(grad, transOut, _detached(b), not transB, transA, kernel=kernel))
        b.backward(batchedMatmul(_detached(a), not transA, grad, transOut, transB, kernel=kernel))

    return Tensor(backend, data, outShape, a.dtype, backward=backward)


def _detached(t: Tensor) -> Tensor:
    """noGrad(): the same data without gradient tracking (Linalg.swift:75,78)."""
    return Tensor(t.backend, t.data, t.shape, t.dtype)

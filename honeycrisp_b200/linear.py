"""`Linear` on the CUDA backend: forward and backward pass without leaving the device.

Mirrors Sources/Honeycrisp/Trainable.swift:508-547: weight `[inCount, outCount]` initialised
uniformly in +-sqrt(3)/sqrt(inCount) (`(rand - 0.5) * (sqrt(3) / 0.5 / sqrt(inCount))`), bias
`[outCount]` of zeros, forward `x . W + b` with inputs of rank > 2 flattened to
`[prod(leading dims), inCount]`.  The backward pass issues what the reference's autodiff issues
for that forward (Linalg.swift:73-80 and Tensor.swift:845-871):

    dX = matmul(a: dY, transA: false, b: W, transB: true,  transOut: false)
    dW = matmul(a: X,  transA: true,  b: dY, transB: false, transOut: false)
    db = sum of dY over its rows            (reduceBroadcast of the broadcast add)

Weights come from numpy's generator, not from Honeycrisp's Philox stream, so parameter values
differ from a Honeycrisp `Linear` with the same seed; shapes, ranges and arithmetic do not.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import numpy as np

from .backend import CUDABackend, CUDAData, DType, _as_dtype


class Linear:
    def __init__(self, backend: CUDABackend, inCount: int, outCount: int, dtype=np.float32, bias: bool = True,
                 seed: int = 0):
        self.backend, self.inCount, self.outCount = backend, int(inCount), int(outCount)
        self.dtype = _as_dtype(dtype)
        rng = np.random.default_rng(seed)
        w = (rng.random((inCount, outCount), dtype=np.float32) - 0.5) * (math.sqrt(3.0) / 0.5 / math.sqrt(inCount))
        self.weight = backend.collection(w.astype(self.dtype.numpy), self.dtype)
        self.bias = backend.collection(np.zeros(outCount, dtype=self.dtype.numpy), self.dtype) if bias else None
        self.weightGrad: Optional[CUDAData] = None
        self.biasGrad: Optional[CUDAData] = None

    def __call__(self, x, shape: Sequence[int]) -> Tuple[CUDAData, list]:
        """Forward.  `x` holds a dense tensor of `shape` whose last dimension is inCount;
        returns the output buffer and its shape."""
        shape = list(int(s) for s in shape)
        assert shape and shape[-1] == self.inCount, f"last dimension must be {self.inCount}: {shape}"
        rows = int(np.prod(shape[:-1])) if len(shape) > 1 else 1
        out = self.backend.linearForward(x, self.weight, self.bias, rows, self.inCount, self.outCount, self.dtype)
        return out, shape[:-1] + [self.outCount]

    def backward(self, x, shape: Sequence[int], outGrad) -> CUDAData:
        """Backward for the forward call on (`x`, `shape`): returns dX and accumulates the
        parameter gradients (Param.addGrad, Trainable.swift:258-266)."""
        shape = list(int(s) for s in shape)
        rows = int(np.prod(shape[:-1])) if len(shape) > 1 else 1
        be = self.backend
        dx = be.matmul(outGrad, False, self.weight, True, False, rows, self.outCount, self.inCount, self.dtype)
        dw = be.matmul(x, True, outGrad, False, False, self.inCount, rows, self.outCount, self.dtype)
        self.weightGrad = dw if self.weightGrad is None else be.add(self.weightGrad, dw, self.inCount * self.outCount,
                                                                    self.dtype)
        if self.bias is not None:
            db = be.columnSum(outGrad, rows, self.outCount, self.dtype)
            self.biasGrad = db if self.biasGrad is None else be.add(self.biasGrad, db, self.outCount, self.dtype)
        return dx

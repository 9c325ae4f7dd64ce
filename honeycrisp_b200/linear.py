"""`Linear` on the CUDA backend: forward and backward pass without leaving the device.

Mirrors Sources/Honeycrisp/Trainable.swift:508-547: weight `[inCount, outCount]` initialised
uniformly in +-sqrt(3)/sqrt(inCount) (`(rand - 0.5) * (sqrt(3) / 0.5 / sqrt(inCount))`), bias
`[outCount]` of zeros, forward `x . W + b` with inputs of rank > 2 flattened to
`[prod(leading dims), inCount]`.  The backward pass issues what the reference's autodiff issues
for that forward (Linalg.swift:73-80 and Tensor.swift:845-871):

    dX = matmul(a: dY, transA: false, b: W, transB: true,  transOut: false)
    dW = matmul(a: X,  transA: true,  b: dY, transB: false, transOut: false)
    db = sum of dY over its rows            (reduceBroadcast of the broadcast add)

Parameter dtypes follow the reference exactly (Trainable.swift:514-544): the weight is created
in `dtype`, the bias ALWAYS in float32 (`Tensor(zeros: [outCount])`), and the forward pass uses
`weight.cast(castParams ?? weight.dtype)` and `bias.cast(castParams ?? bias.dtype)`.  So a layer
computing in float16 is either `Linear(dtype: .float16, castParams: .float16)` (float16 weight,
float32 bias cast on use) or `Linear(dtype: .float32, castParams: .float16)` (float32 master
weights cast on every call); a float16 layer with a bias and no castParams adds float16 to
float32, which the reference's binary ops refuse, and so does this class.  Gradients arrive in the
compute dtype and are cast back to each parameter's dtype (the backward of `cast`).

Weights come from numpy's generator, not from Honeycrisp's Philox stream, so parameter values
differ from a Honeycrisp `Linear` with the same seed; shapes, ranges and arithmetic do not.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import numpy as np

from .backend import CUDABackend, CUDAData, DType, _as_dtype


class Linear:
    def __init__(self, backend: CUDABackend, inCount: int, outCount: int, dtype=np.float32, castParams=None,
                 bias: bool = True, seed: int = 0):
        self.backend, self.inCount, self.outCount = backend, int(inCount), int(outCount)
        self.dtype = _as_dtype(dtype)                                    # of the weight
        self.castParams = _as_dtype(castParams) if castParams is not None else None
        self.biasDType = DType.float32                                   # Trainable.swift:524
        rng = np.random.default_rng(seed)
        w = (rng.random((inCount, outCount), dtype=np.float32) - 0.5) * (math.sqrt(3.0) / 0.5 / math.sqrt(inCount))
        self.weight = backend.collection(w.astype(self.dtype.numpy), self.dtype)
        self.bias = backend.collection(np.zeros(outCount, dtype=np.float32), DType.float32) if bias else None
        self.weightGrad: Optional[CUDAData] = None
        self.biasGrad: Optional[CUDAData] = None

    @property
    def computeDType(self) -> DType:
        return self.castParams or self.dtype

    def _castWeight(self) -> CUDAData:
        ct = self.computeDType
        if ct == self.dtype:
            return self.weight
        return self.backend.cast(self.weight, self.inCount * self.outCount, self.dtype, ct)

    def _castBias(self) -> Optional[CUDAData]:
        if self.bias is None:
            return None
        bt = self.castParams or self.biasDType
        if bt != self.computeDType:
            # h is in the weight's dtype, the bias in float32: the reference's `h + bias` asserts
            raise ValueError(f"Linear: bias is {bt.value} but the product is {self.computeDType.value}; "
                             f"pass castParams (Trainable.swift:540-544)")
        if bt == self.biasDType:
            return self.bias
        return self.backend.cast(self.bias, self.outCount, self.biasDType, bt)

    def __call__(self, x, shape: Sequence[int]) -> Tuple[CUDAData, list]:
        """Forward.  `x` holds a dense tensor of `shape`, in the layer's compute dtype, whose last
        dimension is inCount; returns the output buffer and its shape."""
        shape = list(int(s) for s in shape)
        assert shape and shape[-1] == self.inCount, f"last dimension must be {self.inCount}: {shape}"
        rows = int(np.prod(shape[:-1])) if len(shape) > 1 else 1
        out = self.backend.linearForward(x, self._castWeight(), self._castBias(), rows, self.inCount, self.outCount,
                                         self.computeDType)
        return out, shape[:-1] + [self.outCount]

    def backward(self, x, shape: Sequence[int], outGrad) -> CUDAData:
        """Backward for the forward call on (`x`, `shape`): returns dX and accumulates the
        parameter gradients (Param.addGrad, Trainable.swift:258-266)."""
        shape = list(int(s) for s in shape)
        rows = int(np.prod(shape[:-1])) if len(shape) > 1 else 1
        be = self.backend
        ct = self.computeDType
        dx = be.matmul(outGrad, False, self._castWeight(), True, False, rows, self.outCount, self.inCount, ct)
        dw = be.matmul(x, True, outGrad, False, False, self.inCount, rows, self.outCount, ct)
        if ct != self.dtype:                          # backward of weight.cast(castParams)
            dw = be.cast(dw, self.inCount * self.outCount, ct, self.dtype)
        self.weightGrad = dw if self.weightGrad is None else be.add(self.weightGrad, dw, self.inCount * self.outCount,
                                                                    self.dtype)
        if self.bias is not None:
            db = be.columnSum(outGrad, rows, self.outCount, ct)
            if ct != self.biasDType:                  # backward of bias.cast(castParams)
                db = be.cast(db, self.outCount, ct, self.biasDType)
            self.biasGrad = db if self.biasGrad is None else be.add(self.biasGrad, db, self.outCount, self.biasDType)
        return dx

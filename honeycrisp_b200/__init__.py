"""honeycrisp_b200: sm_100a implementation of Honeycrisp's dense matrix-product path.

Public surface:
  CUDABackend, CUDAData, DType, BackendError (+ subclasses)  - honeycrisp_b200.backend
  Tensor, matmul, batchedMatmul                               - honeycrisp_b200.linalg
  Linear (fused-bias forward, on-device backward)             - honeycrisp_b200.linear
  shardBatch, columnBlock, batchedMatmulSharded, matmulColumnSplit - honeycrisp_b200.sharding
The compute library is honeycrisp_b200/libhccuda.so (C ABI in include/hc_cuda.h).
"""
from .backend import (AllocationFailed, BackendError, CUDABackend, CUDAData, DeviceTimeout, DType,
                      KernelFailed, NotImplementedByBackend)
from .linalg import Tensor, batchedMatmul, matmul
from .linear import Linear

__all__ = [
    "AllocationFailed", "BackendError", "CUDABackend", "CUDAData", "DeviceTimeout", "DType", "KernelFailed",
    "Linear", "NotImplementedByBackend", "Tensor", "batchedMatmul", "matmul",
]

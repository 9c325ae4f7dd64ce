"""ctypes binding of libhccuda.so, symbol for symbol as declared in include/hc_cuda.h.

There is no fallback: if the library is missing and cannot be built, importing raises.
"""
from __future__ import annotations

import ctypes
import os

from . import build as _build

_i64 = ctypes.c_int64
_vp = ctypes.c_void_p
_int = ctypes.c_int
_sz = ctypes.c_size_t

HC_OK = 0
HC_ERR_ALLOCATION_FAILED = 1
HC_ERR_KERNEL_FAILED = 2
HC_ERR_NOT_IMPLEMENTED = 3
HC_ERR_INVALID_ARGUMENT = 4
HC_ERR_TIMEOUT = 5
HC_ERR_CUDA = 6

HC_F16 = 0
HC_F32 = 1

HC_KERNEL_AUTO = 0
HC_KERNEL_SIMT = 1
HC_KERNEL_SIMT_EXACT = 2
HC_KERNEL_TENSOR = 3


class LaunchInfo(ctypes.Structure):
    _fields_ = [
        ("kernel", _int), ("tile_m", _int), ("tile_n", _int), ("tile_k", _int),
        ("stages", _int), ("grid", _int), ("block", _int),
        ("tiles", _i64), ("flops", _i64), ("scratch_bytes", _sz),
    ]


class PlanInfo(ctypes.Structure):
    _fields_ = [
        ("tile_m", _int), ("tile_n", _int), ("ctas_per_tile", _int), ("slabs_per_slot", _int),
        ("parts", _int), ("slots_per_part", _int), ("tiles", _i64), ("workspace_bytes", _sz),
    ]


# name -> (restype, argtypes); the complete export list of include/hc_cuda.h
SIGNATURES = {
    "hc_init": (_int, [_int, ctypes.POINTER(_vp)]),
    "hc_destroy": (None, [_vp]),
    "hc_set_stream": (_int, [_vp, _vp]),
    "hc_get_stream": (_vp, [_vp]),
    "hc_get_device": (_int, [_vp]),
    "hc_alloc": (_int, [_vp, _sz, ctypes.POINTER(_vp)]),
    "hc_free": (_int, [_vp, _vp]),
    "hc_h2d": (_int, [_vp, _vp, _vp, _sz]),
    "hc_d2h": (_int, [_vp, _vp, _vp, _sz]),
    "hc_d2h_async": (_int, [_vp, _vp, _vp, _sz, ctypes.POINTER(_vp)]),
    "hc_h2d_async": (_int, [_vp, _vp, _vp, _sz, ctypes.POINTER(_vp)]),
    "hc_enqueue_wait": (_int, [_vp, _vp]),
    "hc_sync": (_int, [_vp]),
    "hc_event_record": (_int, [_vp, ctypes.POINTER(_vp)]),
    "hc_event_wait": (_int, [_vp]),
    "hc_event_elapsed_ms": (_int, [_vp, _vp, ctypes.POINTER(ctypes.c_float)]),
    "hc_event_destroy": (None, [_vp]),
    "hc_matmul": (_int, [_vp, _int, _vp, _int, _vp, _int, _int, _i64, _i64, _i64, _vp]),
    "hc_batched_matmul": (_int, [_vp, _int, _i64, _vp, _int, _vp, _int, _int, _i64, _i64, _i64, _vp]),
    "hc_batched_matmul_ex": (_int, [_vp, _int, _int, _i64, _vp, _int, _vp, _int, _int, _i64, _i64, _i64, _vp]),
    "hc_batched_matmul_host": (_int, [_vp, _int, _i64, _vp, _int, _vp, _int, _int, _i64, _i64, _i64, _vp]),
    "hc_batched_matmul_host_async": (_int, [_vp, _int, _i64, _vp, _int, _vp, _int, _int, _i64, _i64, _i64, _vp]),
    "hc_host_sync": (_int, [_vp]),
    "hc_matmul_colblock": (_int, [_vp, _int, _int, _vp, _int, _vp, _int, _int, _i64, _i64, _i64, _i64, _i64, _vp]),
    "hc_linear_forward": (_int, [_vp, _int, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "hc_column_sum": (_int, [_vp, _int, _vp, _i64, _i64, _vp]),
    "hc_cast": (_int, [_vp, _int, _int, _vp, _i64, _vp]),
    "hc_add": (_int, [_vp, _int, _vp, _vp, _i64, _vp]),
    "hc_transpose": (_int, [_vp, _int, _i64, _vp, _i64, _i64, _vp]),
    "hc_random": (_int, [_vp, _int, _int, ctypes.c_uint64, ctypes.c_uint64, _i64, _vp, ctypes.POINTER(ctypes.c_uint64)]),
    "hc_matmul_colblock_push": (_int, [_vp, _int, _vp, _int, _vp, _int, _int, _i64, _i64, _i64, _i64, _i64, _vp,
                                      ctypes.POINTER(_vp), _int]),
    "hc_shared_alloc": (_int, [_vp, _sz, ctypes.POINTER(_vp)]),
    "hc_shared_free": (_int, [_vp, _vp]),
    "hc_ipc_export": (_int, [_vp, _vp, _vp]),
    "hc_ipc_open": (_int, [_vp, _vp, ctypes.POINTER(_vp)]),
    "hc_ipc_close": (_int, [_vp, _vp]),
    "hc_matmul_f32_static_scratch": (_int, [_vp, _vp, _int, _vp, _int, _int, _i64, _i64, _i64, _vp]),
    "hc_static_scratch_capacity": (_sz, []),
    "hc_status_string": (ctypes.c_char_p, [_int]),
    "hc_last_error": (ctypes.c_char_p, [_vp]),
    "hc_last_launch_info": (_int, [_vp, ctypes.POINTER(LaunchInfo)]),
    "hc_plan_product": (_int, [_int, _i64, _int, _int, _int, _i64, _i64, _i64, _int, ctypes.POINTER(PlanInfo)]),
    "hc_launch_count": (_i64, [_vp]),
    "hc_check_device_status": (_int, [_vp]),
    "hc_selftest_bounded_wait": (_int, [_vp, _int]),
    "hc_version": (ctypes.c_char_p, []),
}

_lib = None


def lib_path() -> str:
    return _build.LIB_PATH


def load() -> ctypes.CDLL:
    """Load libhccuda.so (building it first if the sources are newer). Raises on failure."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB_PATH
    override = os.environ.get("HC_CUDA_LIB")     # a differently built libhccuda.so, for A/B runs
    if override:
        path = override
    elif not os.path.exists(path) or os.environ.get("HC_CUDA_REBUILD") == "1":
        path = _build.build(force=True)
    elif _build._stale():
        # Sources are newer than the library: rebuild if a compiler is at hand, otherwise say so
        # and use what is there (a copied tree can carry arbitrary file times).
        try:
            path = _build.build()
        except Exception as e:  # noqa: BLE001
            import warnings
            warnings.warn(f"libhccuda.so is older than its sources and could not be rebuilt: {e}")
    L = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(L, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L

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
    "hc_constant": (_int, [_vp, _int, ctypes.c_float, _i64, _vp]),
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
    "hc_copy_last_error": (_sz, [_vp, ctypes.c_char_p, _sz]),
    "hc_last_launch_info": (_int, [_vp, ctypes.POINTER(LaunchInfo)]),
    "hc_plan_product": (_int, [_int, _i64, _int, _int, _int, _i64, _i64, _i64, _int, ctypes.POINTER(PlanInfo)]),
    "hc_launch_count": (_i64, [_vp]),
    "hc_check_device_status": (_int, [_vp]),
    "hc_selftest_bounded_wait": (_int, [_vp, _int]),
    "hc_inject_allocation_failures": (_int, [_vp, _int]),
    "hc_set_tracing": (_int, [_vp, _int]),
    "hc_last_elapsed_ms": (_int, [_vp, ctypes.POINTER(ctypes.c_float)]),
    "hc_group_unique_id": (_int, [_vp]),
    "hc_group_init": (_int, [_vp, _int, _int, _vp, ctypes.POINTER(_vp)]),
    "hc_group_destroy": (None, [_vp]),
    "hc_group_rank": (_int, [_vp]),
    "hc_group_world": (_int, [_vp]),
    "hc_group_set_timeout_ms": (_int, [_vp, _int]),
    "hc_shard_range": (_int, [_i64, _int, _int, ctypes.POINTER(_i64), ctypes.POINTER(_i64)]),
    "hc_column_block": (_int, [_i64, _int, _int, ctypes.POINTER(_i64), ctypes.POINTER(_i64)]),
    "hc_batched_matmul_sharded": (_int, [_vp, _int, _i64, _vp, _int, _vp, _int, _int, _i64, _i64, _i64, _vp, _int]),
    "hc_matmul_nsplit_allgather": (_int, [_vp, _int, _vp, _int, _vp, _int, _i64, _i64, _i64, _vp, _int]),
    "hc_group_result_alloc": (_int, [_vp, _sz, ctypes.POINTER(_vp)]),
    "hc_group_result_free": (_int, [_vp, _vp]),
    "hc_group_barrier": (_int, [_vp]),
    "hc_group_selftest_missing_peer": (_int, [_vp, _int]),
    "hc_version": (ctypes.c_char_p, []),
}

_libs = {}


def lib_path(diagnostics: bool = False) -> str:
    return _build.DIAG_LIB_PATH if diagnostics else _build.LIB_PATH


def load(diagnostics: bool = False) -> ctypes.CDLL:
    """Load libhccuda.so (building it first if the sources are newer). Raises on failure.

    `diagnostics=True` loads the second build of the same sources (libhccuda_diag.so), in which
    the planner's choices can be forced through HC_TC_* environment variables; the test-suite
    uses it to reach every tile shape with small products.  Both can live in one process."""
    if diagnostics in _libs:
        return _libs[diagnostics]
    path = lib_path(diagnostics)
    override = os.environ.get("HC_CUDA_LIB")     # a differently built libhccuda.so, for A/B runs
    if override and not diagnostics:
        path = override
    elif os.environ.get("HC_CUDA_REBUILD") == "1":
        path = _build.build(force=True, diagnostics=diagnostics)
    elif not os.path.exists(path):
        path = _build.build(diagnostics=diagnostics)   # a missing library counts as stale
    elif _build._stale(path):
        # Sources are newer than the library: rebuild if a compiler is at hand, otherwise say so
        # and use what is there (a copied tree can carry arbitrary file times).
        try:
            path = _build.build(diagnostics=diagnostics)
        except Exception as e:  # noqa: BLE001
            import warnings
            warnings.warn(f"{os.path.basename(path)} is older than its sources and could not be rebuilt: {e}")
    L = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(L, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    _libs[diagnostics] = L
    return L

"""The C-ABI library loads on a machine without a GPU and exports everything the header declares."""
import ctypes
import os
import re

import pytest

from honeycrisp_b200 import _lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "hc_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b(hc_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_header_declares_the_hot_path():
    names = declared_functions()
    for required in ("hc_init", "hc_destroy", "hc_matmul", "hc_batched_matmul", "hc_batched_matmul_host",
                     "hc_matmul_colblock", "hc_alloc", "hc_free", "hc_h2d", "hc_d2h", "hc_event_wait"):
        assert required in names


def test_library_exports_every_declared_symbol():
    lib = L.load()
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in include/hc_cuda.h but not exported"
        assert name in L.SIGNATURES, f"{name} has no ctypes signature"
    # and nothing is bound that the header does not declare
    assert set(L.SIGNATURES) <= set(declared_functions())


def test_diagnostics_build_exports_the_same_interface():
    lib = L.load(diagnostics=True)
    for name in declared_functions():
        assert hasattr(lib, name)


def test_partitions_are_host_arithmetic():
    lib = L.load()
    b, c = ctypes.c_int64(), ctypes.c_int64()
    assert lib.hc_shard_range(64, 8, 3, ctypes.byref(b), ctypes.byref(c)) == L.HC_OK and (b.value, c.value) == (24, 8)
    assert lib.hc_column_block(16384, 8, 7, ctypes.byref(b), ctypes.byref(c)) == L.HC_OK and (b.value, c.value) == (14336, 2048)
    assert lib.hc_shard_range(64, 8, 8, ctypes.byref(b), ctypes.byref(c)) == L.HC_ERR_INVALID_ARGUMENT
    assert lib.hc_group_init(None, 1, 0, None, None) == L.HC_ERR_INVALID_ARGUMENT
    assert lib.hc_group_world(None) == 0 and lib.hc_group_rank(None) == -1


def test_header_compiles_as_plain_c(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "hc_cuda.h"\nint main(void) { hc_launch_info i; (void)i; return (int)HC_OK; }\n')
    rc = os.system(f"gcc -std=c99 -Wall -Werror -I{ROOT}/include -c {src} -o {tmp_path}/t.o")
    assert rc == 0


def test_status_strings_and_version():
    lib = L.load()
    assert lib.hc_version().decode() == "0.2"
    seen = {lib.hc_status_string(i).decode() for i in range(7)}
    assert len(seen) == 7
    assert lib.hc_status_string(99).decode() == "unknown status"


def test_null_context_is_rejected_without_touching_a_device():
    lib = L.load()
    assert lib.hc_sync(None) == L.HC_ERR_INVALID_ARGUMENT
    assert lib.hc_matmul(None, L.HC_F32, None, 0, None, 0, 0, 1, 1, 1, None) == L.HC_ERR_INVALID_ARGUMENT
    assert lib.hc_launch_count(None) == 0
    assert lib.hc_init(0, None) == L.HC_ERR_INVALID_ARGUMENT


def test_init_reports_failure_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = L.load()
    ctx = ctypes.c_void_p()
    assert lib.hc_init(0, ctypes.byref(ctx)) != L.HC_OK
    assert not ctx.value
    from honeycrisp_b200 import CUDABackend, KernelFailed
    with pytest.raises(KernelFailed):
        CUDABackend(0)

"""hc_matmul_f32_static_scratch: the float32 tensor-core product for hosts that cannot allocate.

Some programs that embed this library must not let it call cudaMalloc - their own allocator has
claimed the device, or they cannot take the device-wide synchronisation an allocation implies.
For them the library carries a fixed work area (a __device__ array in the library image) and this
entry point uses it instead of allocating.  The test drives it through the C ABI, twice in a row
(the work area keeps the previous call's contents, so the second call shows that nothing
depends on its initial state), and compares with the allocating entry point, which must give the
same bits.  Collected last on purpose: a failure here cannot hide another test behind `-x`.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_static_scratch_product_matches_allocating_product_twice():
    from honeycrisp_b200 import CUDABackend, _lib
    lib = _lib.load()
    be = CUDABackend(0)
    try:
        cap = lib.hc_static_scratch_capacity()
        assert cap >= 8 * (512 * 384 + 384 * 640)
        rng = np.random.default_rng(42)
        for call, (rows, inner, cols, ta, tb, to) in enumerate([(512, 384, 640, False, False, False),
                                                                (384, 260, 520, True, False, True)]):
            a = (rng.random(rows * inner, dtype=np.float32) * 2 - 1)
            b = (rng.random(inner * cols, dtype=np.float32) * 2 - 1)
            a_d, b_d = be.collection(a, np.float32), be.collection(b, np.float32)
            want = be.matmul(a_d, ta, b_d, tb, to, rows, inner, cols, np.float32,
                             kernel=_lib.HC_KERNEL_TENSOR).onCPU(np.float32)
            out = be.allocate(rows * cols * 4)
            st = lib.hc_matmul_f32_static_scratch(be._ctx, a_d.ptr, int(ta), b_d.ptr, int(tb), int(to), rows, inner,
                                                  cols, out.ptr)
            assert st == _lib.HC_OK, lib.hc_last_error(be._ctx).decode()
            got = out.onCPU(np.float32)
            be.checkDeviceStatus()
            # Same kernels on the same split operands: equal bit for bit (the float32 tests
            # elsewhere allow 1e-5 relative Frobenius error against the CPU result).
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"call {call}"
            f64 = (a.reshape((inner, rows) if ta else (rows, inner)).astype(np.float64))
            f64 = f64.T if ta else f64
            bm = b.reshape((cols, inner) if tb else (inner, cols)).astype(np.float64)
            bm = bm.T if tb else bm
            ref = f64 @ bm
            ref = ref.T if to else ref
            err = np.linalg.norm(got.astype(np.float64) - ref.reshape(-1)) / np.linalg.norm(ref)
            assert err < 1e-5
        # A long contraction over few outputs: the allocating path cuts it into parts and sums float32
        # partial matrices; here those live in the static area too, so the bits still agree.
        rows, inner, cols = 128, 8192, 128
        plan = _lib.PlanInfo()
        assert lib.hc_plan_product(_lib.HC_F32, 1, 0, 0, 0, rows, inner, cols, 148, ctypes.byref(plan)) == _lib.HC_OK
        assert plan.parts > 1 and 8 * (rows * inner + inner * cols) + plan.workspace_bytes <= cap
        a = (rng.random(rows * inner, dtype=np.float32) * 2 - 1)
        b = (rng.random(inner * cols, dtype=np.float32) * 2 - 1)
        a_d, b_d = be.collection(a, np.float32), be.collection(b, np.float32)
        want = be.matmul(a_d, False, b_d, False, False, rows, inner, cols, np.float32,
                         kernel=_lib.HC_KERNEL_TENSOR).onCPU(np.float32)
        assert be.lastLaunchInfo()["tiles"] > 1
        out = be.allocate(rows * cols * 4)
        st = lib.hc_matmul_f32_static_scratch(be._ctx, a_d.ptr, 0, b_d.ptr, 0, 0, rows, inner, cols, out.ptr)
        assert st == _lib.HC_OK, lib.hc_last_error(be._ctx).decode()
        got = out.onCPU(np.float32)
        be.checkDeviceStatus()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), "cut contraction"
        ref = a.reshape(rows, inner).astype(np.float64) @ b.reshape(inner, cols).astype(np.float64)
        assert np.linalg.norm(got.astype(np.float64) - ref.reshape(-1)) / np.linalg.norm(ref) < 1e-5
        # A product whose work area does not fit is refused, with the sizes in the message.
        big = 4096
        st = lib.hc_matmul_f32_static_scratch(be._ctx, a_d.ptr, 0, b_d.ptr, 0, 0, big, big, big, out.ptr)
        assert st == _lib.HC_ERR_INVALID_ARGUMENT
        assert str(cap) in lib.hc_last_error(be._ctx).decode()
    finally:
        be.close()

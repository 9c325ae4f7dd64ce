"""The group entry points and the context's housekeeping on ONE GPU: a group of one rank runs the
same code paths as a larger one (barriers with itself, result buffers, the fused epilogue with no
peers), the missing-peer time-out is made on the host side, and the allocation-failure hook shows
that a failed growth of the work area leaves the context usable."""
import ctypes

import numpy as np
import pytest

from oracle import reference_cpu as ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    from honeycrisp_b200 import CUDABackend
    b = CUDABackend(0)
    yield b
    b.checkDeviceStatus()
    b.close()


def test_group_of_one_rank(be):
    from honeycrisp_b200 import _lib
    from honeycrisp_b200.sharding import DeviceGroup
    grp = DeviceGroup(be, 0, 1)
    try:
        assert (be._lib.hc_group_rank(grp._g), be._lib.hc_group_world(grp._g)) == (0, 1)
        rng = np.random.default_rng(7)
        M, K, N = 520, 264, 776
        a = (rng.random((M, K), dtype=np.float32) * 2 - 1)
        b = (rng.random((K, N), dtype=np.float32) * 2 - 1)
        a_d, b_d = be.collection(a, np.float32), be.collection(b, np.float32)
        one = be.matmul(a_d, False, b_d, False, False, M, K, N, np.float32, kernel=_lib.HC_KERNEL_TENSOR).onCPU(np.float32)
        plain = be.allocate(M * N * 4)
        grp.matmulColumnSplit(a_d, False, b_d, False, M, K, N, np.float32, plain)
        assert np.array_equal(plain.onCPU(np.float32), one)
        shared = grp.resultAllocate(M * N * 4)
        for _ in range(2):
            grp.matmulColumnSplit(a_d, False, b_d, False, M, K, N, np.float32, shared, fused=True)
        assert np.array_equal(shared.onCPU(np.float32), one)
        with pytest.raises(ValueError):
            grp.matmulColumnSplit(a_d, False, b_d, False, M, K, N, np.float32, plain, fused=True)
        grp.resultFree(shared)
        # batched: the one rank owns every matrix; gathered or not is the same thing
        q = rng.standard_normal((3, 136, 72)).astype(np.float16)
        k = rng.standard_normal((3, 200, 72)).astype(np.float16)
        q_d, k_d = be.collection(q, np.float16), be.collection(k, np.float16)
        want = be.batchedMatmul(3, q_d, False, k_d, True, False, 136, 72, 200, np.float16).onCPU(np.float16)
        for gather in (False, True):
            out = be.allocate(3 * 136 * 200 * 2)
            grp.batchedMatmulSharded(3, q_d, False, k_d, True, False, 136, 72, 200, np.float16, out, gather=gather)
            assert np.array_equal(out.onCPU(np.float16), want)
        be.checkDeviceStatus()
    finally:
        grp.close()


def test_missing_peer_times_out_and_the_group_stays_usable(be):
    from honeycrisp_b200 import DeviceTimeout
    from honeycrisp_b200.sharding import DeviceGroup
    grp = DeviceGroup(be, 0, 1)
    try:
        grp.selftestMissingPeer(30)
        with pytest.raises(DeviceTimeout):
            be.checkDeviceStatus()
        be.checkDeviceStatus()                      # cleared
        grp.barrier()                               # the counters are back in step
        x = np.ones((64, 128), dtype=np.float32)
        y = np.ones((128, 32), dtype=np.float32)
        out = be.matmul(x, False, y, False, False, 64, 128, 32, np.float32).onCPU(np.float32)
        be.checkDeviceStatus()
        assert np.all(out == 128.0)
    finally:
        grp.close()


def test_failed_growth_of_the_work_area_leaves_the_context_usable():
    from honeycrisp_b200 import AllocationFailed, CUDABackend, _lib
    be = CUDABackend(0)
    try:
        rng = np.random.default_rng(3)
        a = rng.random((256, 128), dtype=np.float32)
        b = rng.random((128, 256), dtype=np.float32)
        a_d, b_d = be.collection(a, np.float32), be.collection(b, np.float32)
        small = be.matmul(a_d, False, b_d, False, False, 256, 128, 256, np.float32, kernel=_lib.HC_KERNEL_TENSOR).onCPU(np.float32)
        A = rng.random((512, 640), dtype=np.float32)
        B = rng.random((640, 384), dtype=np.float32)
        A_d, B_d = be.collection(A, np.float32), be.collection(B, np.float32)
        out = be.allocate(512 * 384 * 4)
        assert be._lib.hc_inject_allocation_failures(be._ctx, 1) == _lib.HC_OK
        with pytest.raises(AllocationFailed):       # the larger product has to grow the work area
            be.matmul(A_d, False, B_d, False, False, 512, 640, 384, np.float32, kernel=_lib.HC_KERNEL_TENSOR, out=out)
        # the old work area is intact: the small product still runs, and gives the same bits
        again = be.matmul(a_d, False, b_d, False, False, 256, 128, 256, np.float32, kernel=_lib.HC_KERNEL_TENSOR).onCPU(np.float32)
        assert np.array_equal(again, small)
        # and now the growth succeeds
        got = be.matmul(A_d, False, B_d, False, False, 512, 640, 384, np.float32, kernel=_lib.HC_KERNEL_TENSOR, out=out).onCPU(np.float32)
        assert ref.rel_frobenius(got, (A.astype(np.float64) @ B.astype(np.float64)).reshape(-1)) < 1e-5
        # results and staging buffers go through the same allocator
        assert be._lib.hc_inject_allocation_failures(be._ctx, 1) == _lib.HC_OK
        with pytest.raises(AllocationFailed):
            be.allocate(1 << 20)
        assert be._lib.hc_inject_allocation_failures(be._ctx, 1) == _lib.HC_OK
        with pytest.raises(AllocationFailed):
            be.batchedMatmulHost(1, a, False, b, False, False, 256, 128, 256, np.float32)
        host = be.batchedMatmulHost(1, a, False, b, False, False, 256, 128, 256, np.float32)
        assert np.array_equal(host, small)
        be.checkDeviceStatus()
    finally:
        be.close()


def test_host_buffer_call_checks_sizes_before_it_copies(be):
    a = np.zeros(4, dtype=np.float32)
    with pytest.raises(ValueError):
        st = be._lib.hc_batched_matmul_host(be._ctx, 1, 1 << 40, a.ctypes.data, 0, a.ctypes.data, 0, 0, 1 << 20, 1 << 20,
                                            1 << 20, a.ctypes.data)
        be._check(st)


def test_repeated_products_reuse_their_preparation(be):
    """Same buffers, same shape: the second call takes the prepared launch; a different operand
    address, shape or flag must not."""
    from honeycrisp_b200 import _lib
    rng = np.random.default_rng(11)
    a = rng.standard_normal((300, 200)).astype(np.float16)
    b = rng.standard_normal((200, 260)).astype(np.float16)
    a_d, b_d = be.collection(a, np.float16), be.collection(b, np.float16)
    out = be.allocate(300 * 260 * 2)
    want = ref.batched_matmul_f64(1, a, False, b, False, False, 300, 200, 260)
    for _ in range(3):
        got = be.matmul(a_d, False, b_d, False, False, 300, 200, 260, np.float16, kernel=_lib.HC_KERNEL_TENSOR, out=out).onCPU(np.float16)
        assert ref.rel_frobenius(got, want) < 2e-3
    # same buffers read the other way round: a different product
    at = np.ascontiguousarray(a.T)                       # [200,300] stored, read as transA
    at_d = be.collection(at, np.float16)
    got_t = be.matmul(at_d, True, b_d, False, False, 300, 200, 260, np.float16, kernel=_lib.HC_KERNEL_TENSOR, out=out).onCPU(np.float16)
    assert ref.rel_frobenius(got_t, want) < 2e-3
    # new contents at the same addresses are picked up (nothing but addresses is remembered)
    a2 = rng.standard_normal((300, 200)).astype(np.float16)
    be._check(be._lib.hc_h2d(be._ctx, a_d.ptr, a2.ctypes.data, a2.nbytes))
    be.sync()
    got2 = be.matmul(a_d, False, b_d, False, False, 300, 200, 260, np.float16, kernel=_lib.HC_KERNEL_TENSOR, out=out).onCPU(np.float16)
    assert ref.rel_frobenius(got2, ref.batched_matmul_f64(1, a2, False, b, False, False, 300, 200, 260)) < 2e-3


def test_tracing_reports_a_products_device_time(be):
    from honeycrisp_b200 import _lib
    ms = ctypes.c_float()
    assert be._lib.hc_last_elapsed_ms(be._ctx, ctypes.byref(ms)) == _lib.HC_ERR_INVALID_ARGUMENT   # tracing is off
    assert be._lib.hc_set_tracing(be._ctx, 1) == _lib.HC_OK
    a = np.ones((512, 512), dtype=np.float16)
    be.matmul(a, False, a, False, False, 512, 512, 512, np.float16)
    assert be._lib.hc_last_elapsed_ms(be._ctx, ctypes.byref(ms)) == _lib.HC_OK
    assert 0.0 < ms.value < 50.0
    assert be._lib.hc_set_tracing(be._ctx, 0) == _lib.HC_OK


def test_tiny_products_take_the_reference_arithmetic_under_auto(be):
    """float32 with a flag set is the two-rounding loop in the reference (BackendCPU.swift:1290-1300):
    the default kernel choice must give those bits for products too small for a tensor-core tile."""
    from honeycrisp_b200 import _lib
    rng = np.random.default_rng(5)
    a = rng.standard_normal((2, 9, 33)).astype(np.float32)
    b = rng.standard_normal((2, 7, 33)).astype(np.float32)
    got = be.batchedMatmul(2, a, False, b, True, False, 9, 33, 7, np.float32).onCPU(np.float32)
    assert be.lastLaunchInfo()["kernel"] == _lib.HC_KERNEL_SIMT_EXACT
    want = ref.batched_matmul(2, a, False, b, True, False, 9, 33, 7, library_fast_path=False)
    assert np.array_equal(got.view(np.uint32), np.asarray(want).reshape(-1).view(np.uint32))


def test_group_creation_rejects_bad_requests_without_waiting_for_anyone(be):
    """Misuse is answered on the spot with a status code: nothing is sent to NCCL, nobody is
    waited for, the context keeps working."""
    from honeycrisp_b200 import _lib
    lib = be._lib
    g = ctypes.c_void_p()
    ident = ctypes.create_string_buffer(128)
    assert lib.hc_group_init(be._ctx, 9, 0, ident, ctypes.byref(g)) == _lib.HC_ERR_INVALID_ARGUMENT     # more than 8 ranks
    assert lib.hc_group_init(be._ctx, 2, 2, ident, ctypes.byref(g)) == _lib.HC_ERR_INVALID_ARGUMENT     # rank outside the group
    assert lib.hc_group_init(be._ctx, 2, 0, None, ctypes.byref(g)) == _lib.HC_ERR_INVALID_ARGUMENT      # no id for a real group
    assert lib.hc_group_init(be._ctx, 0, 0, None, ctypes.byref(g)) == _lib.HC_ERR_INVALID_ARGUMENT
    assert not g.value
    assert lib.hc_group_barrier(None) == _lib.HC_ERR_INVALID_ARGUMENT
    assert lib.hc_matmul_nsplit_allgather(None, 0, None, 0, None, 0, 1, 1, 1, None, 0) == _lib.HC_ERR_INVALID_ARGUMENT
    out = be.matmul(np.ones((64, 64), np.float32), False, np.ones((64, 64), np.float32), False, False, 64, 64, 64,
                    np.float32).onCPU(np.float32)
    assert np.all(out == 64.0)

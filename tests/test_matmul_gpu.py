"""Parity of the CUDA path with the CPU oracle, through the C ABI (needs a B200)."""
import threading

import numpy as np
import pytest

from helpers import FLAG_COMBOS, golden, logical_out, random_operands, stored
from oracle import reference_cpu as ref

pytestmark = pytest.mark.gpu

G = golden()


@pytest.fixture(scope="module")
def be():
    from honeycrisp_b200 import CUDABackend
    b = CUDABackend(0)
    yield b
    b.checkDeviceStatus()
    b.close()


def K():
    from honeycrisp_b200 import _lib
    return _lib


def run(be, count, A, B, ta, tb, to, dtype, kernel=0):
    rows, inner, cols = A.shape[-2], A.shape[-1], B.shape[-1]
    a_st, b_st = stored(A, ta), stored(B, tb)
    out = be.batchedMatmul(count, a_st, ta, b_st, tb, to, rows, inner, cols, dtype, kernel=kernel)
    res = out.onCPU(dtype)[: count * rows * cols]
    be.checkDeviceStatus()
    return res, a_st, b_st


# ---- the reference's own tests, replayed through the Tensor-level mirror --------------------

@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("ta,tb,to", FLAG_COMBOS)
def test_matrix_matrix_product(be, ta, tb, to, dtype):
    """BackendTests.swift:684-712: exact output and both gradients for all eight flag triples."""
    from honeycrisp_b200 import Tensor, matmul
    v = G["matrix_matrix_product"]
    x = np.array(v["x"], dtype=dtype).reshape(v["x_shape"])
    y = np.array(v["y_before_t"], dtype=dtype).reshape(v["y_before_t_shape"]).T
    g = np.array(v["out_grad"], dtype=dtype).reshape(v["out_shape"])
    a = Tensor.fromHost(be, stored(x, ta), stored(x, ta).shape, dtype).onGrad()
    b = Tensor.fromHost(be, stored(y, tb), stored(y, tb).shape, dtype).onGrad()
    sub = matmul(a, ta, b, tb, to)
    out = sub.numpy().T if to else sub.numpy()
    assert list(out.shape) == [2, 4]
    np.testing.assert_array_equal(out.reshape(-1).astype(np.float64), v["out"])
    sub.backward(Tensor.fromHost(be, stored(g, to), stored(g, to).shape, dtype))
    a_grad = a.grad.numpy().T if ta else a.grad.numpy()
    b_grad = b.grad.numpy().T if tb else b.grad.numpy()
    np.testing.assert_array_equal(a_grad.reshape(-1).astype(np.float64), v["a_grad"])
    np.testing.assert_array_equal(b_grad.reshape(-1).astype(np.float64), v["b_grad"])


@pytest.mark.parametrize("kernel", [0, 1, 2, 3])
def test_ones_product_and_half_overflow(be, kernel):
    """BackendTests.swift:713-725; every kernel, including the 3xTF32 path (small integers
    split exactly, so 128 must come out exactly)."""
    v = G["ones_product"]
    a = np.ones(v["a_shape"], dtype=np.float32)
    b = np.ones(v["b_shape"], dtype=np.float32)
    z = be.matmul(a, False, b, False, False, 64, 128, 32, np.float32, kernel=kernel).onCPU(np.float32)
    np.testing.assert_array_equal(z, np.full(64 * 32, v["value"], dtype=np.float32))
    small = be.matmul(a.astype(np.float16), False, b.astype(np.float16), False, False, 64, 128, 32, np.float16,
                      kernel=kernel).onCPU(np.float16)
    assert np.isfinite(small.astype(np.float32).sum())
    s = v["overflow_scale"]
    big = be.matmul((a * s).astype(np.float16), False, (b * s).astype(np.float16), False, False, 64, 128, 32,
                    np.float16, kernel=kernel).onCPU(np.float16)
    assert not np.isfinite(big.astype(np.float32).sum())
    assert np.all(np.isposinf(big.astype(np.float32)))


def test_matrix_vector_product(be):
    """BackendTests.swift:769-783."""
    from honeycrisp_b200 import Tensor, matmul
    v = G["matrix_vector_product"]
    x = Tensor.fromHost(be, v["x"], v["x_shape"], np.float32).onGrad()
    y = Tensor.fromHost(be, v["y"], v["y_shape"], np.float32).onGrad()
    product = matmul(x, False, y, False, False)
    np.testing.assert_array_equal(product.numpy().reshape(-1), np.array(v["out"], dtype=np.float32))
    product.backward(Tensor.fromHost(be, np.ones((2, 1)), [2, 1], np.float32))
    np.testing.assert_array_equal(x.grad.numpy().reshape(-1), np.array(v["x_grad"], dtype=np.float32))
    assert x.grad.shape == v["x_shape"]
    np.testing.assert_array_equal(y.grad.numpy().reshape(-1), np.array(v["y_grad"], dtype=np.float32))
    assert y.grad.shape == v["y_shape"]


@pytest.mark.parametrize("dtype,eps", [(np.float32, 1e-4), (np.float16, 1e-2)])
@pytest.mark.parametrize("ta,tb,to", FLAG_COMBOS)
def test_batched_matmul_matches_single(be, ta, tb, to, dtype, eps):
    """BackendTests.swift:728-767: batched output and both gradients against per-matrix products."""
    from honeycrisp_b200 import Tensor, batchedMatmul, matmul
    A, B = random_operands(7, 3, 2, 3, 4, dtype, dist="uniform01")
    Gr = np.random.default_rng(8).random((3, 2, 4)).astype(dtype)
    a = Tensor.fromHost(be, stored(A, ta), stored(A, ta).shape, dtype).onGrad()
    b = Tensor.fromHost(be, stored(B, tb), stored(B, tb).shape, dtype).onGrad()
    pre = batchedMatmul(a, ta, b, tb, to)
    pre.backward(Tensor.fromHost(be, stored(Gr, to), stored(Gr, to).shape, dtype))
    out = pre.numpy()
    for i in range(3):
        ai = Tensor.fromHost(be, stored(A[i], ta), stored(A[i], ta).shape, dtype).onGrad()
        bi = Tensor.fromHost(be, stored(B[i], tb), stored(B[i], tb).shape, dtype).onGrad()
        single = matmul(ai, ta, bi, tb, to)
        single.backward(Tensor.fromHost(be, stored(Gr[i], to), stored(Gr[i], to).shape, dtype))
        np.testing.assert_allclose(single.numpy().astype(np.float32), out[i].astype(np.float32), atol=eps, rtol=eps)
        np.testing.assert_allclose(ai.grad.numpy().astype(np.float32), a.grad.numpy()[i].astype(np.float32), atol=eps, rtol=eps)
        np.testing.assert_allclose(bi.grad.numpy().astype(np.float32), b.grad.numpy()[i].astype(np.float32), atol=eps, rtol=eps)


def test_concurrent_products_from_many_threads(be):
    """HoneycrispTests.swift:847-871: 100 concurrent [128,16]x[16,1] products + backward passes."""
    from honeycrisp_b200 import Tensor, matmul
    v = G["concurrent_backward"]
    rng = np.random.default_rng(3)
    A = rng.standard_normal(v["a_shape"]).astype(np.float32)
    Bv = rng.standard_normal(v["b_shape"]).astype(np.float32)
    expect = ref.matmul(A, False, Bv, False, False, 128, 16, 1, library_fast_path=False)
    results, errors = [None] * v["count"], []

    def work(i):
        try:
            a = Tensor.fromHost(be, A, A.shape, np.float32).onGrad()
            b = Tensor.fromHost(be, Bv, Bv.shape, np.float32).onGrad()
            out = matmul(a, False, b, False, False, kernel=K().HC_KERNEL_SIMT_EXACT)
            out.backward(Tensor.fromHost(be, np.ones((128, 1)), [128, 1], np.float32))
            results[i] = (out.numpy().reshape(-1), a.grad.numpy(), b.grad.numpy())
        except Exception as e:  # pragma: no cover
            errors.append(e)

    threads = [threading.Thread(target=work, args=(i,)) for i in range(v["count"])]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors
    for out, ga, gb in results:
        assert np.array_equal(out, expect)
        assert np.array_equal(ga, results[0][1]) and np.array_equal(gb, results[0][2])


# ---- bit-exact parity of the CUDA-core kernel with the reference CPU loop ------------------

SHAPES_SMALL = [(1, 1, 1, 1), (2, 3, 4, 1), (7, 5, 3, 2), (64, 128, 32, 1), (129, 65, 130, 3), (300, 17, 7, 2),
                (33, 257, 31, 1), (128, 16, 1, 4), (1, 40, 200, 1)]


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("shape", SHAPES_SMALL)
def test_exact_kernel_is_bit_identical_to_cpu_loop(be, shape, dtype):
    M, Kd, N, cnt = shape
    for (ta, tb, to) in FLAG_COMBOS:
        A, B = random_operands(M * 131 + N, cnt, M, Kd, N, dtype)
        res, a_st, b_st = run(be, cnt, A, B, ta, tb, to, dtype, kernel=K().HC_KERNEL_SIMT_EXACT)
        orc = ref.batched_matmul(cnt, a_st, ta, b_st, tb, to, M, Kd, N, library_fast_path=False)
        assert np.array_equal(res.view(np.uint8), orc.view(np.uint8)), (shape, ta, tb, to)


@pytest.mark.parametrize("shape", SHAPES_SMALL)
def test_fused_kernel_is_bit_identical_for_half(be, shape):
    """Products of two halves are exact in float32, so fusing the multiply-add changes nothing."""
    M, Kd, N, cnt = shape
    for (ta, tb, to) in [(False, False, False), (True, True, True), (False, True, False)]:
        A, B = random_operands(M + N, cnt, M, Kd, N, np.float16)
        res, a_st, b_st = run(be, cnt, A, B, ta, tb, to, np.float16, kernel=K().HC_KERNEL_SIMT)
        orc = ref.batched_matmul(cnt, a_st, ta, b_st, tb, to, M, Kd, N)
        assert np.array_equal(res.view(np.uint16), orc.view(np.uint16))


def test_float32_plain_product_against_host_sgemm(be):
    """The one case the reference sends to a library GEMM (BackendCPU.swift:1256): agreement
    with the host sgemm stand-in within 1e-5 relative Frobenius error, all kernels."""
    A, B = random_operands(0, 1, 256, 512, 384, np.float32, dist="uniform01")
    host = ref.matmul(A, False, B, False, False, 256, 512, 384, library_fast_path=True)
    for kernel in (0, 1, 2, 3):
        res, _, _ = run(be, 1, A, B, False, False, False, np.float32, kernel=kernel)
        assert ref.rel_frobenius(res, host) < 1e-5, kernel


# ---- edge cases -----------------------------------------------------------------------------

def test_empty_dimensions(be):
    for dtype in (np.float32, np.float16):
        z = be.matmul(np.zeros((3, 0), dtype), False, np.zeros((0, 4), dtype), False, False, 3, 0, 4, dtype)
        assert np.all(z.onCPU(dtype)[:12] == 0)           # empty contraction sums to +0
        z = be.matmul(np.zeros((0, 5), dtype), False, np.zeros((5, 4), dtype), False, False, 0, 5, 4, dtype)
        assert z.byteCount == 0 and z.ptr != 0            # max(1, byteCount) allocation, no launch
        z = be.batchedMatmul(0, np.zeros((0,), dtype), False, np.zeros((0,), dtype), False, False, 4, 5, 6, dtype)
        assert z.byteCount == 0


def test_int64_is_not_implemented(be):
    from honeycrisp_b200 import DType, NotImplementedByBackend
    with pytest.raises(NotImplementedByBackend):
        be.matmul(np.zeros(4, np.int64), False, np.zeros(4, np.int64), False, False, 2, 2, 2, DType.int64)


def test_undersized_operand_is_rejected(be):
    with pytest.raises(ValueError):
        be.matmul(np.zeros(5, np.float32), False, np.zeros(6, np.float32), False, False, 2, 3, 2, np.float32)


def test_misaligned_operands_are_repacked_for_the_tensor_cores(be):
    """Leading dimensions that are not 16-byte multiples (and an operand at an odd address) cannot
    be described to TMA; the operands are copied once into the aligned work area and the product
    still runs on the tensor cores, in every flag combination and both dtypes."""
    for dtype, tol in ((np.float16, 2e-3), (np.float32, 1e-5)):
        for (ta, tb, to) in FLAG_COMBOS:
            A, B = random_operands(2, 2, 130, 67, 129, dtype)
            res, a_st, b_st = run(be, 2, A, B, ta, tb, to, dtype, kernel=K().HC_KERNEL_TENSOR)
            info = be.lastLaunchInfo()
            assert info["kernel"] == K().HC_KERNEL_TENSOR and info["scratch_bytes"] > 0
            orc = ref.batched_matmul(2, a_st, ta, b_st, tb, to, 130, 67, 129, library_fast_path=False)
            assert ref.rel_frobenius(res, orc) < tol, (dtype, ta, tb, to)
    # an operand that starts two bytes into an allocation
    A, B = random_operands(3, 1, 256, 128, 264, np.float16)
    raw = be.collection(np.concatenate([np.zeros(1, np.float16), A.reshape(-1)]), np.float16)
    shifted = be.wrap(raw.ptr + 2, A.size * 2, owner=raw)
    got = be.matmul(shifted, False, B.reshape(-1), False, False, 256, 128, 264, np.float16,
                    kernel=K().HC_KERNEL_TENSOR).onCPU(np.float16)[: 256 * 264]
    want = be.matmul(A.reshape(-1), False, B.reshape(-1), False, False, 256, 128, 264, np.float16,
                     kernel=K().HC_KERNEL_TENSOR).onCPU(np.float16)[: 256 * 264]
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    # the default dispatch sends tiny products to the CUDA-core kernel, bit-identical to the CPU loop
    A, B = random_operands(4, 1, 30, 17, 29, np.float16)
    res, a_st, b_st = run(be, 1, A, B, False, False, False, np.float16, kernel=0)
    assert be.lastLaunchInfo()["kernel"] == K().HC_KERNEL_SIMT_EXACT
    assert np.array_equal(res.view(np.uint16), ref.matmul(a_st, False, b_st, False, False, 30, 17, 29).view(np.uint16))


def test_host_buffer_entry_point(be):
    A, B = random_operands(9, 2, 96, 160, 72, np.float16)
    out = be.batchedMatmulHost(2, stored(A, False), False, stored(B, True), True, False, 96, 160, 72, np.float16)
    f64 = ref.batched_matmul_f64(2, stored(A, False), False, stored(B, True), True, False, 96, 160, 72)
    assert ref.rel_frobenius(out, f64) < 2e-3
    orc = ref.batched_matmul(2, stored(A, False), False, stored(B, True), True, False, 96, 160, 72)
    assert ref.rel_frobenius(out, orc) < 1e-3


def test_run_to_run_determinism(be):
    A, B = random_operands(4, 2, 384, 512, 640, np.float16)
    first, _, _ = run(be, 2, A, B, False, True, False, np.float16)
    for _ in range(3):
        again, _, _ = run(be, 2, A, B, False, True, False, np.float16)
        assert np.array_equal(first.view(np.uint16), again.view(np.uint16))


def test_bounded_wait_expires_and_context_stays_usable(be):
    """Failure detection without a fault: a wait that nothing satisfies gives up after its
    limit, the host sees HC_ERR_TIMEOUT once, and the same context keeps working."""
    import time
    from honeycrisp_b200 import DeviceTimeout, _lib
    lib = _lib.load()
    be.checkDeviceStatus()                                   # clean before
    t0 = time.perf_counter()
    assert lib.hc_selftest_bounded_wait(be._ctx, 20) == _lib.HC_OK
    with pytest.raises(DeviceTimeout):
        be.checkDeviceStatus()
    assert 0.015 < time.perf_counter() - t0 < 2.0
    be.checkDeviceStatus()                                   # the status word was cleared
    A, B = random_operands(1, 1, 256, 128, 256, np.float16)
    res, a_st, b_st = run(be, 1, A, B, False, True, False, np.float16, kernel=K().HC_KERNEL_TENSOR)
    f64 = ref.batched_matmul_f64(1, a_st, False, b_st, True, False, 256, 128, 256)
    assert ref.rel_frobenius(res, f64) < 2e-3


def test_pipelined_host_products_equal_the_blocking_form(be):
    """Five products in flight through the two-slot pipeline, different shapes and dtypes; each
    result equals the blocking host call bit for bit."""
    cases = [(np.float16, 2, 96, 160, 72, False, True), (np.float32, 1, 256, 128, 384, False, False),
             (np.float16, 1, 384, 256, 512, True, False), (np.float16, 3, 64, 64, 64, True, True),
             (np.float32, 1, 130, 67, 129, False, False)]
    want, outs, keep = [], [], []
    for i, (dt, cnt, M, Kd, N, ta, tb) in enumerate(cases):
        A, B = random_operands(20 + i, cnt, M, Kd, N, dt)
        a_st, b_st = stored(A, ta), stored(B, tb)
        keep.append((a_st, b_st))
        want.append(be.batchedMatmulHost(cnt, a_st, ta, b_st, tb, False, M, Kd, N, dt).copy())
    for (dt, cnt, M, Kd, N, ta, tb), (a_st, b_st) in zip(cases, keep):
        outs.append(be.batchedMatmulHost(cnt, a_st, ta, b_st, tb, False, M, Kd, N, dt, asynchronous=True))
    be.hostSync()
    be.checkDeviceStatus()
    for w, o in zip(want, outs):
        assert np.array_equal(w.view(np.uint8), o.view(np.uint8))


def test_argument_errors_come_back_as_status_codes(be):
    """Misuse never aborts: the reference traps these with #alwaysAssert before the backend; the
    library reports them."""
    import ctypes
    from honeycrisp_b200 import _lib
    lib = _lib.load()
    buf = be.allocate(64)
    c = be._ctx
    assert lib.hc_matmul(c, _lib.HC_F32, buf.ptr, 0, buf.ptr, 0, 0, -1, 2, 2, buf.ptr) == _lib.HC_ERR_INVALID_ARGUMENT
    assert lib.hc_matmul(c, _lib.HC_F32, None, 0, buf.ptr, 0, 0, 2, 2, 2, buf.ptr) == _lib.HC_ERR_INVALID_ARGUMENT
    assert lib.hc_matmul(c, 7, buf.ptr, 0, buf.ptr, 0, 0, 2, 2, 2, buf.ptr) == _lib.HC_ERR_NOT_IMPLEMENTED
    big = 1 << 40
    assert lib.hc_matmul(c, _lib.HC_F32, buf.ptr, 0, buf.ptr, 0, 0, big, big, big, buf.ptr) == _lib.HC_ERR_INVALID_ARGUMENT
    assert lib.hc_batched_matmul_ex(c, 9, _lib.HC_F32, 1, buf.ptr, 0, buf.ptr, 0, 0, 2, 2, 2, buf.ptr) == _lib.HC_ERR_INVALID_ARGUMENT
    assert lib.hc_matmul_colblock(c, 0, _lib.HC_F32, buf.ptr, 0, buf.ptr, 0, 0, 2, 2, 2, 1, 2, buf.ptr) == _lib.HC_ERR_INVALID_ARGUMENT
    assert b"column block" in lib.hc_last_error(c)
    p = ctypes.c_void_p()
    assert lib.hc_alloc(c, 1 << 60, ctypes.byref(p)) == _lib.HC_ERR_ALLOCATION_FAILED and not p.value
    be.checkDeviceStatus()
    # and the context still works
    z = be.matmul(np.ones((2, 2), np.float32), False, np.ones((2, 2), np.float32), False, False, 2, 2, 2, np.float32)
    assert z.onCPU(np.float32)[:4].tolist() == [2, 2, 2, 2]


def test_two_contexts_and_stream_switching(be):
    """A second context on the same device, and a context moved between streams, give the same
    bits as the module's context."""
    import torch
    from honeycrisp_b200 import CUDABackend
    A, B = random_operands(31, 1, 512, 256, 768, np.float32)
    want, _, _ = run(be, 1, A, B, False, False, False, np.float32, kernel=K().HC_KERNEL_TENSOR)
    other = CUDABackend(0)
    try:
        for _ in range(2):
            s = torch.cuda.Stream()
            other.useStream(s.cuda_stream)
            got, _, _ = run(other, 1, A, B, False, False, False, np.float32, kernel=K().HC_KERNEL_TENSOR)
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
            other.useStream(None)
            got, _, _ = run(other, 1, A, B, False, False, False, np.float32, kernel=K().HC_KERNEL_TENSOR)
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    finally:
        other.close()


def test_results_may_outlive_their_backend():
    """A host with garbage collection releases result buffers late: after the backend that made
    them is closed.  That must neither crash nor leave an error behind for the next context."""
    from honeycrisp_b200 import CUDABackend
    A, B = random_operands(5, 1, 256, 256, 256, np.float16)
    results = []
    for _ in range(2):
        be = CUDABackend(0)
        out = be.matmul(stored(A, False), False, stored(B, False), False, False, 256, 256, 256, np.float16)
        results.append(out.onCPU(np.float16).copy())
        be.checkDeviceStatus()
        be.close()
        with pytest.raises(Exception):
            out.wait()
        del out   # its completion marker is destroyed after the context
    assert np.array_equal(results[0], results[1])


def test_async_read_back_while_later_products_run(be):
    """readInto copies a result on a side stream after the work enqueued so far; products issued
    afterwards do not wait for it, and the bytes equal a blocking read."""
    import torch
    A, B = random_operands(21, 1, 512, 384, 640, np.float16)
    a_st, b_st = stored(A, False), stored(B, False)
    outs = [be.matmul(a_st, False, b_st, False, to, 512, 384, 640, np.float16) for to in (False, True)]
    hosts = [torch.empty(512 * 640, dtype=torch.float16).pin_memory().numpy() for _ in outs]
    reads = [o.readInto(h) for o, h in zip(outs, hosts)]
    later = be.matmul(a_st, False, b_st, False, False, 512, 384, 640, np.float16)   # enqueued behind the reads
    for r, o in zip(reads, outs):
        got = r.wait()
        assert np.array_equal(got.view(np.uint16), o.onCPU(np.float16)[: 512 * 640].view(np.uint16))
    assert np.array_equal(later.onCPU(np.float16).view(np.uint16), outs[0].onCPU(np.float16).view(np.uint16))
    with pytest.raises(ValueError):
        outs[0].readInto(np.zeros(512 * 640 + 8, dtype=np.float16))


def test_async_upload_ordered_by_a_device_side_wait(be):
    """writeFrom copies on a side stream; enqueueWait makes the product that reads the buffer
    wait for it on the device.  Repeated with changing contents, so a product that ran ahead of
    its upload would be caught."""
    import torch
    M, Kd, N = 256, 192, 320
    da, db = be.allocate(M * Kd * 2), be.allocate(Kd * N * 2)
    ha = torch.empty(M * Kd, dtype=torch.float16).pin_memory().numpy()
    hb = torch.empty(Kd * N, dtype=torch.float16).pin_memory().numpy()
    for seed in range(4):
        A, B = random_operands(seed, 1, M, Kd, N, np.float16)
        ha[:] = A.reshape(-1); hb[:] = B.reshape(-1)
        ups = [da.writeFrom(ha), db.writeFrom(hb)]
        for u in ups:
            be.enqueueWait(u)
        out = be.matmul(da, False, db, False, False, M, Kd, N, np.float16)
        res = out.onCPU(np.float16)[: M * N]
        for u in ups:
            u.wait()                                  # the pinned arrays are rewritten next round
        want = ref.batched_matmul(1, stored(A, False), False, stored(B, False), False, False, M, Kd, N)
        assert ref.rel_frobenius(res, want) < 1e-3, seed

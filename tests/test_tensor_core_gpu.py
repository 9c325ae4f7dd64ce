"""The tcgen05 kernels against the oracle, a float64 product and the exact CUDA-core kernel."""
import numpy as np
import pytest

from helpers import FLAG_COMBOS, logical_out, random_operands, stored
from oracle import reference_cpu as ref

pytestmark = pytest.mark.gpu

# Tolerances of the contract: float16 within 2e-3 relative Frobenius error of a float64 product,
# float32 within 1e-5 of the reference's float32 result.
TOL_F16 = 2e-3
TOL_F32 = 1e-5


@pytest.fixture(scope="module")
def be():
    from honeycrisp_b200 import CUDABackend
    b = CUDABackend(0)
    yield b
    b.checkDeviceStatus()
    b.close()


def TENSOR():
    from honeycrisp_b200 import _lib
    return _lib.HC_KERNEL_TENSOR


def run(be, count, A, B, ta, tb, to, dtype, kernel):
    rows, inner, cols = A.shape[-2], A.shape[-1], B.shape[-1]
    a_st, b_st = stored(A, ta), stored(B, tb)
    out = be.batchedMatmul(count, a_st, ta, b_st, tb, to, rows, inner, cols, dtype, kernel=kernel)
    res = out.onCPU(dtype)[: count * rows * cols]
    be.checkDeviceStatus()
    return res, a_st, b_st


# (M, K, N, count): single tile, one and several CTA pairs, ragged edges in every dimension,
# narrow (128-column tile), batched, more tiles than SMs.
SHAPES = [(128, 64, 256, 1), (256, 64, 256, 1), (128, 64, 128, 1), (256, 256, 512, 1), (200, 136, 328, 2),
          (1000, 520, 776, 3), (136, 72, 264, 3), (1024, 1024, 1024, 1), (384, 8, 96, 2), (2048, 128, 2048, 4),
          (5000, 64, 1032, 1)]


@pytest.mark.parametrize("shape", SHAPES)
def test_half_all_flag_combinations(be, shape):
    M, Kd, N, cnt = shape
    for (ta, tb, to) in FLAG_COMBOS:
        A, B = random_operands(M + Kd + N, cnt, M, Kd, N, np.float16)
        res, a_st, b_st = run(be, cnt, A, B, ta, tb, to, np.float16, TENSOR())
        f64 = ref.batched_matmul_f64(cnt, a_st, ta, b_st, tb, to, M, Kd, N)
        assert ref.rel_frobenius(res, f64) < TOL_F16, (shape, ta, tb, to)
        if M * N * Kd * cnt <= 64 * 1024 * 1024:
            # against the reference CPU loop itself: same float32 accumulation, different order
            orc = ref.batched_matmul(cnt, a_st, ta, b_st, tb, to, M, Kd, N)
            assert ref.rel_frobenius(res, orc) < 1e-3, (shape, ta, tb, to)


@pytest.mark.parametrize("shape", [(128, 32, 256, 1), (256, 32, 256, 1), (256, 256, 512, 1), (200, 132, 328, 2),
                                   (1000, 516, 776, 2), (1024, 1024, 1024, 1), (384, 4, 96, 2)])
@pytest.mark.parametrize("dist", ["uniform01", "uniform11"])
def test_float_split_product_all_flag_combinations(be, shape, dist):
    M, Kd, N, cnt = shape
    for (ta, tb, to) in FLAG_COMBOS:
        A, B = random_operands(M + Kd + N, cnt, M, Kd, N, np.float32, dist=dist)
        res, a_st, b_st = run(be, cnt, A, B, ta, tb, to, np.float32, TENSOR())
        f64 = ref.batched_matmul_f64(cnt, a_st, ta, b_st, tb, to, M, Kd, N)
        assert ref.rel_frobenius(res, f64) < TOL_F32, (shape, ta, tb, to)
        if M * N * Kd * cnt <= 64 * 1024 * 1024:
            orc = ref.batched_matmul(cnt, a_st, ta, b_st, tb, to, M, Kd, N)   # the reference's own float32 result
            assert ref.rel_frobenius(res, orc) < TOL_F32, (shape, ta, tb, to)


def test_half_small_integers_are_exact(be):
    """Sums of small-integer products are exact in float32 whatever the order: the tensor-core
    result must equal the CPU loop bit for bit."""
    A, B = random_operands(5, 2, 304, 200, 264, np.float16, dist="smallint")
    for (ta, tb, to) in FLAG_COMBOS:
        res, a_st, b_st = run(be, 2, A, B, ta, tb, to, np.float16, TENSOR())
        orc = ref.batched_matmul(2, a_st, ta, b_st, tb, to, 304, 200, 264)
        assert np.array_equal(res.view(np.uint16), orc.view(np.uint16)), (ta, tb, to)


def test_float_small_integers_are_exact(be):
    A, B = random_operands(6, 1, 260, 132, 520, np.float32, dist="smallint")
    for (ta, tb, to) in FLAG_COMBOS:
        res, a_st, b_st = run(be, 1, A, B, ta, tb, to, np.float32, TENSOR())
        orc = ref.batched_matmul(1, a_st, ta, b_st, tb, to, 260, 132, 520, library_fast_path=False)
        assert np.array_equal(res.view(np.uint32), orc.view(np.uint32)), (ta, tb, to)


def test_float_non_finite_values_propagate(be):
    A, B = random_operands(7, 1, 128, 64, 256, np.float32)
    A[0, 3, 5] = np.inf
    B[0, 9, 17] = np.nan
    res, _, _ = run(be, 1, A, B, False, False, False, np.float32, TENSOR())
    C = res.reshape(128, 256)
    assert np.all(np.isnan(C[:, 17]))
    assert np.all(np.isinf(C[3, :17]) | np.isnan(C[3, :17]))
    good = np.delete(np.delete(C, 3, axis=0), 17, axis=1)
    assert np.all(np.isfinite(good))


def test_long_contraction_keeps_float32_accuracy(be):
    """K = 16384 (the largest configured contraction): the windowed accumulation keeps the
    error flat in K."""
    A, B = random_operands(8, 1, 256, 16384, 256, np.float32, dist="uniform01")
    res, a_st, b_st = run(be, 1, A, B, False, False, False, np.float32, TENSOR())
    f64 = ref.batched_matmul_f64(1, a_st, False, b_st, False, False, 256, 16384, 256)
    assert ref.rel_frobenius(res, f64) < TOL_F32 / 2


def test_column_block_equals_columns_of_full_product(be):
    """hc_matmul_colblock: bitwise equal to the same columns of the one-device product."""
    from honeycrisp_b200 import _lib
    for dtype, trans in ((np.float16, (False, True)), (np.float16, (False, False)), (np.float32, (False, False)),
                         (np.float16, (True, False))):
        ta, tb = trans
        M, Kd, N = 512, 256, 1024
        A, B = random_operands(10, 1, M, Kd, N, dtype)
        full, a_st, b_st = run(be, 1, A, B, ta, tb, False, dtype, TENSOR())
        for to in (False, True):
            full_t = np.ascontiguousarray(full.reshape(M, N).T).reshape(-1) if to else full
            out = be.allocate(M * N * np.dtype(dtype).itemsize)
            for (b0, cnt) in ((0, 256), (256, 512), (768, 256)):
                be.matmulColumnBlock(a_st, ta, b_st, tb, to, M, Kd, N, b0, cnt, dtype, out=out,
                                     kernel=_lib.HC_KERNEL_TENSOR)
            got = out.onCPU(dtype)[: M * N]
            if dtype == np.float32 and to:
                # A transposed output swaps the operand roles, and with them the order in which
                # the two small split products (lo*hi, hi*lo) enter the truncating accumulator.
                assert ref.rel_frobenius(got, full_t) < 1e-6, (dtype, trans, to)
            else:
                assert np.array_equal(got.view(np.uint8), full_t.view(np.uint8)), (dtype, trans, to)


@pytest.mark.parametrize("flags", [(False, True, False), (False, False, False), (True, False, False), (True, True, False)])
def test_config2_shape_properties(be, flags):
    """float16 8192^3 (the headline configuration), checked through properties that need no
    full-size CPU product: sampled rows and columns against float64, and bitwise equality of a
    row block computed as its own smaller product."""
    import torch
    ta, tb, to = flags
    n = 8192
    gen = torch.Generator(device="cuda").manual_seed(1)
    a = (torch.randn((n, n), generator=gen, device="cuda") / n ** 0.5).half()
    b = (torch.randn((n, n), generator=gen, device="cuda") / n ** 0.5).half()
    out = torch.empty((n, n), device="cuda", dtype=torch.float16)
    torch.cuda.synchronize()
    od = be.wrap(out.data_ptr(), out.numel() * 2, out)
    be.matmul(a, ta, b, tb, to, n, n, n, np.float16, out=od)
    be.sync()
    be.checkDeviceStatus()
    A = (a.t() if ta else a)
    Bm = (b.t() if tb else b)
    rows = torch.randint(0, n, (64,), generator=torch.Generator().manual_seed(2)).cuda()
    ref_rows = (A[rows].double() @ Bm.double()).cpu().numpy()
    got_rows = out[rows].float().cpu().numpy()
    assert ref.rel_frobenius(got_rows, ref_rows) < TOL_F16
    cols = torch.randint(0, n, (64,), generator=torch.Generator().manual_seed(3)).cuda()
    ref_cols = (A.double() @ Bm[:, cols].double()).cpu().numpy()
    got_cols = out[:, cols].float().cpu().numpy()
    assert ref.rel_frobenius(got_cols, ref_cols) < TOL_F16

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


@pytest.fixture(scope="module")
def dbe():
    """A context on the diagnostics build of the library, where HC_TC_SHAPE / HC_TC_SPLITS force
    the planner's choices (read at every launch); the shipped library has no such switches."""
    from honeycrisp_b200 import CUDABackend
    b = CUDABackend(0, diagnostics=True)
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
          (5000, 64, 1032, 1),
          # long contractions over wide products take the 256 x 512 tiles: ragged in every dimension, batched
          (304, 3080, 1096, 2), (1024, 4096, 1024, 1)]


@pytest.mark.parametrize("shape", SHAPES)
def test_half_all_flag_combinations(be, shape):
    M, Kd, N, cnt = shape
    for (ta, tb, to) in FLAG_COMBOS:
        A, B = random_operands(M + Kd + N, cnt, M, Kd, N, np.float16)
        res, a_st, b_st = run(be, cnt, A, B, ta, tb, to, np.float16, TENSOR())
        f64 = ref.batched_matmul_f64(cnt, a_st, ta, b_st, tb, to, M, Kd, N)
        assert ref.rel_frobenius(res, f64) < TOL_F16, (shape, ta, tb, to)
        if M * N * Kd * cnt <= 64 * 1024 * 1024 or (ta, tb, to) == (False, True, False):
            # against the reference CPU loop itself: same float32 accumulation, different order
            orc = ref.batched_matmul(cnt, a_st, ta, b_st, tb, to, M, Kd, N)
            assert ref.rel_frobenius(res, orc) < 1e-3, (shape, ta, tb, to)


# HC_TC_SHAPE forces one of the six float16 tile shapes (read at every launch) where the product
# admits it; AUTO picks among them by cost, so each needs its own parity run.
TILE_SHAPES = {1: (256, 512), 2: (256, 256), 3: (128, 256), 4: (128, 128), 5: (256, 128), 6: (256, 64)}


@pytest.mark.parametrize("forced", sorted(TILE_SHAPES))
def test_half_every_tile_shape(dbe, forced, monkeypatch):
    be = dbe
    monkeypatch.setenv("HC_TC_SHAPE", str(forced))
    M, Kd, N, cnt = 520, 2056, 1096, 2   # ragged in every dimension, long enough for the 512-wide tiles
    used = set()
    for (ta, tb, to) in FLAG_COMBOS:
        A, B = random_operands(forced, cnt, M, Kd, N, np.float16)
        res, a_st, b_st = run(be, cnt, A, B, ta, tb, to, np.float16, TENSOR())
        info = be.lastLaunchInfo()
        used.add((info["tile_m"], info["tile_n"]))
        f64 = ref.batched_matmul_f64(cnt, a_st, ta, b_st, tb, to, M, Kd, N)
        assert ref.rel_frobenius(res, f64) < TOL_F16, (forced, ta, tb, to, info)
    assert TILE_SHAPES[forced] in used, (forced, used)


@pytest.mark.parametrize("forced", [2, 3, 4, 5, 6])
def test_float_every_tile_shape(dbe, forced, monkeypatch):
    be = dbe
    monkeypatch.setenv("HC_TC_SHAPE", str(forced))
    monkeypatch.setenv("HC_TC_SPLITS", "1")
    M, Kd, N, cnt = 520, 264, 1096, 2
    used = set()
    for (ta, tb, to) in FLAG_COMBOS:
        A, B = random_operands(forced, cnt, M, Kd, N, np.float32, dist="uniform11")
        res, a_st, b_st = run(be, cnt, A, B, ta, tb, to, np.float32, TENSOR())
        info = be.lastLaunchInfo()
        used.add((info["tile_m"], info["tile_n"]))
        f64 = ref.batched_matmul_f64(cnt, a_st, ta, b_st, tb, to, M, Kd, N)
        assert ref.rel_frobenius(res, f64) < TOL_F32, (forced, ta, tb, to, info)
    assert TILE_SHAPES[forced] in used, (forced, used)


def test_half_small_products_take_small_pair_tiles(be):
    # one wave either way: the smaller shape spreads it over more SMs
    for (n, tile) in [(512, (256, 64)), (1536, (256, 128)), (2048, (256, 256))]:
        A, B = random_operands(n, 1, n, n, n, np.float16)
        res, a_st, b_st = run(be, 1, A, B, False, True, False, np.float16, TENSOR())
        info = be.lastLaunchInfo()
        assert (info["tile_m"], info["tile_n"]) == tile, (n, info)
        f64 = ref.batched_matmul_f64(1, a_st, False, b_st, True, False, n, n, n)
        assert ref.rel_frobenius(res, f64) < TOL_F16


# Few outputs and a long contraction (the weight gradient of a small Linear layer): the
# contraction is cut into parts that run as separate tiles into float32 partial matrices, summed
# in ascending order by a second kernel.
CUT_SHAPES = [(512, 4096, 512, 1), (264, 8200, 328, 3), (128, 4096, 256, 1), (1024, 16384, 1024, 1),
              (520, 4104, 72, 2)]


@pytest.mark.parametrize("shape", CUT_SHAPES)
def test_half_cut_contraction(be, shape):
    M, Kd, N, cnt = shape
    for (ta, tb, to) in FLAG_COMBOS:
        A, B = random_operands(M + N, cnt, M, Kd, N, np.float16, scale=0.25)
        res, a_st, b_st = run(be, cnt, A, B, ta, tb, to, np.float16, TENSOR())
        info = be.lastLaunchInfo()
        rows_t, cols_t = (N, M) if to else (M, N)
        whole_tiles = -(-rows_t // info["tile_m"]) * -(-cols_t // info["tile_n"]) * cnt
        assert info["tiles"] >= 2 * whole_tiles, (shape, ta, tb, to, info)   # it was cut
        f64 = ref.batched_matmul_f64(cnt, a_st, ta, b_st, tb, to, M, Kd, N)
        assert ref.rel_frobenius(res, f64) < TOL_F16, (shape, ta, tb, to, info)


@pytest.mark.parametrize("parts", [1, 2, 5, 16, 64])
def test_half_forced_cuts_agree(dbe, parts, monkeypatch):
    """HC_TC_SPLITS forces the number of parts (1: never cut).  Every cut gives the float64
    product within the float16 tolerance, and a result that float16 represents exactly
    (small integers) is identical whatever the cut."""
    be = dbe
    monkeypatch.setenv("HC_TC_SPLITS", str(parts))
    M, Kd, N = 264, 2120, 200
    A, B = random_operands(3, 1, M, Kd, N, np.float16, scale=0.25)
    res, a_st, b_st = run(be, 1, A, B, False, False, False, np.float16, TENSOR())
    f64 = ref.batched_matmul_f64(1, a_st, False, b_st, False, False, M, Kd, N)
    assert ref.rel_frobenius(res, f64) < TOL_F16, parts
    Ai, Bi = random_operands(4, 1, M, Kd, N, np.float16, dist="smallint")
    resi, ai, bi = run(be, 1, Ai, Bi, False, True, False, np.float16, TENSOR())
    exact = ref.batched_matmul_f64(1, ai, False, bi, True, False, M, Kd, N)
    assert np.array_equal(resi, exact.reshape(-1).astype(np.float16)), parts


@pytest.mark.parametrize("shape", [(512, 4096, 512, 1), (200, 2056, 136, 2), (128, 8192, 128, 1)])
def test_float_cut_contraction(be, shape):
    M, Kd, N, cnt = shape
    for (ta, tb, to) in FLAG_COMBOS:
        A, B = random_operands(M + N + 1, cnt, M, Kd, N, np.float32, dist="uniform11")
        res, a_st, b_st = run(be, cnt, A, B, ta, tb, to, np.float32, TENSOR())
        info = be.lastLaunchInfo()
        f64 = ref.batched_matmul_f64(cnt, a_st, ta, b_st, tb, to, M, Kd, N)
        assert ref.rel_frobenius(res, f64) < TOL_F32, (shape, ta, tb, to, info)


def test_column_block_of_cut_product_equals_whole(be):
    """A block planned as the whole product is cut the same way: bitwise the whole's columns."""
    from honeycrisp_b200 import _lib
    M, Kd, N = 384, 4096, 512
    for dtype in (np.float16, np.float32):
        A, B = random_operands(12, 1, M, Kd, N, dtype, scale=0.25)
        full, a_st, b_st = run(be, 1, A, B, False, True, False, dtype, TENSOR())
        out = be.allocate(M * N * np.dtype(dtype).itemsize)
        for (b0, cnt) in ((0, 128), (128, 256), (384, 128)):
            be.matmulColumnBlock(a_st, False, b_st, True, False, M, Kd, N, b0, cnt, dtype, out=out,
                                 kernel=_lib.HC_KERNEL_TENSOR)
        got = out.onCPU(dtype)[: M * N]
        assert np.array_equal(got.view(np.uint8), full.view(np.uint8)), dtype


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


# ---- the configured workloads at full size, through properties that need no CPU product ----

def _rel(x, r):
    return float((x.double() - r.double()).norm() / r.double().norm())


def test_config1_float32_1024_against_host_sgemm(be):
    """float32 1024^3, U[0,1), no flags: the one case the reference sends to its library GEMM;
    checked against the host sgemm stand-in within 1e-5 relative Frobenius error."""
    A, B = random_operands(0, 1, 1024, 1024, 1024, np.float32, dist="uniform01")
    host = ref.matmul(A, False, B, False, False, 1024, 1024, 1024, library_fast_path=True)
    res, _, _ = run(be, 1, A, B, False, False, False, np.float32, 0)
    from honeycrisp_b200 import _lib
    assert be.lastLaunchInfo()["kernel"] == _lib.HC_KERNEL_TENSOR
    assert ref.rel_frobenius(res, host) < TOL_F32


def test_config3_batched_scores_full_size(be):
    """float16 batched Q.K^T, 64 x [2048,128].[2048,128]^T: every matrix against a float64 product
    (on the device), and bitwise equality of a batch shard computed on its own."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(2)
    q = torch.randn((64, 2048, 128), generator=g, device="cuda").half()
    k = torch.randn((64, 2048, 128), generator=g, device="cuda").half()
    out = torch.empty((64, 2048, 2048), device="cuda", dtype=torch.float16)
    torch.cuda.synchronize()
    be.batchedMatmul(64, q, False, k, True, False, 2048, 128, 2048, np.float16,
                     out=be.wrap(out.data_ptr(), out.numel() * 2, out))
    be.sync()
    be.checkDeviceStatus()
    for i in range(0, 64, 8):
        want = q[i:i + 8].double() @ k[i:i + 8].double().transpose(1, 2)
        assert _rel(out[i:i + 8], want) < TOL_F16
    shard = torch.empty((8, 2048, 2048), device="cuda", dtype=torch.float16)
    be.batchedMatmul(8, q[16:24], False, k[16:24], True, False, 2048, 128, 2048, np.float16,
                     out=be.wrap(shard.data_ptr(), shard.numel() * 2, shard))
    be.sync()
    assert torch.equal(shard, out[16:24])


def test_config4_linear_triple_full_size(be):
    """Forward and both backward products of a Linear layer as autodiff issues them
    (Linalg.swift:73-80): Y = X.W^T, dX = dY.W, dW = (X^T.dY)^T, sampled rows against float64."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn((16384, 4096), generator=g, device="cuda").half()
    w = ((torch.rand((16384, 4096), generator=g, device="cuda") - 0.5) / 32).half()
    dy = torch.randn((16384, 16384), generator=g, device="cuda").half()
    y = torch.empty((16384, 16384), device="cuda", dtype=torch.float16)
    dx = torch.empty((16384, 4096), device="cuda", dtype=torch.float16)
    dw = torch.empty((16384, 4096), device="cuda", dtype=torch.float16)
    torch.cuda.synchronize()
    wrap = lambda t: be.wrap(t.data_ptr(), t.numel() * 2, t)
    be.matmul(x, False, w, True, False, 16384, 4096, 16384, np.float16, out=wrap(y))
    # the backward flag triples of a (transA=F, transB=T, transOut=F) product
    (fa, fb) = ref.matmul_grad_calls(False, True, False)
    assert fa == (False, False, False) and fb == (True, False, True)
    be.matmul(dy, fa[0], w, fa[1], fa[2], 16384, 16384, 4096, np.float16, out=wrap(dx))
    be.matmul(x, fb[0], dy, fb[1], fb[2], 4096, 16384, 16384, np.float16, out=wrap(dw))
    be.sync()
    be.checkDeviceStatus()
    rows = torch.randint(0, 16384, (48,), generator=torch.Generator().manual_seed(5)).cuda()
    assert _rel(y[rows], x[rows].double() @ w.double().t()) < TOL_F16
    assert _rel(dx[rows], dy[rows].double() @ w.double()) < TOL_F16
    assert _rel(dw[rows], dy[:, rows].double().t() @ x.double()) < TOL_F16


def test_config5_float32_16384_against_cuda_core_kernel(be):
    """float32 16384^3, U[-1,1): the 3xTF32 result against the CUDA-core kernel over the whole
    matrix (1e-5 relative Frobenius), sampled rows of both against float64, and a column block
    computed separately equal to the same columns bit for bit."""
    import torch
    from honeycrisp_b200 import _lib
    n = 16384
    g = torch.Generator(device="cuda").manual_seed(4)
    a = torch.rand((n, n), generator=g, device="cuda") * 2 - 1
    b = torch.rand((n, n), generator=g, device="cuda") * 2 - 1
    c_tc = torch.empty((n, n), device="cuda")
    c_cc = torch.empty((n, n), device="cuda")
    torch.cuda.synchronize()
    wrap = lambda t: be.wrap(t.data_ptr(), t.numel() * 4, t)
    be.matmul(a, False, b, False, False, n, n, n, np.float32, out=wrap(c_tc), kernel=_lib.HC_KERNEL_TENSOR)
    be.matmul(a, False, b, False, False, n, n, n, np.float32, out=wrap(c_cc), kernel=_lib.HC_KERNEL_SIMT)
    be.sync()
    be.checkDeviceStatus()
    num = torch.zeros((), device="cuda", dtype=torch.float64)
    den = torch.zeros((), device="cuda", dtype=torch.float64)
    for r0 in range(0, n, 2048):      # norms in slabs: a float64 copy of the whole matrix is 2 GiB
        d = c_tc[r0:r0 + 2048].double() - c_cc[r0:r0 + 2048].double()
        num += (d * d).sum()
        den += (c_cc[r0:r0 + 2048].double() ** 2).sum()
    assert float((num / den).sqrt()) < TOL_F32
    rows = torch.randint(0, n, (32,), generator=torch.Generator().manual_seed(6)).cuda()
    want = a[rows].double() @ b.double()
    assert _rel(c_tc[rows], want) < TOL_F32
    assert _rel(c_cc[rows], want) < TOL_F32
    blk = torch.zeros((n, n), device="cuda")
    be.matmulColumnBlock(a, False, b, False, False, n, n, n, 4096, 2048, np.float32, out=wrap(blk),
                         kernel=_lib.HC_KERNEL_TENSOR)
    be.sync()
    assert torch.equal(blk[:, 4096:6144], c_tc[:, 4096:6144])
    assert float(blk[:, :4096].abs().max()) == 0.0 and float(blk[:, 6144:].abs().max()) == 0.0

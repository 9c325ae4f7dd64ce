"""The CPU oracle against the reference's own known-answer vectors (no GPU needed)."""
import numpy as np
import pytest

from helpers import FLAG_COMBOS, golden, logical_out, random_operands, stored
from oracle import reference_cpu as ref

G = golden()


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("ta,tb,to", FLAG_COMBOS)
def test_matrix_matrix_product_vectors(ta, tb, to, dtype):
    """BackendTests.swift:684-712: exact output and both gradients for all eight flag triples."""
    v = G["matrix_matrix_product"]
    x = np.array(v["x"], dtype=dtype).reshape(v["x_shape"])
    y = np.array(v["y_before_t"], dtype=dtype).reshape(v["y_before_t_shape"]).T  # [3,4]
    g = np.array(v["out_grad"], dtype=dtype).reshape(v["out_shape"])
    rows, inner, cols = 2, 3, 4
    a_st, b_st = stored(x, ta), stored(y, tb)
    out = ref.matmul(a_st, ta, b_st, tb, to, rows, inner, cols)
    assert out.dtype == dtype
    np.testing.assert_array_equal(logical_out(out, 1, rows, cols, to)[0].reshape(-1).astype(np.float64), v["out"])
    # Backward products exactly as Linalg.swift:73-80 issues them; grad arrives in out's storage.
    g_st = stored(g, to)
    (fa, fb) = ref.matmul_grad_calls(ta, tb, to)
    # dA has a's stored shape: rows/cols of that product are a's logical dims after fa's flags.
    da = ref.matmul(g_st, fa[0], b_st, fa[1], fa[2], rows, cols, inner)
    da_logical = logical_out(da, 1, rows, inner, ta)[0]
    np.testing.assert_array_equal(da_logical.reshape(-1).astype(np.float64), v["a_grad"])
    db = ref.matmul(a_st, fb[0], g_st, fb[1], fb[2], inner, rows, cols)
    db_logical = logical_out(db, 1, inner, cols, tb)[0]
    np.testing.assert_array_equal(db_logical.reshape(-1).astype(np.float64), v["b_grad"])


def test_ones_product_and_half_overflow():
    """BackendTests.swift:713-725."""
    v = G["ones_product"]
    a = np.ones(v["a_shape"], dtype=np.float32)
    b = np.ones(v["b_shape"], dtype=np.float32)
    for fast in (True, False):
        z = ref.matmul(a, False, b, False, False, 64, 128, 32, library_fast_path=fast)
        np.testing.assert_array_equal(z, np.full(64 * 32, v["value"], dtype=np.float32))
    small = ref.matmul(a.astype(np.float16), False, b.astype(np.float16), False, False, 64, 128, 32)
    assert np.isfinite(small.astype(np.float32).sum())
    big = ref.matmul((a * v["overflow_scale"]).astype(np.float16), False, (b * v["overflow_scale"]).astype(np.float16),
                     False, False, 64, 128, 32)
    assert not np.isfinite(big.astype(np.float32).sum())
    assert np.all(np.isposinf(big.astype(np.float32)))


def test_matrix_vector_product_vectors():
    """BackendTests.swift:769-783 (cols == 1)."""
    v = G["matrix_vector_product"]
    x = np.array(v["x"], dtype=np.float32).reshape(v["x_shape"])
    y = np.array(v["y"], dtype=np.float32).reshape(v["y_shape"])
    out = ref.matmul(x, False, y, False, False, 2, 3, 1)
    np.testing.assert_array_equal(out, np.array(v["out"], dtype=np.float32))
    g = np.ones((2, 1), dtype=np.float32)
    (fa, fb) = ref.matmul_grad_calls(False, False, False)
    dx = ref.matmul(g, fa[0], y, fa[1], fa[2], 2, 1, 3)
    np.testing.assert_array_equal(dx, np.array(v["x_grad"], dtype=np.float32))
    dy = ref.matmul(x, fb[0], g, fb[1], fb[2], 3, 2, 1)
    np.testing.assert_array_equal(dy, np.array(v["y_grad"], dtype=np.float32))


@pytest.mark.parametrize("dtype,eps", [(np.float32, 1e-4), (np.float16, 1e-2)])
@pytest.mark.parametrize("ta,tb,to", FLAG_COMBOS)
def test_batched_matches_single(ta, tb, to, dtype, eps):
    """BackendTests.swift:728-767: batched output equals the per-matrix products."""
    A, B = random_operands(7, 3, 2, 3, 4, dtype, dist="uniform01")
    out = ref.batched_matmul(3, stored(A, ta), ta, stored(B, tb), tb, to, 2, 3, 4)
    for i in range(3):
        single = ref.matmul(stored(A[i], ta), ta, stored(B[i], tb), tb, to, 2, 3, 4)
        np.testing.assert_allclose(out.reshape(3, -1)[i].astype(np.float32), single.astype(np.float32), atol=eps, rtol=eps)


def test_half_conversions_match_ieee():
    """Widening is exact and narrowing is round-to-nearest-even with overflow to infinity
    (TensorElement.swift:262-277,325-338 via vImage); numpy's float16 casts are IEEE too."""
    all_halves = np.arange(65536, dtype=np.uint32).astype(np.uint16).view(np.float16)
    wide = ref.half_to_float(all_halves)
    expect = all_halves.astype(np.float32)
    assert np.array_equal(wide.view(np.uint32)[~np.isnan(expect)], expect.view(np.uint32)[~np.isnan(expect)])
    assert np.all(np.isnan(wide[np.isnan(expect)]))
    rng = np.random.default_rng(0)
    bits = rng.integers(0, 2**32, 2_000_000, dtype=np.uint64).astype(np.uint32)
    f = bits.view(np.float32)
    f = f[~np.isnan(f)]
    extra = np.array([65504.0, 65519.99, 65520.0, 65536.0, 1e30, -1e30, 2.0**-24, 2.0**-25, 2.0**-25 * 1.0001,
                      2.0**-14, 2.0**-14 * 0.9999, 0.0, -0.0, np.inf, -np.inf], dtype=np.float32)
    f = np.concatenate([f, extra])
    with np.errstate(over="ignore"):
        expect16 = f.astype(np.float16)
    got16 = ref.float_to_half(f)
    assert np.array_equal(got16.view(np.uint16), expect16.view(np.uint16))


@pytest.mark.parametrize("ta,tb,to", FLAG_COMBOS)
def test_loop_against_float64(ta, tb, to):
    A, B = random_operands(11, 2, 37, 53, 29, np.float32)
    out = ref.batched_matmul(2, stored(A, ta), ta, stored(B, tb), tb, to, 37, 53, 29)
    f64 = ref.batched_matmul_f64(2, stored(A, ta), ta, stored(B, tb), tb, to, 37, 53, 29)
    assert ref.rel_frobenius(out, f64) < 1e-6


def test_sgemm_stand_in_matches_loop_within_tolerance():
    """The library GEMM standing in for vDSP_mmul agrees with the literal loop at the tolerance
    quoted for float32 (1e-5 relative Frobenius)."""
    kind, addr, desc = ref.find_sgemm()
    A, B = random_operands(0, 1, 128, 256, 96, np.float32, dist="uniform01")
    fast = ref.matmul(A, False, B, False, False, 128, 256, 96, library_fast_path=True)
    loop = ref.matmul(A, False, B, False, False, 128, 256, 96, library_fast_path=False)
    assert ref.rel_frobenius(fast, loop) < 1e-5, desc


def test_row_sample_is_bit_identical_to_full_run():
    A, B = random_operands(5, 2, 16, 40, 24, np.float32)
    full = ref.batched_matmul(2, A, False, stored(B, True), True, False, 16, 40, 24)
    part = ref.loop_rows(2, A, False, stored(B, True), True, False, 16, 40, 24, 4, 9, threads=3)
    full = full.reshape(2, 16, 24)
    part = part.reshape(2, 16, 24)
    assert np.array_equal(full[:, 4:9].view(np.uint32), part[:, 4:9].view(np.uint32))


def test_empty_dimensions():
    z = ref.matmul(np.zeros((3, 0), np.float32), False, np.zeros((0, 4), np.float32), False, False, 3, 0, 4,
                   library_fast_path=False)
    assert z.shape == (12,) and np.all(z == 0)
    z = ref.matmul(np.zeros((0, 5), np.float16), False, np.zeros((5, 4), np.float16), False, False, 0, 5, 4)
    assert z.size == 0


# ---- the operations around a Linear layer -----------------------------------------------------

@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_linear_forward_is_matmul_then_broadcast_add(dtype):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((6, 4)).astype(dtype)
    w = rng.standard_normal((4, 5)).astype(dtype)      # Linear(4 -> 5), the size HoneycrispTests.swift:700-727 uses
    b = rng.standard_normal(5).astype(dtype)
    y = ref.linear_forward(x, w, b, 6, 4, 5)
    h = ref.matmul(x, False, w, False, False, 6, 4, 5)
    manual = (h.reshape(6, 5).astype(np.float32) + b.astype(np.float32)).astype(dtype).reshape(-1)
    assert np.array_equal(y.view(np.uint8), manual.view(np.uint8))
    assert np.array_equal(ref.linear_forward(x, w, None, 6, 4, 5).view(np.uint8), h.view(np.uint8))
    f64 = (x.astype(np.float64) @ w.astype(np.float64) + b.astype(np.float64)).reshape(-1)
    assert ref.rel_frobenius(y, f64) < (1e-6 if dtype == np.float32 else 2e-3)


def test_column_sum_order_and_rounding():
    # 2048 + 1 + 1 in float16: summed in float32 and narrowed once gives 2050; narrowing after
    # every add would stay at 2048.
    x = np.array([[2048.0], [1.0], [1.0]], dtype=np.float16)
    assert float(ref.column_sum(x, 3, 1)[0]) == 2050.0
    rng = np.random.default_rng(3)
    x = rng.standard_normal((500, 37)).astype(np.float32)
    s = ref.column_sum(x, 500, 37)
    assert ref.rel_frobenius(s, x.astype(np.float64).sum(axis=0)) < 1e-6
    seq = np.zeros(37, dtype=np.float32)
    for r in range(500):
        seq += x[r]
    assert np.array_equal(s.view(np.uint32), seq.view(np.uint32))


def test_cast_and_add_helpers():
    x = np.array([1.0, 65519.0, 65520.0, -1e-8, np.inf], dtype=np.float32)
    with np.errstate(over="ignore"):
        assert np.array_equal(ref.cast(x, np.float16).view(np.uint16), x.astype(np.float16).view(np.uint16))
    a = np.array([1000.0, 0.5], dtype=np.float16)
    b = np.array([0.25, 0.5], dtype=np.float16)
    assert ref.add(a, b).tolist() == [1000.0, 1.0]


# ---- the generator behind Tensor(rand:) / Tensor(randn:) ---------------------------------------

def test_philox_known_answer_and_counter_layout():
    """Philox-4x32-10 with zero key and counter gives the published known-answer words; the
    reference puts the 64-bit offset in counter words 0 and 1 and the seed in the key
    (BackendCPU.swift:177-199)."""
    w = ref.philox4x32_10(0, [0])[0]
    assert [int(x) for x in w] == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    a = ref.philox4x32_10(5, [7, 8, (1 << 32) + 7])
    assert len({tuple(r) for r in a.tolist()}) == 3            # offsets beyond 32 bits matter
    assert not np.array_equal(ref.philox4x32_10(6, [7])[0], a[0])


def test_generator_statistics_and_state_as_the_reference_tests_them():
    """BackendTests.swift:1800-1824: moments of 100 000 samples, and restoring the state
    reproduces the same tensors."""
    x, off = ref.random_sample(0, 0, 100000, "normal", np.float32)
    assert abs(float(x.mean())) < 0.03 and abs(float(x.std()) - 1) < 0.03
    z, off2 = ref.random_sample(0, off, 100000, "uniform", np.float32)
    assert abs(float(z.mean()) - 0.5) < 0.03 and abs(float(z.std()) - 0.288675135) < 0.03
    assert off == 50001 and off2 == 50001 + 25001             # loops run `through: count`
    a, o1 = ref.random_sample(3, 10, 1234, "normal", np.float32)
    b, o2 = ref.random_sample(3, o1, 1234, "normal", np.float32)
    assert not np.array_equal(a, b)
    c, _ = ref.random_sample(3, 10, 1234, "normal", np.float32)
    d, _ = ref.random_sample(3, o1, 1234, "normal", np.float32)
    assert np.array_equal(a, c) and np.array_equal(b, d)
    assert float(z.max()) <= 1.0 and float(z.min()) >= 0.0

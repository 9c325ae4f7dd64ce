"""Consecutive products on the backend's own stream: a product's operand loads may start before
the product enqueued just before it has finished, but only when that product cannot have written
them.  Chains where each product reads the previous result must therefore still be exact, and
independent products must be unaffected."""
import numpy as np
import pytest

from oracle import reference_cpu as ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    from honeycrisp_b200 import CUDABackend
    b = CUDABackend(0)          # keeps its own stream: the case the overlap applies to
    yield b
    b.checkDeviceStatus()
    b.close()


def TENSOR():
    from honeycrisp_b200 import _lib
    return _lib.HC_KERNEL_TENSOR


@pytest.mark.parametrize("n", [256, 512, 1024])
def test_dependent_chain_is_exact(be, n):
    """x_{i+1} = x_i * P with P a permutation matrix: every product reads the previous product's
    result, products are exact in float16, and any load that ran ahead of its producer would
    surface as a wrong permutation."""
    rng = np.random.default_rng(n)
    x0 = rng.integers(-8, 9, (n, n)).astype(np.float16)
    perm = rng.permutation(n)
    P = np.zeros((n, n), dtype=np.float16)
    P[np.arange(n), perm] = 1.0
    x_d, p_d = be.collection(x0, np.float16), be.collection(P, np.float16)
    bufs = [be.allocate(n * n * 2) for _ in range(2)]
    cur = x_d
    steps = 24
    for i in range(steps):
        out = bufs[i % 2]
        be.matmul(cur, False, p_d, False, False, n, n, n, np.float16, kernel=TENSOR(), out=out, mark=False)
        cur = out
    got = cur.onCPU(np.float16)[: n * n].reshape(n, n)
    want = x0
    for _ in range(steps):
        want = want[:, np.argsort(perm)]
    assert np.array_equal(got, want)


def test_independent_products_interleaved_with_dependent_ones(be):
    """A, B fixed; C1 = A*B (independent of what ran before), then D = C1*B (reads C1), repeated
    with the roles of the buffers rotating: equal to doing each product with a sync in between."""
    rng = np.random.default_rng(3)
    n = 384
    a = rng.integers(-3, 4, (n, n)).astype(np.float16)
    b = (rng.integers(-1, 2, (n, n)) * (rng.random((n, n)) < 0.02)).astype(np.float16)   # sparse: stays exact
    a_d, b_d = be.collection(a, np.float16), be.collection(b, np.float16)
    c1, d1 = be.allocate(n * n * 2), be.allocate(n * n * 2)
    for _ in range(6):
        be.matmul(a_d, False, b_d, False, False, n, n, n, np.float16, kernel=TENSOR(), out=c1, mark=False)
        be.matmul(c1, False, b_d, False, False, n, n, n, np.float16, kernel=TENSOR(), out=d1, mark=False)
    want_c = (a.astype(np.float64) @ b.astype(np.float64))
    want_d = want_c @ b.astype(np.float64)
    assert np.abs(want_d).max() < 2048          # exactly representable in float16
    assert np.array_equal(c1.onCPU(np.float16)[: n * n].astype(np.float64).reshape(n, n), want_c)
    assert np.array_equal(d1.onCPU(np.float16)[: n * n].astype(np.float64).reshape(n, n), want_d)


def test_float32_chain_through_the_split_pre_pass(be):
    """float32 products read a work area their own pre-pass writes: the chain K1 -> split -> K2 must
    keep its order."""
    rng = np.random.default_rng(5)
    n = 256
    x0 = rng.integers(-4, 5, (n, n)).astype(np.float32)
    perm = rng.permutation(n)
    P = np.zeros((n, n), dtype=np.float32)
    P[np.arange(n), perm] = 1.0
    p_d = be.collection(P, np.float32)
    cur = be.collection(x0, np.float32)
    bufs = [be.allocate(n * n * 4) for _ in range(2)]
    for i in range(10):
        out = bufs[i % 2]
        be.matmul(cur, False, p_d, False, False, n, n, n, np.float32, kernel=TENSOR(), out=out, mark=False)
        cur = out
    want = x0
    for _ in range(10):
        want = want[:, np.argsort(perm)]
    assert np.array_equal(cur.onCPU(np.float32)[: n * n].reshape(n, n), want)

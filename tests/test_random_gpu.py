"""Device-side Philox samples against the CPU oracle of Honeycrisp's generator."""
import numpy as np
import pytest

from oracle import reference_cpu as ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    from honeycrisp_b200 import CUDABackend
    b = CUDABackend(0)
    yield b
    b.close()


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("count", [1, 3, 4, 5, 1000, 1024 * 1024 + 3])
def test_uniform_is_bit_identical(be, count, dtype):
    be.seed(0)
    be._rng_state[1] = (1 << 32) - 2 if count == 5 else 0      # one case crosses the 32-bit counter word
    off0 = be._rng_state[1]
    got = be.sample(count, "uniform", dtype).onCPU(dtype)[:count]
    want, nxt = ref.random_sample(0, off0, count, "uniform", dtype)
    assert np.array_equal(got.view(np.uint8), want.view(np.uint8))
    assert be._rng_state[1] == nxt


@pytest.mark.parametrize("count", [1, 2, 7, 1234, 100000])
def test_normal_matches_to_float_rounding(be, count):
    be.seed(12345678901234)
    got = be.sample(count, "normal", np.float32).onCPU(np.float32)[:count]
    want, nxt = ref.random_sample(12345678901234, 0, count, "normal", np.float32)
    # Box-Muller runs through logf/cosf/sinf, which differ between math libraries in the last
    # ulps; the words feeding it are identical.
    np.testing.assert_allclose(got, want, rtol=2e-5, atol=2e-6)
    assert be._rng_state[1] == nxt
    second = be.sample(count, "normal", np.float32).onCPU(np.float32)[:count]
    want2, _ = ref.random_sample(12345678901234, nxt, count, "normal", np.float32)
    np.testing.assert_allclose(second, want2, rtol=2e-5, atol=2e-6)


def test_config1_inputs_as_tensor_rand_seed0(be):
    """Configuration 1 literally: A and B are consecutive Tensor(rand: [1024, 1024]) draws of a
    generator seeded with 0; their float32 product on the tensor cores against the host sgemm."""
    be.seed(0)
    a = be.sample(1024 * 1024, "uniform", np.float32)
    b = be.sample(1024 * 1024, "uniform", np.float32)
    wa, off = ref.random_sample(0, 0, 1024 * 1024, "uniform", np.float32)
    wb, _ = ref.random_sample(0, off, 1024 * 1024, "uniform", np.float32)
    assert np.array_equal(a.onCPU(np.float32)[: 1024 * 1024], wa)
    assert np.array_equal(b.onCPU(np.float32)[: 1024 * 1024], wb)
    c = be.matmul(a, False, b, False, False, 1024, 1024, 1024, np.float32).onCPU(np.float32)[: 1024 * 1024]
    host = ref.matmul(wa, False, wb, False, False, 1024, 1024, 1024, library_fast_path=True)
    assert ref.rel_frobenius(c, host) < 1e-5

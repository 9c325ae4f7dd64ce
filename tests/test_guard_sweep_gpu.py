"""A seeded sweep over small and awkward shapes with guard bytes around every result buffer and
the result pre-filled with NaN patterns: nothing may be written outside the result, every
element of the result must be written, and the values must match the oracle."""
import itertools

import numpy as np
import pytest

from helpers import FLAG_COMBOS, random_operands, stored
from oracle import reference_cpu as ref

pytestmark = pytest.mark.gpu

GUARD = 512          # bytes before and after the result; keeps the result 16-byte aligned
SENTINEL = 0xA5


@pytest.fixture(scope="module")
def be():
    from honeycrisp_b200 import CUDABackend
    b = CUDABackend(0)
    yield b
    b.checkDeviceStatus()
    b.close()


def guarded_run(be, cnt, A, B, ta, tb, to, dtype, kernel):
    from honeycrisp_b200 import _lib
    lib = _lib.load()
    M, Kd, N = A.shape[-2], A.shape[-1], B.shape[-1]
    nbytes = cnt * M * N * np.dtype(dtype).itemsize
    host = np.full(GUARD + nbytes + GUARD, SENTINEL, dtype=np.uint8)
    host[GUARD:GUARD + nbytes] = 0xFF                       # NaN in both dtypes
    buf = be.allocate(host.size)
    assert lib.hc_h2d(be._ctx, buf.ptr, host.ctypes.data, host.size) == 0
    be.sync()
    out = be.wrap(buf.ptr + GUARD, nbytes, owner=buf)
    a_st, b_st = stored(A, ta), stored(B, tb)
    be.batchedMatmul(cnt, a_st, ta, b_st, tb, to, M, Kd, N, dtype, kernel=kernel, out=out)
    back = buf.onCPU(np.uint8)
    be.checkDeviceStatus()
    assert np.all(back[:GUARD] == SENTINEL), "wrote before the result"
    assert np.all(back[GUARD + nbytes:GUARD + nbytes + GUARD] == SENTINEL), "wrote past the result"
    res = back[GUARD:GUARD + nbytes].view(dtype)
    assert not np.any(np.isnan(res.astype(np.float32))), "left part of the result unwritten"
    return res, a_st, b_st


DIMS = [1, 2, 3, 7, 8, 15, 16, 17, 31, 33, 63, 64, 65, 127, 128, 129, 255, 257]


def test_any_shape_through_the_default_dispatch(be):
    """Dimensions from 1 to 257 around every tile and vector boundary, all eight flag triples,
    both dtypes, one and three matrices; the exact CUDA-core kernel must match the CPU loop bit
    for bit, the default dispatch within tolerance."""
    from honeycrisp_b200 import _lib
    rng = np.random.default_rng(2024)
    cases = [(int(rng.choice(DIMS)), int(rng.choice(DIMS)), int(rng.choice(DIMS)), FLAG_COMBOS[int(rng.integers(8))],
              [np.float32, np.float16][int(rng.integers(2))], [1, 3][int(rng.integers(2))]) for _ in range(160)]
    for i, (M, Kd, N, (ta, tb, to), dtype, cnt) in enumerate(cases):
        A, B = random_operands(i, cnt, M, Kd, N, dtype)
        res, a_st, b_st = guarded_run(be, cnt, A, B, ta, tb, to, dtype, _lib.HC_KERNEL_SIMT_EXACT)
        orc = ref.batched_matmul(cnt, a_st, ta, b_st, tb, to, M, Kd, N, library_fast_path=False)
        assert np.array_equal(res.view(np.uint8), orc.view(np.uint8)), (M, Kd, N, ta, tb, to, dtype, cnt)
        res, _, _ = guarded_run(be, cnt, A, B, ta, tb, to, dtype, _lib.HC_KERNEL_AUTO)
        assert ref.rel_frobenius(res, orc) < (1e-5 if dtype == np.float32 else 2e-3), (M, Kd, N, ta, tb, to, dtype, cnt)


ALIGNED = [8, 16, 24, 40, 64, 72, 120, 128, 136, 200, 256, 264, 392, 520]


def test_aligned_shapes_through_the_tensor_core_kernels(be):
    """Every combination of tile-edge cases the TMA paths can take (dimensions are multiples of
    eight, so every leading dimension is 16-byte aligned for both dtypes)."""
    from honeycrisp_b200 import _lib
    rng = np.random.default_rng(7)
    cases = [(int(rng.choice(ALIGNED)), int(rng.choice(ALIGNED)), int(rng.choice(ALIGNED)),
              FLAG_COMBOS[int(rng.integers(8))], [np.float32, np.float16][int(rng.integers(2))],
              [1, 2][int(rng.integers(2))]) for _ in range(160)]
    for i, (M, Kd, N, (ta, tb, to), dtype, cnt) in enumerate(cases):
        A, B = random_operands(1000 + i, cnt, M, Kd, N, dtype, dist="uniform11")
        res, a_st, b_st = guarded_run(be, cnt, A, B, ta, tb, to, dtype, _lib.HC_KERNEL_TENSOR)
        orc = ref.batched_matmul(cnt, a_st, ta, b_st, tb, to, M, Kd, N, library_fast_path=False)
        assert ref.rel_frobenius(res, orc) < (1e-5 if dtype == np.float32 else 2e-3), (M, Kd, N, ta, tb, to, dtype, cnt)

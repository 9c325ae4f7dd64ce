"""A Linear layer's forward and backward pass on the device, against the CPU oracle."""
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


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("rows,n_in,n_out", [(4, 5, 3), (2, 3, 4), (130, 67, 129), (64, 128, 32)])
def test_fused_bias_is_bit_identical_to_matmul_then_add_small(be, rows, n_in, n_out, dtype):
    """Shapes TMA cannot describe (and the reference's own Linear(4 -> 5) test size) run on the
    CUDA-core kernel, whose product is bit-identical to the CPU loop for float16; the fused bias
    add must then match the reference's separate add bit for bit."""
    rng = np.random.default_rng(rows + n_in)
    x = rng.standard_normal((rows, n_in)).astype(dtype)
    w = rng.standard_normal((n_in, n_out)).astype(dtype)
    b = rng.standard_normal(n_out).astype(dtype)
    got = be.linearForward(x, w, b, rows, n_in, n_out, dtype).onCPU(dtype)[: rows * n_out]
    h = be.matmul(x, False, w, False, False, rows, n_in, n_out, dtype).onCPU(dtype)[: rows * n_out]
    assert np.array_equal(got.view(np.uint8), ref.broadcast_add_rows(h, b, rows, n_out).view(np.uint8))
    want = ref.linear_forward(x, w, b, rows, n_in, n_out)
    from honeycrisp_b200 import _lib
    if dtype == np.float16 and be.lastLaunchInfo()["kernel"] == _lib.HC_KERNEL_SIMT_EXACT:
        # CUDA-core product in the reference's arithmetic = the CPU loop (float32 without flags is a
        # library sgemm in the reference, so only float16 is bit-comparable end to end)
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    else:
        assert ref.rel_frobenius(got, want) < (1e-5 if dtype == np.float32 else 2e-3)
    none = be.linearForward(x, w, None, rows, n_in, n_out, dtype).onCPU(dtype)[: rows * n_out]
    assert np.array_equal(none.view(np.uint8), h.view(np.uint8))


@pytest.mark.parametrize("dtype,tol", [(np.float32, 1e-5), (np.float16, 2e-3)])
@pytest.mark.parametrize("rows,n_in,n_out", [(256, 128, 256), (1000, 520, 776), (384, 64, 96), (2048, 4096, 1024),
                                             # long contractions over few outputs: cut into parts, bias added by the
                                             # kernel that sums them (aligned, and a result pitch no vector store fits)
                                             (256, 4096, 256), (264, 4104, 198)])
def test_fused_bias_on_the_tensor_core_path(be, rows, n_in, n_out, dtype, tol):
    """The tensor-core epilogue adds the bias to the rounded product: identical, bit for bit, to
    this library's own product followed by the oracle's add; and within tolerance of float64."""
    from honeycrisp_b200 import _lib
    rng = np.random.default_rng(n_out)
    x = rng.standard_normal((rows, n_in)).astype(dtype)
    w = (rng.standard_normal((n_in, n_out)) / np.sqrt(n_in)).astype(dtype)
    b = rng.standard_normal(n_out).astype(dtype)
    got = be.linearForward(x, w, b, rows, n_in, n_out, dtype).onCPU(dtype)[: rows * n_out]
    assert be.lastLaunchInfo()["kernel"] == _lib.HC_KERNEL_TENSOR
    h = be.matmul(x, False, w, False, False, rows, n_in, n_out, dtype).onCPU(dtype)[: rows * n_out]
    assert np.array_equal(got.view(np.uint8), ref.broadcast_add_rows(h, b, rows, n_out).view(np.uint8))
    f64 = (x.astype(np.float64) @ w.astype(np.float64) + b.astype(np.float64)).reshape(-1)
    assert ref.rel_frobenius(got, f64) < tol


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("rows,cols", [(1, 7), (9, 1), (33, 130), (4096, 520), (257, 4099),
                                       # tall inputs with 16-byte rows stream through shared memory: every strip
                                       # width (32, 64, 128 bytes), ragged last strip, ragged last row block
                                       (512, 8), (1000, 72), (777, 1096), (2049, 4104), (600, 16384), (5000, 20000)])
def test_column_sum_is_bit_identical_to_the_cpu_loop(be, rows, cols, dtype):
    x = np.random.default_rng(rows * cols).standard_normal((rows, cols)).astype(dtype)
    got = be.columnSum(x, rows, cols, dtype).onCPU(dtype)[:cols]
    want = ref.column_sum(x, rows, cols)
    assert np.array_equal(got.view(np.uint8), want.view(np.uint8))


def test_cast_and_add_are_bit_identical(be):
    rng = np.random.default_rng(9)
    x32 = (rng.standard_normal(100003) * 1e3).astype(np.float32)
    x32[:4] = [np.inf, -np.inf, 65520.0, 1e-8]
    h = be.cast(x32, x32.size, np.float32, np.float16).onCPU(np.float16)[: x32.size]
    assert np.array_equal(h.view(np.uint16), ref.cast(x32, np.float16).view(np.uint16))
    back = be.cast(h, h.size, np.float16, np.float32).onCPU(np.float32)[: h.size]
    assert np.array_equal(back.view(np.uint32), ref.cast(h, np.float32).view(np.uint32))
    for dt in (np.float32, np.float16):
        a = rng.standard_normal(50001).astype(dt)
        b = rng.standard_normal(50001).astype(dt)
        got = be.add(a, b, a.size, dt).onCPU(dt)[: a.size]
        assert np.array_equal(got.view(np.uint8), ref.add(a, b).reshape(-1).view(np.uint8))


def test_constant_is_the_value_narrowed_once(be):
    """Backend.constant (Backend.swift:787-791): the CPU backend writes Float(value) through the
    element type (BackendCPU.swift:1796-1815); every count, including the ragged ends around the
    16-byte groups, and a start that is not 16-byte aligned."""
    from honeycrisp_b200 import _lib
    for dt in (np.float32, np.float16):
        for value in (0.1, 3.0, -0.0, 65520.0, 1e-8, -7.25):
            for count in (0, 1, 7, 8, 9, 4099):
                got = be.constant(value, count, dt).onCPU(dt)[:count]
                with np.errstate(over="ignore"):   # 65520 is infinity in float16, as in the reference
                    want = np.full(count, np.float32(value)).astype(dt)
                assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), (dt, value, count)
        eb = np.dtype(dt).itemsize
        buf = be.constant(1.0, 64, dt)
        for first, count in ((1, 37), (3, 5), (5, 59)):
            assert be._lib.hc_constant(be._ctx, 0 if dt == np.float16 else 1, 2.5, count, buf.ptr + first * eb) == _lib.HC_OK
            got = buf.onCPU(dt)[:64]
            want = np.ones(64, dt)
            want[first:first + count] = 2.5
            assert np.array_equal(got, want), (dt, first, count)
            assert be._lib.hc_constant(be._ctx, 0 if dt == np.float16 else 1, 1.0, 64, buf.ptr) == _lib.HC_OK
    assert be._lib.hc_constant(be._ctx, 1, 0.0, -1, None) == _lib.HC_ERR_INVALID_ARGUMENT
    assert be._lib.hc_constant(be._ctx, 7, 0.0, 4, buf.ptr) == _lib.HC_ERR_NOT_IMPLEMENTED


# (weight dtype, castParams, compute dtype): the three ways the reference's Linear is used
# (Trainable.swift:514-544) - plain float32; float16 weights with the float32 bias cast on use;
# float32 master weights cast to float16 on every call.
@pytest.mark.parametrize("wdtype,cast,cdtype,tol", [(np.float32, None, np.float32, 1e-5),
                                                    (np.float16, np.float16, np.float16, 2e-3),
                                                    (np.float32, np.float16, np.float16, 2e-3)])
def test_linear_layer_forward_and_backward(be, wdtype, cast, cdtype, tol):
    """Linear(inCount -> outCount) on a [batch, seq, in] input: output, input gradient, weight
    gradient and bias gradient against the oracle's products, sums and casts."""
    from honeycrisp_b200 import Linear
    layer = Linear(be, 256, 384, dtype=wdtype, castParams=cast, seed=3)
    w = layer.weight.onCPU(wdtype)[: 256 * 384].reshape(256, 384)
    assert np.abs(w.astype(np.float32)).max() <= np.sqrt(3.0) / np.sqrt(256) + 1e-3
    assert layer.bias.byteCount == 384 * 4                      # the bias is float32 whatever the layer's dtype
    assert not layer.bias.onCPU(np.float32)[:384].any()
    rng = np.random.default_rng(1)
    b32 = rng.standard_normal(384).astype(np.float32)
    layer.bias = be.collection(b32, np.float32)
    x = rng.standard_normal((4, 96, 256)).astype(cdtype)
    y, yshape = layer(x, x.shape)
    assert yshape == [4, 96, 384]
    rows = 4 * 96
    wc, bc = ref.cast(w, cdtype).reshape(256, 384), ref.cast(b32, cdtype).reshape(-1)   # weight.cast / bias.cast
    want_y = ref.linear_forward(x.reshape(rows, 256), wc, bc, rows, 256, 384)
    assert ref.rel_frobenius(y.onCPU(cdtype)[: rows * 384], want_y) < tol
    g = rng.standard_normal((4, 96, 384)).astype(cdtype)
    dx = layer.backward(x, x.shape, g)
    (fa, fb) = ref.matmul_grad_calls(False, False, False)
    want_dx = ref.matmul(g.reshape(rows, 384), fa[0], wc, fa[1], fa[2], rows, 384, 256)
    want_dw = ref.matmul(x.reshape(rows, 256), fb[0], g.reshape(rows, 384), fb[1], fb[2], 256, rows, 384)
    assert ref.rel_frobenius(dx.onCPU(cdtype)[: rows * 256], want_dx) < tol
    # gradients come back in the parameters' own dtypes (the backward of cast)
    assert layer.weightGrad.byteCount == 256 * 384 * np.dtype(wdtype).itemsize
    assert ref.rel_frobenius(layer.weightGrad.onCPU(wdtype)[: 256 * 384], ref.cast(want_dw, wdtype).reshape(-1)) < tol
    want_db = ref.cast(ref.column_sum(g.reshape(rows, 384), rows, 384), np.float32).reshape(-1)
    assert layer.biasGrad.byteCount == 384 * 4
    assert np.array_equal(layer.biasGrad.onCPU(np.float32)[:384].view(np.uint8), want_db.view(np.uint8))
    # a second backward accumulates (Param.addGrad)
    layer.backward(x, x.shape, g)
    assert np.array_equal(layer.biasGrad.onCPU(np.float32)[:384].view(np.uint8), ref.add(want_db, want_db).reshape(-1).view(np.uint8))


def test_linear_layer_refuses_what_the_reference_refuses(be):
    """float16 weights, float32 bias, no castParams: `h + bias` mixes dtypes, which the reference's
    binary ops assert against; without a bias the same layer is fine."""
    from honeycrisp_b200 import Linear
    x = np.ones((8, 64), dtype=np.float16)
    with pytest.raises(ValueError):
        Linear(be, 64, 32, dtype=np.float16)(x, x.shape)
    out, shape = Linear(be, 64, 32, dtype=np.float16, bias=False)(x, x.shape)
    assert shape == [8, 32] and out.byteCount == 8 * 32 * 2


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("cnt,rows,cols", [(1, 1, 1), (1, 2, 3), (3, 33, 65), (2, 1000, 31), (1, 2048, 512),
                                           # even sides: float16 moves 64 x 64 tiles with 4-byte accesses
                                           (2, 130, 66), (3, 64, 64), (1, 70, 4098)])
def test_materialised_transpose(be, cnt, rows, cols, dtype):
    x = np.random.default_rng(cols).standard_normal((cnt, rows, cols)).astype(dtype)
    got = be.transpose(x, cnt, rows, cols, dtype).onCPU(dtype)[: x.size].reshape(cnt, cols, rows)
    assert np.array_equal(got, np.swapaxes(x, 1, 2))


def test_transposed_operand_equals_the_transpose_flag(be):
    """`m1.t() &* m2` as the reference's benchmark issues it (a materialised transpose, then a
    plain product) equals the product with transA set, bit for bit."""
    rng = np.random.default_rng(4)
    m1 = rng.random((1024, 1024), dtype=np.float32).astype(np.float16)
    m2 = rng.random((1024, 1024), dtype=np.float32).astype(np.float16)
    m1_d, m2_d = be.collection(m1, np.float16), be.collection(m2, np.float16)
    t = be.transpose(m1_d, 1, 1024, 1024, np.float16)
    a = be.matmul(t, False, m2_d, False, False, 1024, 1024, 1024, np.float16).onCPU(np.float16)
    b = be.matmul(m1_d, True, m2_d, False, False, 1024, 1024, 1024, np.float16).onCPU(np.float16)
    assert np.array_equal(a.view(np.uint16), b.view(np.uint16))

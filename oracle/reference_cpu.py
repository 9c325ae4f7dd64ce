"""numpy/ctypes front end of the CPU oracle.  TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the CPU-baseline leg of the benchmark import this module;
the shipped package never does.  The arithmetic lives in oracle/hc_oracle.c (a restatement of
Honeycrisp's CPUBackend.batchedMatmul, Sources/Honeycrisp/BackendCPU.swift:1234-1313); this
file adds

* the host sgemm that stands in for Accelerate's vDSP_mmul (BackendCPU.swift:1256), found in
  the OpenBLAS builds that ship inside the Python wheels on this image,
* a float64 product with the same flag semantics (for the float16 tolerance, which is quoted
  against a float64 product),
* the relative Frobenius error,
* the autodiff flag algebra of Tensor.matmul (Sources/Honeycrisp/Linalg.swift:73-80) so the
  reference's gradient known-answer vectors can be replayed.
"""
from __future__ import annotations

import ctypes
import glob
import os
import sys

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
if _HERE not in sys.path:
    sys.path.insert(0, _HERE)
import build as _oracle_build  # noqa: E402  (oracle/build.py)

_lib = None
_sgemm = None  # (kind, address, owner, set_threads)


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = _oracle_build.build()
        L = ctypes.CDLL(path)
        i64, vp, ci = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int
        L.hc_oracle_batched_matmul_f32.argtypes = [i64, vp, ci, vp, ci, ci, i64, i64, i64, vp, vp, vp, ci]
        L.hc_oracle_batched_matmul_f32.restype = ci
        L.hc_oracle_batched_matmul_f16.argtypes = [i64, vp, ci, vp, ci, ci, i64, i64, i64, vp]
        L.hc_oracle_batched_matmul_f16.restype = ci
        L.hc_oracle_loop_rows_f32.argtypes = [i64, vp, ci, vp, ci, ci, i64, i64, i64, vp, i64, i64, ci]
        L.hc_oracle_loop_rows_f32.restype = None
        L.hc_oracle_half_to_float.argtypes = [vp, vp, i64]
        L.hc_oracle_float_to_half.argtypes = [vp, vp, i64]
        _lib = L
    return _lib


def find_sgemm():
    """Locate a row-major cblas sgemm.  Returns (kind, address, description) with kind in
    {"lp64", "ilp64"} or (None, None, reason)."""
    global _sgemm
    if _sgemm is not None:
        return _sgemm[:3]
    roots = [p for p in sys.path if p.endswith("site-packages")]
    candidates = []
    for r in roots:
        candidates += [(p, "cblas_sgemm", "lp64", "openblas_set_num_threads")
                       for p in sorted(glob.glob(os.path.join(r, "opencv_python_headless.libs", "libopenblas*.so*")))]
        candidates += [(p, "scipy_cblas_sgemm", "lp64", "scipy_openblas_set_num_threads")
                       for p in sorted(glob.glob(os.path.join(r, "scipy.libs", "libscipy_openblas-*.so*")))]
        candidates += [(p, "scipy_cblas_sgemm64_", "ilp64", "scipy_openblas_set_num_threads64_")
                       for p in sorted(glob.glob(os.path.join(r, "numpy.libs", "libscipy_openblas64_*.so*")))]
    for path, sym, kind, thr in candidates:
        try:
            L = ctypes.CDLL(path)
            fn = getattr(L, sym)
        except (OSError, AttributeError):
            continue
        setter = getattr(L, thr, None)
        _sgemm = (kind, ctypes.cast(fn, ctypes.c_void_p).value, f"{os.path.basename(path)}:{sym}", L, setter)
        return _sgemm[:3]
    _sgemm = (None, None, "no OpenBLAS with a cblas sgemm found", None, None)
    return _sgemm[:3]


def set_sgemm_threads(n: int) -> bool:
    find_sgemm()
    setter = _sgemm[4]
    if setter is None:
        return False
    setter.argtypes = [ctypes.c_int]
    setter(int(n))
    return True


def _ptr(x: np.ndarray):
    return ctypes.c_void_p(x.ctypes.data)


def batched_matmul(matrix_count, a, trans_a, b, trans_b, trans_out, rows, inner, cols,
                   library_fast_path=True):
    """CPUBackend.batchedMatmul on flat numpy operands (float32 or float16).

    `a` holds matrix_count dense matrices of shape [rows,inner] ([inner,rows] if trans_a), `b`
    likewise [inner,cols] ([cols,inner] if trans_b); the result is flat, [rows,cols] per matrix
    ([cols,rows] if trans_out).  float32 with no flags goes to the host sgemm unless
    library_fast_path is False, everything else through the literal loop.
    """
    a = np.ascontiguousarray(a).reshape(-1)
    b = np.ascontiguousarray(b).reshape(-1)
    assert a.dtype == b.dtype and a.dtype in (np.float32, np.float16)
    assert a.size == matrix_count * rows * inner and b.size == matrix_count * inner * cols
    out = np.empty(matrix_count * rows * cols, dtype=a.dtype)
    L = lib()
    if a.dtype == np.float32:
        kind, addr, _ = find_sgemm()
        use_fast = bool(library_fast_path) and not (trans_a or trans_b or trans_out)
        if use_fast and addr is None:
            # numpy's own float32 matmul is the same OpenBLAS sgemm behind another door.
            A = a.reshape(matrix_count, rows, inner)
            B = b.reshape(matrix_count, inner, cols)
            return np.matmul(A, B).reshape(-1)
        rc = L.hc_oracle_batched_matmul_f32(
            matrix_count, _ptr(a), int(trans_a), _ptr(b), int(trans_b), int(trans_out), rows, inner,
            cols, _ptr(out), addr if kind == "lp64" else None, addr if kind == "ilp64" else None,
            int(use_fast))
    else:
        rc = L.hc_oracle_batched_matmul_f16(
            matrix_count, _ptr(a.view(np.uint16)), int(trans_a), _ptr(b.view(np.uint16)), int(trans_b),
            int(trans_out), rows, inner, cols, _ptr(out.view(np.uint16)))
    if rc != 0:
        raise RuntimeError(f"oracle failed with code {rc}")
    return out


def matmul(a, trans_a, b, trans_b, trans_out, rows, inner, cols, library_fast_path=True):
    """CPUBackend.matmul (BackendCPU.swift:1222-1232)."""
    return batched_matmul(1, a, trans_a, b, trans_b, trans_out, rows, inner, cols, library_fast_path)


def loop_rows(matrix_count, a32, trans_a, b32, trans_b, trans_out, rows, inner, cols, row_begin,
              row_end, threads=1, out=None):
    """The literal loop on float32 operands for rows [row_begin,row_end) of each matrix.
    Returns the full-size float32 output buffer with only those rows filled."""
    a32 = np.ascontiguousarray(a32, dtype=np.float32).reshape(-1)
    b32 = np.ascontiguousarray(b32, dtype=np.float32).reshape(-1)
    if out is None:
        out = np.zeros(matrix_count * rows * cols, dtype=np.float32)
    lib().hc_oracle_loop_rows_f32(matrix_count, _ptr(a32), int(trans_a), _ptr(b32), int(trans_b),
                                  int(trans_out), rows, inner, cols, _ptr(out), row_begin, row_end,
                                  int(threads))
    return out


def float_to_half(x32):
    x32 = np.ascontiguousarray(x32, dtype=np.float32).reshape(-1)
    out = np.empty(x32.size, dtype=np.float16)
    lib().hc_oracle_float_to_half(_ptr(x32), _ptr(out.view(np.uint16)), x32.size)
    return out


def half_to_float(x16):
    x16 = np.ascontiguousarray(x16, dtype=np.float16).reshape(-1)
    out = np.empty(x16.size, dtype=np.float32)
    lib().hc_oracle_half_to_float(_ptr(x16.view(np.uint16)), _ptr(out), x16.size)
    return out


def logical_operands(matrix_count, a, trans_a, b, trans_b, rows, inner, cols):
    """Views of the stored operands as [matrix_count, rows, inner] and [matrix_count, inner, cols]."""
    a = np.asarray(a).reshape(-1)
    b = np.asarray(b).reshape(-1)
    A = a.reshape(matrix_count, inner, rows).transpose(0, 2, 1) if trans_a else a.reshape(matrix_count, rows, inner)
    B = b.reshape(matrix_count, cols, inner).transpose(0, 2, 1) if trans_b else b.reshape(matrix_count, inner, cols)
    return A, B


def batched_matmul_f64(matrix_count, a, trans_a, b, trans_b, trans_out, rows, inner, cols):
    """float64 product with the same storage conventions; flat float64 result."""
    A, B = logical_operands(matrix_count, a, trans_a, b, trans_b, rows, inner, cols)
    C = np.matmul(A.astype(np.float64), B.astype(np.float64))
    if trans_out:
        C = C.transpose(0, 2, 1)
    return np.ascontiguousarray(C).reshape(-1)


def rel_frobenius(x, ref) -> float:
    x = np.asarray(x, dtype=np.float64).reshape(-1)
    ref = np.asarray(ref, dtype=np.float64).reshape(-1)
    den = np.linalg.norm(ref)
    num = np.linalg.norm(x - ref)
    if den == 0.0:
        return 0.0 if num == 0.0 else float("inf")
    return float(num / den)


def matmul_grad_calls(trans_a, trans_b, trans_out):
    """Flag triples of the two backward products of Tensor.matmul (Linalg.swift:73-80):
    dA = matmul(a: grad, transA: transOut, b: B, transB: !transB, transOut: transA)
    dB = matmul(a: A, transA: !transA, b: grad, transB: transOut, transOut: transB)."""
    return ((bool(trans_out), not trans_b, bool(trans_a)), (not trans_a, bool(trans_out), bool(trans_b)))


# ---- around a Linear layer -----------------------------------------------------------------

def broadcast_add_rows(h, bias, rows, cols):
    """binaryOp(.add) of h[rows,cols] and bias[cols] broadcast over rows, both of one dtype: widen
    to Float, add, narrow (Sources/Honeycrisp/BackendCPU.swift:295-303; float32 goes through
    vDSP_vadd only when neither side is broadcast, :276)."""
    h = np.asarray(h).reshape(rows, cols)
    bias = np.asarray(bias).reshape(cols)
    assert h.dtype == bias.dtype
    out = h.astype(np.float32) + bias.astype(np.float32)[None, :]
    return (out.astype(h.dtype) if h.dtype == np.float32 else float_to_half(out)).reshape(-1)


def linear_forward(x, weight, bias, rows, in_count, out_count):
    """Linear.callAsFunction (Sources/Honeycrisp/Trainable.swift:530-546): matmul with no flags,
    then the broadcast add of the bias when there is one."""
    h = matmul(x, False, weight, False, False, rows, in_count, out_count)
    return h if bias is None else broadcast_add_rows(h, bias, rows, out_count)


def column_sum(x, rows, cols):
    """reduce(.sum) over the leading axis: one Float accumulator per column, rows ascending,
    narrowed once (BackendCPU.swift:808-827).  For float32 the reference calls vDSP_sve
    (:792-806), whose order is unknown; this is the literal loop for both dtypes."""
    x = np.asarray(x).reshape(rows, cols)
    acc = np.zeros(cols, dtype=np.float32)
    for r in range(rows):
        acc = acc + x[r].astype(np.float32)
    return acc if x.dtype == np.float32 else float_to_half(acc)


def cast(x, out_dtype):
    """Backend.cast through Float (BackendCPU.swift:2018-2058)."""
    x = np.asarray(x)
    if out_dtype == np.float16:
        return float_to_half(x.astype(np.float32))
    return x.astype(np.float32)


def add(a, b):
    """binaryOp(.add) on equal shapes: widen, add, narrow."""
    a, b = np.asarray(a), np.asarray(b)
    out = a.astype(np.float32) + b.astype(np.float32)
    return out if a.dtype == np.float32 else float_to_half(out).reshape(a.shape)


# ---- the generator behind Tensor(rand:) / Tensor(randn:) ------------------------------------

def philox4x32_10(seed, offsets):
    """Philox-4x32-10 as Sources/Honeycrisp/BackendCPU.swift:177-199 writes it: counter
    (offset_lo, offset_hi, 0, 0), key (seed_lo, seed_hi).  `offsets`: uint64 array; returns
    uint32 [len, 4]."""
    offsets = np.asarray(offsets, dtype=np.uint64)
    c0 = (offsets & np.uint64(0xFFFFFFFF)).astype(np.uint64)
    c1 = (offsets >> np.uint64(32)).astype(np.uint64)
    c2 = np.zeros_like(c0)
    c3 = np.zeros_like(c0)
    k0 = np.uint64(int(seed) & 0xFFFFFFFF)
    k1 = np.uint64((int(seed) >> 32) & 0xFFFFFFFF)
    A, B, M = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57), np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0, p2 = c0, c2
        pb, pa = B * p2, A * p0
        c0 = (pb >> np.uint64(32)) ^ c1 ^ k0
        c2 = (pa >> np.uint64(32)) ^ c3 ^ k1
        c1 = pb & M
        c3 = pa & M
        k0 = (k0 + np.uint64(0x9E3779B9)) & M
        k1 = (k1 + np.uint64(0xBB67AE85)) & M
    return np.stack([c0, c1, c2, c3], axis=1).astype(np.uint32)


def random_sample(seed, offset, count, dist, dtype):
    """CPURandomGenerator._sample (BackendCPU.swift:78-123).  Returns (values, next_offset)."""
    if dist == "uniform":
        n = count // 4 + 1                       # stride(from: 0, through: count, by: 4)
        words = philox4x32_10(seed, np.arange(n, dtype=np.uint64) + np.uint64(offset)).reshape(-1)[:count]
        vals = (words.astype(np.float64) / np.float64(0xFFFFFFFF)).astype(np.float32)
    else:
        n = count // 2 + 1                       # stride(from: 0, through: count, by: 2)
        w = philox4x32_10(seed, np.arange(n, dtype=np.uint64) + np.uint64(offset))
        # Loop index i (one counter value) writes positions i..i+3 from its word pairs (c0,c1) and
        # (c2,c3); index i+2 then overwrites i+2 and i+3.  So every position below `count` ends up
        # holding the (c0,c1) pair of the counter value number floor(position / 2).
        denom = np.float32(0xFFFFFFFF)           # Float(0xffff_ffff) == 2^32
        u1 = np.maximum(np.float32(1e-5), w[:, 0].astype(np.float32) / denom)
        u2 = w[:, 1].astype(np.float32) / denom
        r = np.sqrt(np.float32(-2.0) * np.log(u1))
        phi = np.float32(2.0) * np.float32(np.pi) * u2
        pairs = np.stack([(r * np.cos(phi)).astype(np.float32), (r * np.sin(phi)).astype(np.float32)], axis=1)
        vals = pairs.reshape(-1)[:count]
    vals = vals if dtype == np.float32 else float_to_half(vals)
    return vals, int(offset) + n

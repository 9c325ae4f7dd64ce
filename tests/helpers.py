"""Shared helpers of the test-suite: golden vectors, seeded operands in stored layout."""
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
FLAG_COMBOS = [(ta, tb, to) for ta in (False, True) for tb in (False, True) for to in (False, True)]


def golden():
    with open(os.path.join(HERE, "golden", "matmul_vectors.json")) as f:
        return json.load(f)


def stored(logical, trans):
    """Storage of a logical [..., r, c] operand: transposed per matrix when its flag is set."""
    x = np.asarray(logical)
    if trans:
        x = np.swapaxes(x, -1, -2)
    return np.ascontiguousarray(x)


def logical_out(flat, count, rows, cols, trans_out):
    """Logical [count, rows, cols] view of a flat result."""
    x = np.asarray(flat).reshape(-1)
    if trans_out:
        return np.swapaxes(x.reshape(count, cols, rows), -1, -2)
    return x.reshape(count, rows, cols)


def random_operands(seed, count, rows, inner, cols, dtype, dist="normal", scale=1.0):
    """Seeded logical operands A[count,rows,inner], B[count,inner,cols] of `dtype`."""
    rng = np.random.default_rng(seed)
    if dist == "normal":
        A = rng.standard_normal((count, rows, inner), dtype=np.float32) * scale
        B = rng.standard_normal((count, inner, cols), dtype=np.float32) * scale
    elif dist == "uniform01":
        A = rng.random((count, rows, inner), dtype=np.float32)
        B = rng.random((count, inner, cols), dtype=np.float32)
    elif dist == "uniform11":
        A = rng.random((count, rows, inner), dtype=np.float32) * 2 - 1
        B = rng.random((count, inner, cols), dtype=np.float32) * 2 - 1
    elif dist == "smallint":
        A = rng.integers(-4, 5, (count, rows, inner)).astype(np.float32)
        B = rng.integers(-4, 5, (count, inner, cols)).astype(np.float32)
    else:
        raise ValueError(dist)
    return A.astype(dtype), B.astype(dtype)

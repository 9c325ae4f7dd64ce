"""Writes tests/golden/matmul_vectors.json: the known-answer vectors of the reference's own
matrix-product tests, transcribed from the test source (read as text; the reference cannot be
run on Linux).  Each entry names the lines it comes from, paths relative to the Honeycrisp
project.  Run `python tests/golden/make_vectors.py` to regenerate.
"""
import json
import os

VECTORS = {
    "matrix_matrix_product": {
        "source": "Sources/HCTestUtils/BackendTests.swift:684-712",
        "note": "for all 8 (transA, transB, transOut) and both float dtypes; exact equality",
        "x": [1, 2, 3, 4, 5, 6],
        "x_shape": [2, 3],
        "y_before_t": [-1, -2, -3, -4, -5, -6, -7, -8, -9, -10, -11, -12],
        "y_before_t_shape": [4, 3],
        "out_grad": [8, 7, 6, 5, 4, 3, 2, 1],
        "out_shape": [2, 4],
        "out": [-14, -32, -50, -68, -32, -77, -122, -167],
        "a_grad": [-128.0, -154.0, -180.0, -40.0, -50.0, -60.0],
        "b_grad": [24.0, 19.0, 14.0, 9.0, 36.0, 29.0, 22.0, 15.0, 48.0, 39.0, 30.0, 21.0],
    },
    "ones_product": {
        "source": "Sources/HCTestUtils/BackendTests.swift:713-725",
        "note": "ones[64,128] x ones[128,32] == 128 exactly in float32; float16 result finite; "
                "with both operands x1000 the float16 result is not finite",
        "a_shape": [64, 128],
        "b_shape": [128, 32],
        "value": 128.0,
        "overflow_scale": 1000.0,
    },
    "matrix_vector_product": {
        "source": "Sources/HCTestUtils/BackendTests.swift:769-783",
        "note": "float32, upstream gradient of ones; exact equality",
        "x": [1, 2, 3, 4, 5, 6],
        "x_shape": [2, 3],
        "y": [-1, -3, 2],
        "y_shape": [3, 1],
        "out": [-1, -7],
        "x_grad": [-1, -3, 2, -1, -3, 2],
        "y_grad": [5, 7, 9],
    },
    "batched_vs_single": {
        "source": "Sources/HCTestUtils/BackendTests.swift:728-767",
        "note": "random [3,2,3] x [3,3,4]; batched output and both gradients must match the "
                "per-matrix products within atol=rtol=eps",
        "x_shape": [3, 2, 3],
        "y_shape": [3, 3, 4],
        "eps_float32": 1e-4,
        "eps_float16": 1e-2,
    },
    "concurrent_backward": {
        "source": "Tests/HoneycrispTests/HoneycrispTests.swift:847-871",
        "note": "100 concurrent [128,16] x [16,1] products and backward passes from detached tasks",
        "a_shape": [128, 16],
        "b_shape": [16, 1],
        "count": 100,
    },
}

if __name__ == "__main__":
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "matmul_vectors.json")
    with open(path, "w") as f:
        json.dump(VECTORS, f, indent=1)
        f.write("\n")
    print(path)

"""A/B of libhccuda.so and libhccuda_mc.so in one process: bitwise equality and timing."""
import json, sys, time
import numpy as np
from honeycrisp_b200 import CUDABackend, _lib

be0 = CUDABackend(0)
be1 = CUDABackend(0, multicast=True)
res = {}

def dev_arr(be, arr):
    return be.collection(arr.reshape(-1), arr.dtype)

def run(be, a_d, b_d, ta, tb, tout, M, K, N, out=None, batch=1):
    if batch == 1:
        return be.matmul(a_d, ta, b_d, tb, tout, M, K, N, np.float16, out=out)
    return be.batchedMatmul(batch, a_d, ta, b_d, tb, tout, M, K, N, np.float16, out=out)

def check(M, K, N, ta, tb, tout=False, batch=1, seed=0):
    rng = np.random.default_rng(seed)
    a = (rng.standard_normal((batch, M * K)) / np.sqrt(K)).astype(np.float16)
    b = rng.standard_normal((batch, K * N)).astype(np.float16)
    outs = []
    info = []
    for be in (be0, be1):
        a_d, b_d = dev_arr(be, a), dev_arr(be, b)
        o = run(be, a_d, b_d, ta, tb, tout, M, K, N, batch=batch)
        info.append(be.lastLaunchInfo())
        outs.append(o.onCPU(np.float16)[: batch * M * N].copy())
        be.checkDeviceStatus()
    same = bool(np.array_equal(outs[0].view(np.uint16), outs[1].view(np.uint16)))
    key = f"{batch}x{M}x{K}x{N} {int(ta)}{int(tb)}{int(tout)}"
    res[key] = {"same_bits": same, "tile0": [info[0]["tile_m"], info[0]["tile_n"]], "tile1": [info[1]["tile_m"], info[1]["tile_n"]],
                "grid1": info[1]["grid"], "finite": bool(np.isfinite(outs[1].astype(np.float32)).all())}
    print(key, res[key], flush=True)
    return same

ok = True
for (M, K, N) in [(1024, 1024, 1024), (2048, 2048, 2048), (4096, 4096, 4096)]:
    for ta in (False, True):
        for tb in (False, True):
            ok &= check(M, K, N, ta, tb)
ok &= check(4096 + 256, 2048, 4096 + 128, False, True)
ok &= check(4096 + 264, 2048, 2048 + 72, False, False)
ok &= check(2048, 4096, 2048, True, False, tout=True)
ok &= check(1024, 2048, 2048, False, True, batch=3)
ok &= check(512, 1024, 1024, False, False)
res["all_same"] = bool(ok)

def timeit(be, M, K, N, ta, tb, reps):
    rng = np.random.default_rng(1)
    a = (rng.standard_normal(M * K) / np.sqrt(K)).astype(np.float16)
    b = rng.standard_normal(K * N).astype(np.float16)
    a_d, b_d = dev_arr(be, a), dev_arr(be, b)
    out = be.allocate(M * N * 2)
    for _ in range(3):
        run(be, a_d, b_d, ta, tb, False, M, K, N, out=out)
    m0 = be.marker()
    for _ in range(reps):
        run(be, a_d, b_d, ta, tb, False, M, K, N, out=out)
    m1 = be.marker()
    m1.wait()
    return m0.elapsedMs(m1) / reps

if ok:
    for (M, K, N, ta, tb, reps) in [(8192, 8192, 8192, False, True, 20), (8192, 8192, 8192, False, False, 20),
                                    (8192, 8192, 8192, True, False, 20), (8192, 8192, 8192, True, True, 20),
                                    (16384, 4096, 16384, False, True, 8), (4096, 4096, 4096, False, True, 40),
                                    (16384, 16384, 16384, False, True, 3)]:
        rows = []
        for rnd in range(3):
            t0 = timeit(be0, M, K, N, ta, tb, reps)
            t1 = timeit(be1, M, K, N, ta, tb, reps)
            rows.append((t0, t1))
        fl = 2.0 * M * K * N
        t0 = sorted(r[0] for r in rows)[1]; t1 = sorted(r[1] for r in rows)[1]
        key = f"time {M}x{K}x{N} {int(ta)}{int(tb)}"
        res[key] = {"plain_ms": t0, "mc_ms": t1, "plain_tflops": fl / t0 / 1e9, "mc_tflops": fl / t1 / 1e9, "ratio": t0 / t1, "rounds": rows}
        print(key, res[key], flush=True)
    # sustained: 1.2 s each, alternating
    for name, be in (("plain", be0), ("mc", be1), ("plain2", be0), ("mc2", be1)):
        t = timeit(be, 8192, 8192, 8192, False, True, 1200)
        res["sustained_" + name] = 2.0 * 8192**3 / t / 1e9
        print("sustained", name, res["sustained_" + name], flush=True)
print(json.dumps(res))
print("ALL_SAME", ok)

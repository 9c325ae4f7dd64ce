#!/usr/bin/env python
"""Benchmark of the dense matrix-product hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--all-configs]

One step = one pass of the headline workload: float16 GEMM M=N=K=8192, fp32 accumulate, over
all four transA/transB combinations (four products, 4.398 TFLOP).  With N > 1 (launched by
torchrun, one rank per GPU) every rank runs that step on its own operands - independent
products, nothing exchanged - and `value` is the aggregate over the box (replicas: weak scaling).
The configurations that SHARD are timed in the same run and reported under `sharded`: the
batched attention-score product split over the batch (no collective) and the float32 16384^3
product split over columns, exchanged by NCCL all-gather and by the fused epilogue push; each
with the whole problem timed on rank 0 alone in the same run, the same way, as its 1-GPU time.
At N = 1 `configs` holds the single-GPU roofline blocks of the other configurations.

Prints ONE JSON line on stdout (rank 0).  `value` is timed with operands resident in HBM;
`e2e` is the same step from pinned host buffers through the C ABI (inputs copied to the device once
per step, four products, four results read back), copies inside the timed region.
`--impl reference` times the reference's CPU path (the oracle port of CPUBackend's loop) on the
host cores instead.  `--all-configs` adds quick numbers for the other four configurations
under "extra".
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "GEMM TFLOP/s (box aggregate; per GPU = value / n_gpus)"
UNIT = "TFLOP/s"
N_DIM = 8192
COMBOS = [(False, False), (False, True), (True, False), (True, True)]  # (transA, transB)
WORKLOAD = "float16 GEMM M=N=K=8192, fp32 accumulate, float16 out, all four transA/transB, N(0,1)/sqrt(K), seed 1"
FLOPS_PER_GEMM = 2.0 * N_DIM ** 3
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one 8192^3 launch of the tensor-core
# kernel, from the latest ncu capture summarised under profiles/ (865 MB read + 120 MB written).
# The algorithmic minimum is 3 * 8192^2 * 2 = 403 MB.
NCU_DRAM_BYTES_PER_LAUNCH = 0.985e9
NCU_DRAM_SOURCE = ("ncu capture of tc_gemm_kernel<2, 256, 4, 8, 0, 2, 2, 1, 0> (256x512 pair tile, half-by-half drain) "
                   "at 8192^3, profiles/tc_gemm_f16_8192.md; not measured by this run")


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"burst": float(p["bf16_tflops"]), "sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "hbm_gbs": float(p["hbm_gbs"]), "source": "measured"}
    return {"burst": 1590.0, "sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """SM clock, power and throttle reasons of one GPU, sampled while the timed region runs.

    Read through NVML inside this process every few milliseconds (reading only; nothing is set), so
    that even a timed region of tens of milliseconds gets samples that lie inside it; where NVML
    cannot be loaded, an `nvidia-smi --query-gpu ... -lms` child process is used instead, whose
    start-up alone can outlast a short region."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []
        self.nvml = None
        self.handle = None
        self.samples = []      # (sm MHz, power W, reasons bit mask) from NVML
        self.running = False
        self.max_mhz = None
        try:
            import pynvml
            pynvml.nvmlInit()
            handle = None
            try:
                import torch
                props = torch.cuda.get_device_properties(index)
                bus = "%08x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
                handle = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
            except Exception:  # noqa: BLE001
                handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            self.nvml, self.handle = pynvml, handle
        except Exception:  # noqa: BLE001
            self.nvml = None

    def _poll(self):
        n, h = self.nvml, self.handle
        reasons_fn = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or n.nvmlDeviceGetCurrentClocksThrottleReasons
        while self.running:
            try:
                self.samples.append((float(n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM)),
                                     n.nvmlDeviceGetPowerUsage(h) / 1000.0, int(reasons_fn(h))))
            except Exception:  # noqa: BLE001
                break
            time.sleep(0.003)

    def start(self):
        if self.nvml:
            self.running = True
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def _stop_nvml(self):
        self.running = False
        self.thread.join(timeout=2)
        n = self.nvml
        bits = {"hw_slowdown": getattr(n, "nvmlClocksEventReasonHwSlowdown", 0x8),
                "hw_thermal_slowdown": getattr(n, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                "sw_thermal_slowdown": getattr(n, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                "sw_power_cap": getattr(n, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["no samples"]}
        sm = [x[0] for x in self.samples]
        power = [x[1] for x in self.samples]
        reasons = sorted(name for name, bit in bits.items() if any(x[2] & bit for x in self.samples))
        return {"sm_mhz": statistics.median(sm), "sm_min_mhz": min(sm), "sm_max_mhz": self.max_mhz,
                "power_w_max": max(power), "samples": len(sm), "reasons": reasons,
                "source": "NVML, every 3 ms inside the timed region"}

    def stop(self):
        if self.nvml and self.running:
            return self._stop_nvml()
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        for line in self.lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1])); power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(self.NAMES, parts[3:7]):
                if val == "Active":
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # "under load" = samples in the upper half of the power range seen
        cut = (max(power) + min(power)) / 2
        loaded = [s for s, p in zip(sm, power) if p >= cut] or sm
        return {"sm_mhz": statistics.median(loaded), "sm_max_mhz": max(mx), "power_w_max": max(power),
                "samples": len(sm), "reasons": sorted(reasons), "source": "nvidia-smi -lms 50"}


def bind_near_gpu(local):
    """Run this process (and first-touch its pinned buffers) on the CPUs of the GPU's own NUMA node,
    as read from sysfs.  Returns what was done, and the affinity to restore afterwards."""
    info = {"numa_node": None, "cpus_bound": None}
    before = None
    try:
        import torch
        pr = torch.cuda.get_device_properties(local)
        bdf = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        base = f"/sys/bus/pci/devices/{bdf}"
        node = int(open(base + "/numa_node").read().strip())
        info["numa_node"] = node
        cpus = set()
        for part in open(base + "/local_cpulist").read().strip().split(","):
            if not part:
                continue
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        before = os.sched_getaffinity(0)
        cpus &= before
        if node >= 0 and cpus and cpus != before:
            os.sched_setaffinity(0, cpus)
            info["cpus_bound"] = len(cpus)
    except Exception as e:  # noqa: BLE001 - placement is an optimisation of the measurement
        info["error"] = str(e)[:120]
    return info, before


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# ------------------------------------------------------------------------------------------------
# reference arm: the reference's CPU path on the host cores
# ------------------------------------------------------------------------------------------------

def cpu_sample(rows_per_combo: int, threads: int, a32, b32, out32):
    """One bounded sample of the workload on the CPU: `rows_per_combo` output rows of each of
    the four products through the oracle's loop.  Returns (seconds, flops)."""
    from oracle import reference_cpu as ref
    t0 = time.perf_counter()
    for ta, tb in COMBOS:
        ref.loop_rows(1, a32, ta, b32, tb, False, N_DIM, N_DIM, N_DIM, 0, rows_per_combo, threads=threads, out=out32)
    dt = time.perf_counter() - t0
    return dt, 4 * 2.0 * rows_per_combo * N_DIM * N_DIM


def cpu_sgemm_baseline(threads: int, a32, b32):
    """The reference's float32 fast path on the host: CPUBackend.matmul with no flags calls the
    platform sgemm (vDSP_mmul, BackendCPU.swift:1245-1258); here the same call through the host
    BLAS the oracle found.  Configuration 1 (1024^3, U[0,1), seed 0) on all cores and on one,
    and the headline shape (8192^3, float16 values widened) on all cores."""
    import numpy as np
    from oracle import reference_cpu as ref
    kind, _, where = ref.find_sgemm()
    if kind is None:
        return {"unavailable": where}
    rng = np.random.default_rng(0)
    a1 = rng.random((1024, 1024), dtype=np.float32); b1 = rng.random((1024, 1024), dtype=np.float32)

    def best_of(fn, reps, warm=True):
        if warm:
            fn()
        best = float("inf")
        for _ in range(reps):
            t0 = time.perf_counter(); fn(); best = min(best, time.perf_counter() - t0)
        return best

    out = {"library": where, "cores": threads}
    ref.set_sgemm_threads(threads)
    t = best_of(lambda: ref.matmul(a1, False, b1, False, False, 1024, 1024, 1024), 5)
    out["c1_1024_all_cores"] = {"ms": t * 1e3, "tflops": 2 * 1024 ** 3 / t / 1e12}
    ref.set_sgemm_threads(1)
    t = best_of(lambda: ref.matmul(a1, False, b1, False, False, 1024, 1024, 1024), 2)
    out["c1_1024_one_thread"] = {"ms": t * 1e3, "tflops": 2 * 1024 ** 3 / t / 1e12,
                                 "note": "the reference's CPU backend runs on one worker thread"}
    ref.set_sgemm_threads(threads)
    t = best_of(lambda: ref.matmul(a32, False, b32, False, False, N_DIM, N_DIM, N_DIM), 1, warm=False)
    out["headline_shape_8192_all_cores"] = {"ms": t * 1e3, "tflops": 2.0 * N_DIM ** 3 / t / 1e12}
    return out


def cpu_operands():
    import numpy as np
    rng = np.random.default_rng(1)
    scale = 1.0 / np.sqrt(N_DIM)
    # float16 operands widened once, as CPUBackend does before its loop (BackendCPU.swift:2018-2030);
    # the widening is outside the timed sample, which favours the CPU number.
    a32 = (rng.standard_normal((N_DIM, N_DIM), dtype=np.float32) * scale).astype(np.float16).astype(np.float32)
    b32 = (rng.standard_normal((N_DIM, N_DIM), dtype=np.float32) * scale).astype(np.float16).astype(np.float32)
    out32 = np.zeros(N_DIM * N_DIM, dtype=np.float32)
    return a32, b32, out32


def calibrate_rows(threads, a32, b32, out32, target_s):
    """Rows per product (a multiple of the thread count) so that one sample takes about target_s."""
    dt, _ = cpu_sample(threads, threads, a32, b32, out32)   # one row per thread
    per_row = dt / threads
    rows = int(max(threads, min(N_DIM, target_s / max(per_row, 1e-9))))
    rows = (rows // threads) * threads or threads
    if rows > threads:
        # Second point: throughput per row is not constant (caches, memory bandwidth shared by the
        # threads), so correct the estimate with a sample of the chosen size.
        dt, _ = cpu_sample(rows, threads, a32, b32, out32)
        if dt > 1.3 * target_s or dt < 0.6 * target_s:
            rows = int(max(threads, min(N_DIM, rows * target_s / dt)))
            rows = (rows // threads) * threads or threads
    return rows


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    a32, b32, out32 = cpu_operands()
    rows = calibrate_rows(threads, a32, b32, out32, target_s=2.0)
    for _ in range(args.warmup):
        cpu_sample(rows, threads, a32, b32, out32)
    t_total, f_total = 0.0, 0.0
    for _ in range(args.steps):
        dt, fl = cpu_sample(rows, threads, a32, b32, out32)
        t_total += dt
        f_total += fl
    value = f_total / t_total / 1e12
    sample = (f"{rows} of {N_DIM} output rows of each of the four products per step through the port of "
              f"CPUBackend's loop (float16 operands widened to float32 beforehand, fp32 accumulate), "
              f"OpenMP over rows on {threads} threads; the reference itself runs this loop on one thread")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t_total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 in, f32 accumulate",
        "data": "synthetic", "config": {"workload": WORKLOAD, "sampled": True},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------

def run_ours(args):
    import numpy as np
    import torch

    from honeycrisp_b200 import CUDABackend
    from honeycrisp_b200 import _lib as L

    rank, world, local = dist_env()
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(local)
    use_dist = world > 1
    if use_dist:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    placement, affinity_before = bind_near_gpu(local)

    be = CUDABackend(local)
    # The backend keeps its own stream, on which nothing but the library launches kernels (it may
    # then start a product's operand loads before the previous product has finished); torch only
    # records timing events there.  torch's own work (data generation, the vendor-library legs)
    # runs on torch's streams, separated from the backend's by device synchronisation.
    stream = torch.cuda.ExternalStream(be.stream(), device=torch.device("cuda", local))

    n = N_DIM
    gen = torch.Generator(device="cuda").manual_seed(1 + rank)
    a = (torch.randn((n, n), generator=gen, device="cuda") / n ** 0.5).half()
    b = (torch.randn((n, n), generator=gen, device="cuda") / n ** 0.5).half()
    out = torch.empty((n, n), device="cuda", dtype=torch.float16)
    out_d = be.wrap(out.data_ptr(), out.numel() * 2, out)
    torch.cuda.synchronize()

    def step():
        for ta, tb in COMBOS:
            be.matmul(a, ta, b, tb, False, n, n, n, np.float16, out=out_d)

    def barrier():
        if use_dist:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    be.checkDeviceStatus()

    sampler = ClockSampler(local)
    launches0 = be.launchCount()
    barrier()
    if rank == 0:
        sampler.start()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = e0.elapsed_time(e1)
    launches = be.launchCount() - launches0
    be.checkDeviceStatus()
    if use_dist:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        lt = torch.tensor([launches], device="cuda", dtype=torch.int64)
        dist.all_reduce(lt, op=dist.ReduceOp.SUM)
        launches = int(lt.item())
    total_flops = FLOPS_PER_GEMM * 4 * args.steps * world
    value = total_flops / (ms * 1e-3) / 1e12

    # ---- end to end: host buffers through hc_batched_matmul_host, copies in the timed region
    e2e_steps = max(1, min(args.steps, 10))
    ha = a.cpu().pin_memory()
    hb = b.cpu().pin_memory()
    hout = torch.empty((n, n), dtype=torch.float16).pin_memory()
    ha_np, hb_np, hout_np = ha.numpy(), hb.numpy(), hout.numpy().reshape(-1)

    houts = [torch.empty((n, n), dtype=torch.float16).pin_memory().numpy().reshape(-1) for _ in range(3)]
    houts.append(hout_np)

    def e2e_step():
        # Four products from pinned host operands to pinned host results; the library pipelines
        # copy-in / product / copy-out of neighbouring products.  The step ends when all four
        # results are in host memory.
        for (ta, tb), ho in zip(COMBOS, houts):
            be.batchedMatmulHost(1, ha_np, ta, hb_np, tb, False, n, n, n, np.float16, out=ho, asynchronous=True)
        be.hostSync()

    e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = time.perf_counter() - t0
    if use_dist:
        t = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_value = FLOPS_PER_GEMM * 4 * e2e_steps * world / e2e_s / 1e12
    h2d = 4 * 2 * n * n * 2
    d2h = 4 * n * n * 2

    # The same step the way a Tensor program issues it: A and B become device buffers once per
    # step (Backend.collection) and the four products use them; all four results are read back.
    # Reported beside `e2e` (which stages the operands for every product), not instead of it.
    # Two sets of device operands: the inputs of step i+1 are uploaded (side stream) while the
    # results of step i are still being read back; host links are full duplex.
    dab = [(be.allocate(n * n * 2), be.allocate(n * n * 2)) for _ in range(2)]
    # Two sets of result buffers, on the device and (pinned) on the host: the products of step i+1
    # run while the results of step i are still on their way to the host, so the link never idles.
    douts = [[be.allocate(n * n * 2) for _ in range(4)] for _ in range(2)]
    houts2 = [houts, [torch.empty((n, n), dtype=torch.float16).pin_memory().numpy().reshape(-1) for _ in range(4)]]

    def upload(step):
        da, db = dab[step % 2]
        return [da.writeFrom(ha_np.reshape(-1)), db.writeFrom(hb_np.reshape(-1))]

    def staged_steps(count):
        pending = upload(0)
        in_flight = []                              # read-backs of the previous step
        for step in range(count):
            da, db = dab[step % 2]
            for u in pending:
                be.enqueueWait(u)                   # the products wait on the device, not the host
            reads = []
            for (ta, tb), do, ho in zip(COMBOS, douts[step % 2], houts2[step % 2]):
                be.batchedMatmul(1, da, ta, db, tb, False, n, n, n, np.float16, out=do, mark=False)
                reads.append(do.readInto(ho))       # side stream: the next product runs meanwhile
            nxt = upload(step + 1) if step + 1 < count else []
            for r in in_flight:
                r.wait()                            # step i-1 has ended: its four results are in host memory,
            in_flight = reads                       # and its buffers are free for step i+1
            for u in pending:
                u.wait()
            pending = nxt
        for r in in_flight:
            r.wait()

    staged_steps(1)
    barrier()
    t0 = time.perf_counter()
    staged_steps(e2e_steps)
    barrier()
    staged_s = time.perf_counter() - t0
    if use_dist:
        t = torch.tensor([staged_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        staged_s = float(t.item())
    e2e_staged = {"value": FLOPS_PER_GEMM * 4 * e2e_steps * world / staged_s / 1e12, "unit": UNIT,
                  "h2d_bytes_per_step": world * 2 * n * n * 2, "d2h_bytes_per_step": world * d2h, "steps": e2e_steps,
                  "bytes_are": "whole job (all ranks), like value",
                  "what": ("A and B uploaded once per step (hc_h2d_async, the next step's while this step's results "
                           "are read back), four products on them, each result read back with hc_d2h_async while the "
                           "next product runs; a step has ended when its four results are in host memory, and the products "
                           "of the next step run meanwhile (two sets of result buffers)")}
    for d in [x for pair in dab for x in pair] + [x for four in douts for x in four]:
        d.free()

    # ---- per-launch timing of the dominant kernel for the roofline (events around each launch)
    evs = []
    for ta, tb in COMBOS * 2:
        s0 = torch.cuda.Event(enable_timing=True); s1 = torch.cuda.Event(enable_timing=True)
        s0.record(stream)
        be.matmul(a, ta, b, tb, False, n, n, n, np.float16, out=out_d)
        s1.record(stream)
        evs.append((s0, s1))
    torch.cuda.synchronize()
    launch_ms = statistics.mean(x.elapsed_time(y) for x, y in evs)
    info = be.lastLaunchInfo()

    # The other configurations, lightest first: products of tens of microseconds are bound by
    # latencies that scale with the SM clock, and the clock stays low for a while after seconds at
    # the power cap - so they are timed before the long legs, and a sharded time and its 1-GPU time
    # are always taken next to each other.
    sharded, single, sustained = None, None, None
    groups = None
    if not args.quick:
        from honeycrisp_b200.sharding import DeviceGroup
        groups = (DeviceGroup.fromTorchDistributed(be) if use_dist else DeviceGroup(be, 0, 1), DeviceGroup(be, 0, 1))
        sharded = {"world": world,
                   "how": "host-launched through hc_batched_matmul_sharded / hc_matmul_nsplit_allgather, CUDA events on "
                          "the context's stream, max over ranks; one_gpu_ms: the whole problem on rank 0 alone in this "
                          "run, the same way"}
        sharded.update(sharded_c3(be, groups, stream, rank, world))
        if world == 1:
            single = single_gpu_configs(be, stream, heavy=False)
        # Sustained regime: the same step for about a second and a half, so that the power cap has
        # settled (the default 20-100 steps end within the burst), with the vendor library's product
        # on the same operands timed the same way right after it.
        sustained = sustained_leg(be, stream, step, a, b, out, barrier, use_dist, world)

    link = link_probe(stream, use_dist, world)

    if not args.quick:
        sharded.update(sharded_c5(be, groups, stream, rank, world))   # collective: every rank takes part
        if world == 1:
            single.update(single_gpu_configs(be, stream, heavy=True))
        groups[1].close()
        groups[0].close()

    if rank != 0:
        if use_dist:
            dist.destroy_process_group()
        return

    if affinity_before:
        os.sched_setaffinity(0, affinity_before)      # the CPU baseline below uses every core again
    peaks = load_peaks()
    timed_s = ms * 1e-3
    # The sustained figure is the denominator for a timed region long enough for the power cap
    # to settle (hundreds of milliseconds); the burst figure otherwise.
    use_sustained = timed_s > 0.25
    peak = peaks["sustained"] if use_sustained else peaks["burst"]
    achieved = value / world
    roofline = {
        "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
        "peak_kind": ("sustained" if use_sustained else "burst") + " bf16 cuBLAS, of " + peaks["source"],
        "frac_of_burst": achieved / peaks["burst"], "frac_of_sustained": achieved / peaks["sustained"],
        "frac_of_nominal_2250": achieved / 2250.0,
        "single_launch_tflops": FLOPS_PER_GEMM / (launch_ms * 1e-3) / 1e12,
        "traffic": NCU_DRAM_BYTES_PER_LAUNCH, "traffic_source": NCU_DRAM_SOURCE,
        "traffic_algorithmic_bytes": 3 * N_DIM * N_DIM * 2,
        "algorithmic_flops_per_launch": FLOPS_PER_GEMM,
    }

    threads = os.cpu_count() or 1
    a32, b32, out32 = cpu_operands()
    rows = calibrate_rows(threads, a32, b32, out32, target_s=12.0)
    dt, fl = cpu_sample(rows, threads, a32, b32, out32)
    cpu_sgemm = cpu_sgemm_baseline(threads, a32, b32)
    cpu_baseline = {
        "value": fl / dt / 1e12, "unit": UNIT, "cores": threads, "kind": "port",
        "sample": (f"{rows} of {N_DIM} output rows of each of the four products ({dt:.1f} s) through the port of "
                   f"CPUBackend's loop, OpenMP over rows; the reference runs it on one thread"),
    }

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 in, f32 accumulate", "data": "synthetic",
        "config": {"workload": WORKLOAD, "products_per_step": 4, "l2": "inputs larger than L2 (384 MB per product)",
                   "kernel": info, "per_rank": "each rank runs the step on its own operands; no collective "
                   "(replicas - the configurations that shard are under `sharded`)"},
        "clocks": clocks,
        # The step as a Tensor program issues it: the step's inputs (A, B) go from pinned host memory to
        # the device once, the four products use them, all four results are read back to pinned host
        # memory (hc_h2d, hc_batched_matmul, hc_d2h_async).  Beside it the host-buffer call
        # (hc_batched_matmul_host_async), which stages both operands again for every product.
        "e2e": e2e_staged,
        "e2e_host_buffer_call_per_product": {
            "value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": world * h2d, "d2h_bytes_per_step": world * d2h,
            "steps": e2e_steps,
            "what": "hc_batched_matmul_host_async per product: A and B staged from host memory four times per step"},
        "gpu_launches": launches,
        "roofline": roofline,
        "cpu_baseline": cpu_baseline,
        "cpu_sgemm_baseline": cpu_sgemm,
    }
    line["e2e"]["link_probe"] = link
    line["e2e"]["host_placement"] = placement
    line["e2e"]["note"] = ("bound by the host link: the four results are 0.54 GB per step and rank, and every GPU of "
                           "this box hangs off the same host memory (link_probe: plain pinned-memory copies, all ranks "
                           "at once)")
    if sustained:
        line["sustained"] = sustained
    if sharded:
        line["sharded"] = sharded
    if single:
        line["configs"] = single
    if args.all_configs and world == 1:
        line["extra"] = other_configs(be, stream, rank, world)
    emit(line)
    if use_dist:
        dist.destroy_process_group()


def other_configs(be, stream, rank, world):
    """Quick device-resident numbers for configurations 1, 3, 4 and 5 (single GPU)."""
    import numpy as np
    import torch

    def timed(fn, iters):
        torch.cuda.synchronize()
        for _ in range(3):
            fn()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(iters):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    res = {}
    g = torch.Generator(device="cuda").manual_seed(0)
    a = torch.rand((1024, 1024), generator=g, device="cuda"); b = torch.rand((1024, 1024), generator=g, device="cuda")
    o = torch.empty((1024, 1024), device="cuda"); od = be.wrap(o.data_ptr(), o.numel() * 4, o)
    ms = timed(lambda: be.matmul(a, False, b, False, False, 1024, 1024, 1024, np.float32, out=od), 20)
    res["c1_f32_1024"] = {"ms": ms, "tflops": 2 * 1024 ** 3 / ms / 1e9}
    q = torch.randn((64, 2048, 128), generator=g, device="cuda").half(); k = torch.randn((64, 2048, 128), generator=g, device="cuda").half()
    o = torch.empty((64, 2048, 2048), device="cuda", dtype=torch.float16); od = be.wrap(o.data_ptr(), o.numel() * 2, o)
    ms = timed(lambda: be.batchedMatmul(64, q, False, k, True, False, 2048, 128, 2048, np.float16, out=od), 20)
    res["c3_f16_batched_qkT"] = {"ms": ms, "tflops": 2 * 64 * 2048 * 2048 * 128 / ms / 1e9,
                                 "hbm_gbs": (2 * 64 * 2048 * 128 * 2 + 64 * 2048 * 2048 * 2) / ms / 1e6}
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(20):
                be.batchedMatmul(64, q, False, k, True, False, 2048, 128, 2048, np.float16, out=od, mark=False)
        def replay():
            with torch.cuda.stream(stream):     # a replay goes to torch's current stream
                graph.replay()
        ms = timed(replay, 5) / 20
        res["c3_f16_batched_qkT_graph"] = {"ms": ms, "tflops": 2 * 64 * 2048 * 2048 * 128 / ms / 1e9}
        del graph
    except Exception as e:
        res["c3_f16_batched_qkT_graph"] = {"error": str(e)[:200]}
    del q, k, o
    x = torch.randn((16384, 4096), generator=g, device="cuda").half()
    w = ((torch.rand((16384, 4096), generator=g, device="cuda") - 0.5) / 32).half()
    dy = torch.randn((16384, 16384), generator=g, device="cuda").half()
    y = torch.empty((16384, 16384), device="cuda", dtype=torch.float16); yd = be.wrap(y.data_ptr(), y.numel() * 2, y)
    dx = torch.empty((16384, 4096), device="cuda", dtype=torch.float16); dxd = be.wrap(dx.data_ptr(), dx.numel() * 2, dx)
    dw = torch.empty((16384, 4096), device="cuda", dtype=torch.float16); dwd = be.wrap(dw.data_ptr(), dw.numel() * 2, dw)

    def triple():
        be.matmul(x, False, w, True, False, 16384, 4096, 16384, np.float16, out=yd)       # Y = X W^T
        be.matmul(dy, False, w, False, False, 16384, 16384, 4096, np.float16, out=dxd)    # dX = dY W
        be.matmul(x, True, dy, False, True, 4096, 16384, 16384, np.float16, out=dwd)      # dW = (X^T dY)^T = dY^T X

    ms = timed(triple, 5)
    res["c4_f16_linear_triple"] = {"ms": ms, "tflops": 3 * 2 * 16384 * 16384 * 4096 / ms / 1e9}
    del w, y, dx, dw
    # The same work as Honeycrisp's Linear issues it (weight [in,out]; forward with the bias add
    # fused into the epilogue; backward dX = dY.W^T, dW = X^T.dY, db = column sum of dY).
    from honeycrisp_b200 import Linear
    layer = Linear(be, 4096, 16384, dtype=np.float16, seed=3)

    def layer_step():
        layer.weightGrad = None
        layer.biasGrad = None
        layer(x, (16384, 4096))
        layer.backward(x, (16384, 4096), dy)

    ms = timed(layer_step, 5)
    res["linear_layer_fwd_bwd_f16"] = {"ms": ms, "tflops": 3 * 2 * 16384 * 16384 * 4096 / ms / 1e9,
                                       "includes": "fused bias add, bias-gradient column sum"}
    del x, dy, layer
    # The reference's own benchmark protocol (Sources/HCMatrixBench/Entrypoint.swift:12-27): fp16
    # `m1.t() &* m2`, one warm-up and one timed run including the wait, wall clock, 2*inner^2*outer
    # flop; only the square cases pass the reference's shape assert.  "folded" passes the transpose
    # as a flag instead of materialising it.
    proto = {}
    for inner in (512, 1024, 2048):
        be.seed(0)
        m1 = be.sample(inner * inner, "uniform", np.float16)
        m2 = be.sample(inner * inner, "uniform", np.float16)
        be.sync()

        def run_mat():
            t = be.transpose(m1, 1, inner, inner, np.float16)
            be.matmul(t, False, m2, False, False, inner, inner, inner, np.float16).wait()

        def run_fold():
            be.matmul(m1, True, m2, False, False, inner, inner, inner, np.float16).wait()

        out = {}
        for name, fn in (("materialised", run_mat), ("folded", run_fold)):
            fn()
            t0 = time.perf_counter()
            fn()
            dt = time.perf_counter() - t0
            out[name + "_gflops"] = 2.0 * inner ** 3 / dt / 1e9
        proto[str(inner)] = out
    res["hcmatrixbench_protocol_f16"] = proto
    a = torch.rand((16384, 16384), generator=g, device="cuda") * 2 - 1
    b = torch.rand((16384, 16384), generator=g, device="cuda") * 2 - 1
    o = torch.empty((16384, 16384), device="cuda"); od = be.wrap(o.data_ptr(), o.numel() * 4, o)
    ms = timed(lambda: be.matmul(a, False, b, False, False, 16384, 16384, 16384, np.float32, out=od), 2)
    res["c5_f32_16384_3xtf32"] = {"ms": ms, "tflops_effective": 2 * 16384 ** 3 / ms / 1e9}
    del a, b, o
    # The operations either side of a Linear product, each returning a fresh buffer (as the
    # reference's do), with the bytes they have to move: HBM-bound kernels.
    n = 8192 * 8192
    x32 = torch.randn(n, generator=g, device="cuda")
    x16 = x32.half()
    y16 = torch.randn(n, generator=g, device="cuda").half()
    dy = torch.randn((16384, 16384), generator=g, device="cuda").half()
    ops = {
        "column_sum_f16_16384x16384": (lambda: be.columnSum(dy, 16384, 16384, np.float16), 16384 * 16384 * 2),
        "cast_f32_to_f16_64M": (lambda: be.cast(x32, n, np.float32, np.float16), n * 6),
        "cast_f16_to_f32_64M": (lambda: be.cast(x16, n, np.float16, np.float32), n * 6),
        "add_f16_64M": (lambda: be.add(x16, y16, n, np.float16), n * 6),
        "add_f32_64M": (lambda: be.add(x32, x32, n, np.float32), n * 12),
        "transpose_f16_8192x8192": (lambda: be.transpose(x16, 1, 8192, 8192, np.float16), n * 4),
        "transpose_f32_8192x8192": (lambda: be.transpose(x32, 1, 8192, 8192, np.float32), n * 8),
    }
    lin = {}
    for name, (fn, nbytes) in ops.items():
        keep = [fn(), fn()]          # two results alive: the pool has both buffers before timing starts
        ms = timed(fn, 10)
        lin[name] = {"ms": ms, "tb_per_s": nbytes / ms / 1e9}
        del keep
    res["linear_ops"] = lin
    be.checkDeviceStatus()
    return res


def run_probe(args):
    """A few launches of ONE product, for profiler captures:
    `--probe M,K,N[,count] --dtype f16|f32 --flags tA,tB --steps K`.  Several products separated
    by `:` run one after the other in one process (a size sweep) and print one JSON list."""
    specs = args.probe.split(":")
    if len(specs) == 1:
        emit(probe_one(args, specs[0]))
    else:
        emit({"probes": [probe_one(args, spec) for spec in specs]})


def probe_one(args, spec):
    import numpy as np
    import torch

    from honeycrisp_b200 import CUDABackend

    dims = [int(x) for x in spec.split(",")]
    M, K, N = dims[:3]
    cnt = dims[3] if len(dims) > 3 else 1
    ta, tb = (bool(int(x)) for x in args.flags.split(","))
    npdt, tdt = (np.float16, torch.float16) if args.dtype == "f16" else (np.float32, torch.float32)
    be = CUDABackend(0)
    stream = torch.cuda.ExternalStream(be.stream(), device=torch.device("cuda", 0))   # events only; see run_ours
    lib_stream = torch.cuda.Stream()
    g = torch.Generator(device="cuda").manual_seed(1)
    a = (torch.randn((cnt, K, M) if ta else (cnt, M, K), generator=g, device="cuda") / K ** 0.25).to(tdt)
    b = (torch.randn((cnt, N, K) if tb else (cnt, K, N), generator=g, device="cuda") / K ** 0.25).to(tdt)
    out = torch.empty((cnt, M, N), device="cuda", dtype=tdt)
    od = be.wrap(out.data_ptr(), out.numel() * out.element_size(), out)
    torch.cuda.synchronize()
    be.batchedMatmul(cnt, a, ta, b, tb, False, M, K, N, npdt, out=od)
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        be.batchedMatmul(cnt, a, ta, b, tb, False, M, K, N, npdt, out=od, mark=False)
    e1.record(stream)
    torch.cuda.synchronize()
    be.checkDeviceStatus()
    ms = e0.elapsed_time(e1) / args.steps
    if args.graph:
        # the same launches replayed from a CUDA graph: device time without the host's launch rate
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(args.steps):
                be.batchedMatmul(cnt, a, ta, b, tb, False, M, K, N, npdt, out=od, mark=False)
        with torch.cuda.stream(stream):         # a replay goes to torch's current stream
            graph.replay()
            e0.record(stream)
            for _ in range(5):
                graph.replay()
            e1.record(stream)
        torch.cuda.synchronize()
        be.checkDeviceStatus()
        ms = e0.elapsed_time(e1) / (5 * args.steps)
    lib_ms = None
    if args.compare_library:
        # the vendor library (cuBLAS through torch.matmul) on the same operands, timed the same way
        if args.dtype == "f32":
            torch.backends.cuda.matmul.allow_tf32 = False
        A = a.transpose(-1, -2) if ta else a
        B = b.transpose(-1, -2) if tb else b
        ref_out = torch.empty_like(out)
        run_lib = lambda: torch.matmul(A, B, out=ref_out)
        torch.cuda.synchronize()
        with torch.cuda.stream(lib_stream):
            for _ in range(3):
                run_lib()
            if args.graph:
                g2 = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g2, stream=lib_stream):
                    for _ in range(args.steps):
                        run_lib()
                g2.replay()
                e0.record(lib_stream)
                for _ in range(5):
                    g2.replay()
                e1.record(lib_stream)
                torch.cuda.synchronize()
                lib_ms = e0.elapsed_time(e1) / (5 * args.steps)
            else:
                e0.record(lib_stream)
                for _ in range(args.steps):
                    run_lib()
                e1.record(lib_stream)
                torch.cuda.synchronize()
                lib_ms = e0.elapsed_time(e1) / args.steps
    info = be.lastLaunchInfo()
    be.close()
    return {"probe": [M, K, N, cnt], "dtype": args.dtype, "flags": [ta, tb], "ms": ms, "graph": bool(args.graph),
            "library_ms": lib_ms, "library_tflops": (2.0 * cnt * M * N * K / lib_ms / 1e9) if lib_ms else None,
            "tflops": 2.0 * cnt * M * N * K / ms / 1e9, "kernel": info}


def _max_over_ranks(x, use_dist):
    import torch
    if not use_dist:
        return float(x)
    import torch.distributed as dist
    t = torch.tensor([x], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sustained_leg(be, stream, step, a, b, out, barrier, use_dist, world):
    import torch
    n = N_DIM
    steps = 400
    barrier()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        step()
    e1.record(stream)
    barrier()
    ms = _max_over_ranks(e0.elapsed_time(e1), use_dist)
    res = {"steps": steps, "ms_per_step": ms / steps, "tflops": FLOPS_PER_GEMM * 4 * steps * world / ms / 1e9,
           "timed_s": ms / 1e3}
    views = [(a.t() if ta else a, b.t() if tb else b) for ta, tb in COMBOS]

    def lib_step():
        for x, y in views:
            torch.matmul(x, y, out=out)

    lib_stream = torch.cuda.Stream()
    with torch.cuda.stream(lib_stream):
        for _ in range(3):
            lib_step()
        barrier()
        e0.record(lib_stream)
        for _ in range(steps):
            lib_step()
        e1.record(lib_stream)
    barrier()
    lms = _max_over_ranks(e0.elapsed_time(e1), use_dist)
    res["library_same_run"] = {"what": "torch.matmul (cuBLAS) on the same operands, same four layouts, same loop",
                               "ms_per_step": lms / steps, "tflops": FLOPS_PER_GEMM * 4 * steps * world / lms / 1e9}
    res["ratio_to_library"] = lms / ms
    peaks = load_peaks()
    res["frac_of_sustained_peak"] = res["tflops"] / world / peaks["sustained"]
    return res


def link_probe(stream, use_dist, world):
    """Plain copies between pinned host memory and the device, every rank at once: what the host
    side of the box can deliver per GPU, the ceiling of any end-to-end number."""
    import torch
    stream = torch.cuda.current_stream()      # torch's copies run on torch's stream
    nbytes = 512 << 20
    host = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    dev = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    out = {"bytes": nbytes, "concurrent_ranks": world}
    for name, (dst, src) in (("h2d_gbs_per_gpu", (dev, host)), ("d2h_gbs_per_gpu", (host, dev))):
        dst.copy_(src, non_blocking=True)
        torch.cuda.synchronize()
        if use_dist:
            import torch.distributed as dist
            dist.barrier()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(4):
            dst.copy_(src, non_blocking=True)
        e1.record(stream)
        torch.cuda.synchronize()
        ms = _max_over_ranks(e0.elapsed_time(e1), use_dist)
        out[name] = 4 * nbytes / ms / 1e6
    return out


def _device_timed(fn, iters, stream, use_dist, warm=3):
    import torch
    torch.cuda.synchronize()                  # operands made on torch's stream are complete
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    if use_dist:
        import torch.distributed as dist
        dist.barrier()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(iters):
        fn()
    e1.record(stream)
    torch.cuda.synchronize()
    if use_dist:
        import torch.distributed as dist
        dist.barrier()
    return _max_over_ranks(e0.elapsed_time(e1) / iters, use_dist)


def sharded_c3(be, groups, stream, rank, world):
    """float16 batched Q.K^T (64 x [2048,128].[2048,128]^T) split over the batch, no collective:
    host-launched through the group entry point, device-timed, max over ranks; next to it the whole
    batch on rank 0 alone, same loop, three rounds alternating, medians."""
    import numpy as np
    import torch

    use_dist = world > 1
    grp, one = groups
    peaks = load_peaks()
    cnt, rows, inner, cols = 64, 2048, 128, 2048
    begin, count = grp.shard(cnt)
    g = torch.Generator(device="cuda").manual_seed(2)
    q = torch.randn((cnt, rows, inner), generator=g, device="cuda").half()
    k = torch.randn((cnt, cols, inner), generator=g, device="cuda").half()
    o = torch.empty(cnt * rows * cols, device="cuda", dtype=torch.float16)
    qp, kp, op = q[begin:].data_ptr(), k[begin:].data_ptr(), o.data_ptr()
    q0, k0 = q.data_ptr(), k.data_ptr()
    shard = lambda: grp.batchedMatmulSharded(cnt, qp, False, kp, True, False, rows, inner, cols, np.float16, op)
    whole = lambda: one.batchedMatmulSharded(cnt, q0, False, k0, True, False, rows, inner, cols, np.float16, op)
    shard_ms, whole_ms = [], []
    for _ in range(3):
        shard_ms.append(_device_timed(shard, 200, stream, use_dist, warm=10))
        t = _device_timed(whole, 50, stream, False, warm=5) if rank == 0 else 0.0
        whole_ms.append(_max_over_ranks(t, use_dist))
    ms, one_ms = statistics.median(shard_ms), statistics.median(whole_ms)
    flops = 2.0 * cnt * rows * cols * inner
    algo_bytes = 2 * cnt * rows * inner * 2 + cnt * rows * cols * 2
    c3 = {"ms": ms, "box_tflops": flops / ms / 1e9, "matrices_per_rank": count, "collective": "none",
          "box_algorithmic_gbs": algo_bytes / ms / 1e6, "rounds_ms": shard_ms,
          "one_gpu_ms": one_ms, "one_gpu_rounds_ms": whole_ms, "speedup_over_one_gpu": one_ms / ms,
          "roofline": {"bound": "hbm", "achieved": algo_bytes / world / ms / 1e6, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                       "frac": algo_bytes / world / ms / 1e6 / peaks["hbm_gbs"], "per": "GPU"}}
    del q, k, o
    be.checkDeviceStatus()
    return {"c3": c3}


def sharded_c5(be, groups, stream, rank, world):
    """float32 16384^3 split over columns: blocks exchanged by ncclAllGather + one unpack kernel
    (c5_nccl), or by the product kernel's epilogue with peer stores (c5_fused); and the whole product
    on rank 0 alone in the same run."""
    import numpy as np
    import torch

    from honeycrisp_b200.sharding import columnBlock

    use_dist = world > 1
    grp, one = groups
    peaks = load_peaks()
    res = {}
    n = 16384
    g = torch.Generator(device="cuda").manual_seed(4)
    a = torch.rand((n, n), generator=g, device="cuda") * 2 - 1
    b = torch.rand((n, n), generator=g, device="cuda") * 2 - 1
    flops = 2.0 * n ** 3
    gathered = (world - 1) / world * n * n * 4           # bytes every GPU receives
    c = torch.empty((n, n), device="cuda")
    ap, bp, cp = a.data_ptr(), b.data_ptr(), c.data_ptr()
    nccl = lambda: grp.matmulColumnSplit(ap, False, bp, False, n, n, n, np.float32, cp)
    cb, cw = columnBlock(n, rank, world)
    be_out = be.wrap(c.data_ptr(), n * n * 4, c)
    block_only = lambda: be.matmulColumnBlock(a, False, b, False, False, n, n, n, cb, cw, np.float32, out=be_out)
    # The whole call and this rank's block product alone, alternating (the clock under the power
    # cap drifts by a few per cent within seconds; alternating keeps the difference honest).
    whole_ms, block_ms = [], []
    nccl(); block_only()
    for _ in range(5):
        whole_ms.append(_device_timed(nccl, 1, stream, use_dist, warm=0))
        block_ms.append(_device_timed(block_only, 1, stream, use_dist, warm=0))
    ms, bms = statistics.median(whole_ms), statistics.median(block_ms)
    res["c5_nccl"] = {"ms": ms, "box_tflops_effective": flops / ms / 1e9, "gathered_bytes_per_gpu": gathered,
                      "block_product_ms": bms, "exchange_ms": max(ms - bms, 0.0),
                      "exchange_is": "ncclAllGather of the packed blocks + the unpack kernel (whole call minus block product)"}
    if world > 1 and ms > bms:
        res["c5_nccl"]["nvlink_gbs_in_per_gpu"] = gathered / (ms - bms) / 1e6
    nccl_result = c
    fused_out = grp.resultAllocate(n * n * 4)
    fp = fused_out.ptr
    fused = lambda: grp.matmulColumnSplit(ap, False, bp, False, n, n, n, np.float32, fp, fused=True)
    ms = _device_timed(fused, 5, stream, use_dist, warm=2)
    be.sync()
    nccl()
    be.sync()
    same = bool(torch.equal(fused_out.asTorch((n, n), torch.float32), nccl_result))
    res["c5_fused"] = {"ms": ms, "box_tflops_effective": flops / ms / 1e9, "gathered_bytes_per_gpu": gathered,
                       "equals_nccl_result": same,
                       "includes": "entry and exit flag barriers of every call"}
    if world > 1:
        res["c5_fused"]["nvlink_gbs_in_per_gpu_overlapped"] = gathered / ms / 1e6
    grp.resultFree(fused_out)
    one_ms = 0.0
    if rank == 0:
        whole = lambda: one.matmulColumnSplit(ap, False, bp, False, n, n, n, np.float32, cp)
        one_ms = _device_timed(whole, 3, stream, False, warm=1)
    one_ms = _max_over_ranks(one_ms, use_dist)
    for key in ("c5_nccl", "c5_fused"):
        res[key]["one_gpu_ms"] = one_ms
        res[key]["speedup_over_one_gpu"] = one_ms / res[key]["ms"]
        res[key]["roofline"] = {"bound": "tensor", "achieved": res[key]["box_tflops_effective"] / world,
                                "peak": peaks["burst"] / 6, "unit": "TFLOP/s (effective; 3xTF32 does 3x the MMA work at half the bf16 rate)",
                                "frac": res[key]["box_tflops_effective"] / world / (peaks["burst"] / 6), "per": "GPU"}
    del a, b, c
    be.checkDeviceStatus()
    return res


def single_gpu_configs(be, stream, heavy):
    """Roofline blocks on one GPU (host-launched, device-timed): configurations 1 and 3 (light), or
    configuration 5 (heavy)."""
    import numpy as np
    import torch
    peaks = load_peaks()
    res = {}
    g = torch.Generator(device="cuda").manual_seed(0)
    if not heavy:
        a = torch.rand((1024, 1024), generator=g, device="cuda"); b = torch.rand((1024, 1024), generator=g, device="cuda")
        o = torch.empty((1024, 1024), device="cuda"); od = be.wrap(o.data_ptr(), o.numel() * 4, o)
        ms = _device_timed(lambda: be.matmul(a, False, b, False, False, 1024, 1024, 1024, np.float32, out=od, mark=False),
                           200, stream, False, warm=10)
        tf = 2 * 1024 ** 3 / ms / 1e9
        res["c1_f32_1024"] = {"ms": ms, "tflops_effective": tf,
                              "roofline": {"bound": "latency (64 tiles, one wave); against the 3xTF32 tensor ceiling for scale",
                                           "achieved": tf, "peak": peaks["burst"] / 6, "unit": "TFLOP/s", "frac": tf / (peaks["burst"] / 6)}}
        q = torch.randn((64, 2048, 128), generator=g, device="cuda").half(); k = torch.randn((64, 2048, 128), generator=g, device="cuda").half()
        o = torch.empty((64, 2048, 2048), device="cuda", dtype=torch.float16); od = be.wrap(o.data_ptr(), o.numel() * 2, o)
        ms = _device_timed(lambda: be.batchedMatmul(64, q, False, k, True, False, 2048, 128, 2048, np.float16, out=od, mark=False),
                           50, stream, False, warm=5)
        nbytes = 2 * 64 * 2048 * 128 * 2 + 64 * 2048 * 2048 * 2
        res["c3_f16_batched_qkT"] = {"ms": ms, "tflops": 2 * 64 * 2048 * 2048 * 128 / ms / 1e9,
                                     "roofline": {"bound": "hbm", "achieved": nbytes / ms / 1e6, "peak": peaks["hbm_gbs"],
                                                  "unit": "GB/s", "frac": nbytes / ms / 1e6 / peaks["hbm_gbs"],
                                                  "algorithmic_bytes": nbytes}}
        del q, k, o
    else:
        n = 16384
        a = torch.rand((n, n), generator=g, device="cuda") * 2 - 1
        b = torch.rand((n, n), generator=g, device="cuda") * 2 - 1
        o = torch.empty((n, n), device="cuda"); od = be.wrap(o.data_ptr(), o.numel() * 4, o)
        ms = _device_timed(lambda: be.matmul(a, False, b, False, False, n, n, n, np.float32, out=od, mark=False), 3, stream, False, warm=1)
        tf = 2 * n ** 3 / ms / 1e9
        res["c5_f32_16384_3xtf32"] = {"ms": ms, "tflops_effective": tf,
                                      "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["burst"] / 6,
                                                   "unit": "TFLOP/s effective (3xTF32: 3x the MMA work at half the bf16 rate)",
                                                   "frac": tf / (peaks["burst"] / 6),
                                                   "frac_of_sustained": tf / (peaks["sustained"] / 6)}}
        del a, b, o
        # Configuration 4: the three products of a Linear layer's forward and backward pass as the
        # reference's autodiff issues them (Y = X.W^T, dX = dY.W, dW = dY^T.X through transOut).
        x = torch.randn((16384, 4096), generator=g, device="cuda").half()
        w = ((torch.rand((16384, 4096), generator=g, device="cuda") - 0.5) / 32).half()
        dy = torch.randn((16384, 16384), generator=g, device="cuda").half()
        y = torch.empty((16384, 16384), device="cuda", dtype=torch.float16); yd = be.wrap(y.data_ptr(), y.numel() * 2, y)
        dx = torch.empty((16384, 4096), device="cuda", dtype=torch.float16); dxd = be.wrap(dx.data_ptr(), dx.numel() * 2, dx)
        dw = torch.empty((16384, 4096), device="cuda", dtype=torch.float16); dwd = be.wrap(dw.data_ptr(), dw.numel() * 2, dw)

        def triple():
            be.matmul(x, False, w, True, False, 16384, 4096, 16384, np.float16, out=yd, mark=False)
            be.matmul(dy, False, w, False, False, 16384, 16384, 4096, np.float16, out=dxd, mark=False)
            be.matmul(x, True, dy, False, True, 4096, 16384, 16384, np.float16, out=dwd, mark=False)

        ms = _device_timed(triple, 5, stream, False, warm=2)
        tf = 3 * 2 * 16384 * 16384 * 4096 / ms / 1e9
        res["c4_f16_linear_triple"] = {"ms": ms, "tflops": tf,
                                       "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["burst"], "unit": "TFLOP/s",
                                                    "frac": tf / peaks["burst"], "frac_of_sustained": tf / peaks["sustained"]}}
        del x, w, dy, y, dx, dw
    be.checkDeviceStatus()
    return res


_REAL_STDOUT = None


def quiet_stdout():
    """Libraries (NCCL's version banner, for one) write to file descriptor 1.  The contract is
    one JSON line on stdout, so everything else is sent to stderr and the line is written to
    the saved descriptor."""
    global _REAL_STDOUT
    if _REAL_STDOUT is None:
        sys.stdout.flush()
        _REAL_STDOUT = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)


def emit(line: dict):
    out = _REAL_STDOUT or sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()


def main():
    quiet_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--all-configs", action="store_true")
    ap.add_argument("--quick", action="store_true", help="headline step only: no sustained leg, no sharded/other configurations")
    ap.add_argument("--probe", default=None, help="M,K,N[,count]: run one product a few times (profiler target)")
    ap.add_argument("--dtype", choices=["f16", "f32"], default="f16")
    ap.add_argument("--flags", default="0,1", help="transA,transB for --probe")
    ap.add_argument("--graph", action="store_true", help="--probe: time CUDA-graph replays of the launches")
    ap.add_argument("--compare-library", action="store_true", help="--probe: also time torch.matmul (cuBLAS)")
    args = ap.parse_args()
    if args.probe:
        run_probe(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

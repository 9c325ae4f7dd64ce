"""The benchmark's reference arm (the CPU port of the reference's loop, no GPU involved): it must
print exactly one JSON line on stdout with the keys the measurement contract names."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, lines
    d = json.loads(lines[0])
    assert d["impl"] == "reference"
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["value"] > 0 and d["higher_is_better"] is True and d["vs_baseline"] is None
    assert "workload" in d["config"]
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("port", "reference") and cb["cores"] >= 1 and cb["sample"] and cb["value"] == d["value"]
    e = d["e2e"]
    assert e["value"] == d["value"] and e["unit"] == d["unit"]
    assert e["h2d_bytes_per_step"] == 0 and e["d2h_bytes_per_step"] == 0


def test_reference_arm_under_a_multi_rank_launch_runs_on_rank_zero_only():
    env = dict(os.environ, RANK="1", LOCAL_RANK="1", WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29999")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                          "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=120, cwd=ROOT, env=env)
    assert out.returncode == 0, out.stderr[-2000:]
    assert out.stdout.strip() == ""        # the other ranks exit without work and without output


def _load_bench():
    import importlib.util
    spec = importlib.util.spec_from_file_location("hc_bench", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_clock_sampler_summarises_what_a_fake_nvml_reports():
    """The sampler only reads; here against a fake NVML: samples taken while it runs, the power-cap
    bit named, the median and the minimum clock reported."""
    import time
    import types
    bench = _load_bench()
    clocks = iter([1965, 1800, 1500, 1500, 1500] + [1400] * 10000)
    fake = types.SimpleNamespace(NVML_CLOCK_SM=1, nvmlDeviceGetClockInfo=lambda h, c: next(clocks),
                                 nvmlDeviceGetPowerUsage=lambda h: 987000,
                                 nvmlDeviceGetCurrentClocksEventReasons=lambda h: 0x4,
                                 nvmlClocksEventReasonSwPowerCap=0x4)
    s = bench.ClockSampler(0)
    s.nvml, s.handle, s.max_mhz = fake, object(), 1965.0
    s.start()
    time.sleep(0.06)
    out = s.stop()
    assert out["samples"] >= 5 and out["sm_max_mhz"] == 1965.0 and out["sm_min_mhz"] == 1400.0
    assert 1400.0 <= out["sm_mhz"] <= 1965.0
    assert out["reasons"] == ["sw_power_cap"] and abs(out["power_w_max"] - 987.0) < 1e-6


def test_clock_sampler_without_nvml_or_nvidia_smi_says_so():
    bench = _load_bench()
    s = bench.ClockSampler(0)
    if s.nvml is None:     # no GPU here: NVML does not initialise
        old = os.environ.get("PATH", "")
        os.environ["PATH"] = ""
        try:
            s.start()
            out = s.stop()
        finally:
            os.environ["PATH"] = old
        assert out["sm_mhz"] is None and out["reasons"]

"""bench.py on a machine without a GPU: the CPU arm's JSON line, the rank rule of that arm, the FLOP convention and
the clock-sample window."""
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def run_bench(*args, env=None):
    e = dict(os.environ)
    e.update(env or {})
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=600, env=e, cwd=ROOT)


def test_reference_arm_prints_one_contract_line():
    out = run_bench("--impl", "reference", "--workload", "c3", "--steps", "1", "--warmup", "0")
    assert out.returncode == 0, out.stderr
    lines = [l for l in out.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "fmha_fwd_tflops" and d["unit"] == "TFLOP/s"
    assert d["n_gpus"] == 1 and d["steps"] == 1 and d["warmup"] == 0 and d["higher_is_better"] is True
    assert d["value"] > 0 and d["ms_per_step"] > 0 and d["gpu_launches"] == 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["cpu_baseline"]["value"] == d["value"] == d["e2e"]["value"]
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert "S=4096" in d["config"]["workload"] and "slices per step" in d["config"]["sample"]


def test_reference_arm_runs_on_rank_0_only():
    out = run_bench("--impl", "reference", "--workload", "c3", "--gpus", "2", "--steps", "1", "--warmup", "0",
                    env={"RANK": "1", "LOCAL_RANK": "1", "WORLD_SIZE": "2"})
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_flop_convention_and_algorithmic_bytes():
    import bench
    # 4 B H S^2 D (src/fmha-pipeline/fmha_forward.cu:572-573), halved for a causal mask
    assert bench.flops_of(4, 16, 4096, 128, False) == 4 * 4 * 16 * 4096 * 4096 * 128
    assert bench.flops_of(2, 32, 8192, 128, True) == 2 * 2 * 32 * 8192 * 8192 * 128
    # Q + K + V read once, O (16 bit) written once
    assert bench.algo_bytes_of(bench.WORKLOADS["c4"]) == 4 * 2 * 8192 * 32 * 128 * 2
    assert bench.algo_bytes_of(bench.WORKLOADS["c5"]) == 3 * 4 * 8192 * 16 * 128 + 4 * 8192 * 16 * 128 * 2


def test_clock_sampler_uses_the_samples_of_the_timed_region():
    import bench

    class Done:
        def terminate(self): pass
        def wait(self, timeout=None): return 0

    s = bench.ClockSampler(0)
    s.proc = Done()
    t = time.monotonic()
    idle = "1965, 1965, 150.0, Not Active, Not Active, Not Active, Not Active"
    busy = "1600, 1965, 900.0, Not Active, Not Active, Not Active, Active"
    s.lines = [(t - 5.0 + 0.01 * i, idle) for i in range(50)] + [(t - 1.0 + 0.02 * i, busy) for i in range(10)]
    got = s.stop(t - 1.0, t - 0.8)
    assert got["sm_mhz"] == 1600.0 and got["window"] == "timed region" and got["reasons"] == ["sw_power_cap"]
    assert got["samples"] == 10 and got["power_w_max"] == 900.0
    # too few samples inside the window: everything collected is reported, and the line says so
    s2 = bench.ClockSampler(0)
    s2.proc = Done()
    s2.lines = [(t - 5.0, idle), (t - 4.9, idle), (t - 1.0, busy)]
    got = s2.stop(t - 1.0, t - 0.9)
    assert got["samples"] == 3 and got["window"] == "warm-up and timed region"

#!/usr/bin/env python
"""Headline benchmark: FMHA forward TFLOP/s on B200 (and the CPU reference arm).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c4|c3|c5]

One "step" is one pass of the hot path over one batch of synthetic input: a single
cfk_fmha_forward call (one kernel launch) on the workload's tensors.  The default workload is the
S=8192, D=128 causal bf16 forward of the baseline (B=2, H=32 per GPU); with N > 1 ranks every rank runs
its own (batch, head) slices of that size with no data-path collective (weak scaling), and the value is
the FLOPs of all ranks over the slowest rank's device time.  FLOP convention: 4*B*H*Sq*Skv*D, halved
for causal (the reference's formula, src/fmha-pipeline/fmha_forward.cu:572-573, which has no causal
mode).  Inputs are seeded synthetic N(0,1) tensors; the reference measures on the same kind of data
(fmha_forward.cu:489-500).

Prints ONE JSON line on rank 0.  `--impl reference` times the CPU restatement of the reference's
unfused attention (oracle/) on the host cores for the same config, on a bounded sample per step.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "cutlass-kernels_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

WORKLOADS = {
    # name: (dtype code, B, H, S, D, causal, description)
    "c4": (1, 2, 32, 8192, 128, True, "fmha_fwd bf16 causal B=2 H=32 S=8192 D=128 (per GPU), out fp16"),
    "c3": (0, 4, 16, 4096, 128, False, "fmha_fwd fp16 B=4 H=16 S=4096 D=128 (per GPU), out fp16 + lse"),
    "c5": (2, 4, 16, 8192, 128, False, "fmha_fwd e4m3 B=4 H=16 S=8192 D=128 (per GPU), per-tensor scales, out fp16"),
}
DT_NAME = {0: "fp16", 1: "bf16", 2: "e4m3"}
NOMINAL = {0: 2250.0, 1: 2250.0, 2: 4500.0}


# DRAM bytes (read + write) of ONE launch of the FMHA kernel per workload, from one ncu capture of the CLI
# driver on the same shape (the files under profiles/ give the commands).  The algorithmic bytes are Q + K + V
# read once and O written once; the excess is K/V re-read by query blocks that missed them in L2.
NCU_DRAM_BYTES_PER_LAUNCH = {"c4": 715.0e6, "c3": 253.3e6, "c5": 310.4e6}


def algo_bytes_of(wl):
    dt, B, H, S, D, causal, _ = wl
    n = B * H * S * D
    return n * (3 * (1 if dt == 2 else 2) + 2)     # Q, K, V in the input type; O in fp16


def flops_of(B, H, S, D, causal):
    return 4.0 * B * H * S * S * D * (0.5 if causal else 1.0)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    return 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a timed region runs."""

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
            "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={q}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def wait_first(self, limit_s=1.5):
        """Blocks until nvidia-smi has delivered its first sample (it needs a few hundred ms to start)."""
        t0 = time.monotonic()
        while self.proc and not self.lines and time.monotonic() - t0 < limit_s:
            time.sleep(0.01)

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.monotonic(), line.strip()))

    def stop(self, t_begin=None, t_end=None):
        """Summary of the samples that arrived between t_begin and t_end (time.monotonic(); a sample is printed
        up to one interval after it was taken), or of all samples if fewer than three fall inside."""
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        inside = [l for (t, l) in self.lines
                  if (t_begin is None or t >= t_begin) and (t_end is None or t <= t_end + 0.03)]
        window = "timed region"
        if len(inside) < 3:
            inside, window = [l for (_, l) in self.lines], "warm-up and timed region"
        for l in inside:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1])); pw.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm_sorted = sorted(sm)
        return {"sm_mhz": sm_sorted[len(sm_sorted) // 2], "sm_max_mhz": max(mx), "power_w_max": max(pw),
                "samples": len(sm), "window": window, "reasons": sorted(reasons)}


def make_inputs(torch, lib, wl, seed, device):
    """Seeded N(0,1) Q/K/V for the workload, generated on the device by the library's fill kernel
    (e4m3: quantised with a per-tensor scale amax/448)."""
    import cfk_b200
    dt, B, H, S, D, causal, _ = wl
    n = B * S * H * D
    tdt = {0: torch.float16, 1: torch.bfloat16, 2: torch.float8_e4m3fn}[dt]
    outs, scales = [], []
    for i in range(3):
        if dt == 2:
            f = torch.empty(n, dtype=torch.float32, device=device)
            lib.fill(f, cfk_b200.FP32, n, seed + 1 + i, "normal")
            s = float(f.abs().max()) / 448.0
            t = torch.empty(B, S, H, D, dtype=tdt, device=device)
            lib.convert(f, cfk_b200.FP32, t, cfk_b200.E4M3, n, 1.0 / s)
            del f
        else:
            s = 1.0
            t = torch.empty(B, S, H, D, dtype=tdt, device=device)
            lib.fill(t, dt, n, seed + 1 + i, "normal")
        outs.append(t)
        scales.append(s)
    return outs, scales


def fmha_call(lib, wl, q, k, v, o, scales, lse=None, iterations=1, stream=None):
    dt, B, H, S, D, causal, _ = wl
    lib.fmha_forward(q, k, v, o, dtype=dt, batch=B, heads=H, seqlen_q=S, seqlen_kv=S, head_dim=D,
                     softmax_scale=1.0 / math.sqrt(D), causal=causal, lse=lse, q_descale=scales[0],
                     k_descale=scales[1], v_descale=scales[2], iterations=iterations, stream=stream)


def cpu_attention_sample(orc, torch, wl, qkv_f32_slices, budget_s):
    """Times the CPU oracle on whole (batch, head) slices of the workload until ~budget_s is used."""
    dt, B, H, S, D, causal, _ = wl
    per_slice = flops_of(1, 1, S, D, causal)
    done, t_total = 0, 0.0
    for (q, k, v) in qkv_f32_slices:
        t0 = time.perf_counter()
        orc.attention(q, k, v, 1.0 / math.sqrt(D), causal)
        t_total += time.perf_counter() - t0
        done += 1
        if t_total >= budget_s:
            break
    return done, t_total, done * per_slice / t_total / 1e12


def slices_for_cpu(torch, wl, q, k, v, scales, count):
    """float32 copies of `count` (batch, head) slices, shaped [1][S][1][D] (de-quantised values)."""
    dt, B, H, S, D, causal, _ = wl
    out = []
    for i in range(count):
        b, h = (i // H) % B, i % H
        out.append(tuple((x[b:b + 1, :, h:h + 1, :].float() * s).cpu().numpy() for x, s in zip((q, k, v), scales)))
    return out


def run_reference(args, wl, rank, world):
    """CPU arm: the oracle's unfused fp32 attention on the host cores.  One step = a bounded sample of
    the workload: `slices` whole (batch, head) problems of the same S, D and mask."""
    if rank != 0:
        return
    # torchrun exports OMP_NUM_THREADS=1 to its workers; this arm is the only work of the job, so it takes
    # every core the process may run on (the OpenMP runtime reads the variable when the oracle is loaded).
    if "TORCHELASTIC_RUN_ID" in os.environ or world > 1:
        os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))
    from oracle.oracle import CfkOracle
    orc = CfkOracle()
    dt, B, H, S, D, causal, desc = wl
    per_slice = flops_of(1, 1, S, D, causal)
    rng_shape = (1, S, 1, D)
    q, k, v = (orc.fill(rng_shape, seed=3081 + i) for i in range(3))
    if dt != 2:
        q, k, v = (orc.dequantize(orc.quantize(x, DT_NAME[dt]), DT_NAME[dt]) for x in (q, k, v))
    t0 = time.perf_counter()
    orc.attention(q, k, v, 1.0 / math.sqrt(D), causal)
    t_one = time.perf_counter() - t0
    total_steps = args.steps + args.warmup
    slices = max(1, min(8, int(120.0 / max(t_one, 1e-3) / max(total_steps, 1))))
    for _ in range(args.warmup):
        for _ in range(slices):
            orc.attention(q, k, v, 1.0 / math.sqrt(D), causal)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        for _ in range(slices):
            orc.attention(q, k, v, 1.0 / math.sqrt(D), causal)
    dt_s = time.perf_counter() - t0
    value = args.steps * slices * per_slice / dt_s / 1e12
    sample = f"{slices} of {B * H} (batch, head) slices per step, full S={S}, D={D}, causal={causal}"
    line = {
        "impl": "reference", "metric": "fmha_fwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt_s / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": desc, "accumulate": "fp32", "algorithmic_bytes_per_launch": algo_bytes_of(wl), "flop_convention": "4*B*H*S*S*D, halved for causal", "sample": sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": orc.threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "CPU restatement of the reference's unfused fp32 attention (include/utils/fmha_cutlass.hpp:154-317); "
                "the reference's own kernels are sm_90a-only and its checker needs CUTLASS, so neither runs here",
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c4", choices=sorted(WORKLOADS))
    ap.add_argument("--no-extras", action="store_true", help="skip the secondary configs and the CPU baseline")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    wl = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, wl, rank, world)
        return

    import torch
    import torch.distributed as dist

    import cfk_b200
    lib = cfk_b200.load()      # no fallback: raises if the CUDA library is missing
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    dt, B, H, S, D, causal, desc = wl
    (q, k, v), scales = make_inputs(torch, lib, wl, seed=3080 + 1000 * rank, device=device)
    o = torch.full((B, S, H, D), -1.0, dtype=torch.float16, device=device)
    lse = torch.empty(B, H, S, dtype=torch.float32, device=device)
    stream = torch.cuda.current_stream()
    sptr = stream.cuda_stream
    step_flops = flops_of(B, H, S, D, causal)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing (value) ----
    for _ in range(args.warmup):
        fmha_call(lib, wl, q, k, v, o, scales, lse, stream=sptr)
    lib.check_device()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        sampler.wait_first()
    barrier()
    t_begin = time.monotonic()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        fmha_call(lib, wl, q, k, v, o, scales, lse, stream=sptr)
    e1.record(stream)
    barrier()
    t_end = time.monotonic()
    ms = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None
    lib.check_device()
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    value = world * step_flops / (ms_max * 1e-3) / 1e12

    # ---- end-to-end through the C ABI with host buffers (e2e) ----
    hq, hk, hv = (torch.empty(x.shape, dtype=x.dtype, pin_memory=True) for x in (q, k, v))
    for h, d in zip((hq, hk, hv), (q, k, v)):
        h.copy_(d)
    ho = torch.empty(o.shape, dtype=o.dtype, pin_memory=True)
    h2d = sum(x.numel() * x.element_size() for x in (hq, hk, hv))
    d2h = ho.numel() * ho.element_size()
    e2e_steps = max(4, min(args.steps, 16))

    # Every step copies its Q, K, V from pinned host memory, runs the kernel and reads O back to the host.  The three
    # stages run on three streams over two sets of device buffers, so step i+1's upload and step i-1's download
    # overlap step i's kernel (PCIe is full duplex); nothing is skipped or reused between steps.
    s_up, s_dn = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)
    sets = [(q, k, v, o), tuple(torch.empty_like(x) for x in (q, k, v, o))]
    hos = [ho, torch.empty(o.shape, dtype=o.dtype, pin_memory=True)]
    ev_up = [torch.cuda.Event() for _ in range(2)]     # inputs of the set are on the device
    ev_run = [torch.cuda.Event() for _ in range(2)]    # the kernel has consumed the set and written its O
    ev_dn = [torch.cuda.Event() for _ in range(2)]     # O of the set has been read back

    def e2e_pipeline(n):
        for i in range(n):
            b = i & 1
            qd, kd, vd, od = sets[b]
            with torch.cuda.stream(s_up):
                s_up.wait_event(ev_run[b])             # the kernel of step i-2 no longer reads this set
                qd.copy_(hq, non_blocking=True); kd.copy_(hk, non_blocking=True); vd.copy_(hv, non_blocking=True)
                ev_up[b].record(s_up)
            stream.wait_event(ev_up[b])
            stream.wait_event(ev_dn[b])                # O of step i-2 has left the device
            fmha_call(lib, wl, qd, kd, vd, od, scales, lse, stream=sptr)
            ev_run[b].record(stream)
            with torch.cuda.stream(s_dn):
                s_dn.wait_event(ev_run[b])
                hos[b].copy_(od, non_blocking=True)
                ev_dn[b].record(s_dn)
        stream.wait_stream(s_dn)
        stream.wait_stream(s_up)

    e2e_pipeline(2)
    barrier()
    e0.record(stream)
    e2e_pipeline(e2e_steps)
    e1.record(stream)
    barrier()
    t = torch.tensor([e0.elapsed_time(e1) / e2e_steps], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item())
    e2e_value = world * step_flops / (e2e_ms * 1e-3) / 1e12
    lib.check_device()

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- rank 0: parity spot-check, CPU baseline, secondary configs ----
    burst, sustained, peak_kind = measured_peaks()
    per_gpu = step_flops / (ms * 1e-3) / 1e12
    # DRAM bytes (read + write) of one kernel launch on this workload, from one ncu capture of the CLI driver
    # on the same shape (profiles/fmha_fwd_*.md name the command); the algorithmic bytes are Q+K+V+O.
    traffic = NCU_DRAM_BYTES_PER_LAUNCH.get(args.workload)
    # Tensor-core ceiling of this run's own clocks: the library's dense-UMMA probe on the workload's operand type
    # (one CTA per SM, operands resident in shared memory), a burst of a few ms and a sustained third of a second.
    # For e4m3 it is the roofline denominator (no library GEMM figure exists); for 16-bit types it is reported
    # beside the driver-measured cuBLAS figures.
    def umma_probe(groups, reps):
        lib.umma_peak(dt, 2000, stream=sptr)
        torch.cuda.synchronize()
        e0.record(stream)
        fl = 0.0
        for _ in range(reps):
            fl += lib.umma_peak(dt, groups, stream=sptr)
        e1.record(stream)
        torch.cuda.synchronize()
        return fl / (e0.elapsed_time(e1) * 1e-3) / 1e12
    umma_burst = umma_probe(20000, 1)
    umma_sustained = umma_probe(100000, 10 if dt != 2 else 20)
    lib.check_device()
    if dt == 2:
        burst, sustained, peak_kind = umma_burst, umma_sustained, "live cfk_umma_peak"
    line = {
        "metric": "fmha_fwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_max, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": DT_NAME[dt], "data": "synthetic",
        "config": {"workload": desc, "accumulate": "fp32", "algorithmic_bytes_per_launch": algo_bytes_of(wl), "flop_convention": "4*B*H*S*S*D, halved for causal",
                   "l2": "inputs (3 x %d MiB per GPU) exceed the 126 MB L2" % (q.numel() * q.element_size() >> 20),
                   "parallelism": "batch x head slices per GPU, no collective"},
        "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": burst, "unit": "TFLOP/s", "frac": per_gpu / burst,
                     "traffic": traffic,
                     "peak_source": f"{peak_kind} {'e4m3 UMMA' if dt == 2 else 'bf16 GEMM'} burst (timed region {ms * args.steps:.0f} ms)",
                     "umma_peak_live": {"dtype": DT_NAME[dt], "burst": umma_burst, "sustained": umma_sustained,
                                        "what": "dense tcgen05.mma 128x256 from shared memory, all SMs, this run"},
                     "peak_sustained": sustained, "frac_sustained": per_gpu / sustained,
                     "nominal": NOMINAL[dt], "frac_nominal": per_gpu / NOMINAL[dt]},
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms, "steps": e2e_steps,
                "how": "pinned host buffers; upload, kernel and download of consecutive steps overlap on three streams"},
        "gpu_launches": args.steps,
        "clocks": clocks,
    }

    if not args.no_extras:
        from oracle.oracle import CfkOracle
        orc = CfkOracle()
        # parity of the timed output: two (batch, head) slices against the CPU oracle
        fmha_call(lib, wl, q, k, v, o, scales, lse, stream=sptr)
        torch.cuda.synchronize()
        worst = {"max_abs": 0.0, "rel_rms": 0.0, "mismatch_pct": 0.0}
        sl = slices_for_cpu(torch, wl, q, k, v, scales, 2)
        for i, (qf, kf, vf) in enumerate(sl):
            b, h = (i // H) % B, i % H
            ref = orc.attention(qf, kf, vf, 1.0 / math.sqrt(D), causal)
            cmp = orc.compare(o[b:b + 1, :, h:h + 1, :].float().cpu().numpy(), ref["o"])
            for kx in worst:
                worst[kx] = max(worst[kx], cmp[kx])
        worst["slices_checked"] = len(sl)
        line["parity"] = worst
        # CPU baseline: the oracle on whole slices of the same workload, ~15 s
        n_try = B * H
        cpu_sl = slices_for_cpu(torch, wl, q, k, v, scales, n_try)
        done, t_cpu, cpu_tf = cpu_attention_sample(orc, torch, wl, cpu_sl, budget_s=12.0)
        line["cpu_baseline"] = {"value": cpu_tf, "unit": "TFLOP/s", "cores": orc.threads, "kind": "port",
                                "sample": f"{done} of {B * H} (batch, head) slices, full S={S}, D={D}, "
                                          f"causal={causal}, {t_cpu:.1f} s"}
        del cpu_sl, sl
        # secondary configs (device-resident, same timing recipe, fewer steps)
        others = {}
        del q, k, v, o, lse, hq, hk, hv, ho, sets, hos
        torch.cuda.empty_cache()
        for name in sorted(WORKLOADS):
            if name == args.workload:
                continue
            w2 = WORKLOADS[name]
            (q2, k2, v2), sc2 = make_inputs(torch, lib, w2, seed=77, device=device)
            o2 = torch.empty(w2[1], w2[3], w2[2], w2[4], dtype=torch.float16, device=device)
            for _ in range(3):
                fmha_call(lib, w2, q2, k2, v2, o2, sc2, stream=sptr)
            torch.cuda.synchronize()
            e0.record(stream)
            for _ in range(10):
                fmha_call(lib, w2, q2, k2, v2, o2, sc2, stream=sptr)
            e1.record(stream)
            torch.cuda.synchronize()
            ms2 = e0.elapsed_time(e1) / 10
            tf = flops_of(w2[1], w2[2], w2[3], w2[4], w2[5]) / (ms2 * 1e-3) / 1e12
            others[name] = {"workload": w2[6], "ms": ms2, "tflops": tf, "frac_nominal": tf / NOMINAL[w2[0]],
                            "frac_measured_bf16_burst": tf / measured_peaks()[0],
                            "note": "10 back-to-back launches after 3 warm-up launches (burst-like)"}
            del q2, k2, v2, o2
            torch.cuda.empty_cache()
        n = 8192
        a = torch.empty(n, n, dtype=torch.float16, device=device)
        b = torch.empty(n, n, dtype=torch.float16, device=device)
        c = torch.empty(n, n, dtype=torch.float16, device=device)
        lib.fill(a, cfk_b200.FP16, n * n, 1, "uniform")
        lib.fill(b, cfk_b200.FP16, n * n, 2, "uniform")
        lib.gemm(a, b, c, dtype=cfk_b200.FP16, m=n, n=n, k=n, iterations=3, stream=sptr)
        torch.cuda.synchronize()
        e0.record(stream)
        lib.gemm(a, b, c, dtype=cfk_b200.FP16, m=n, n=n, k=n, iterations=10, stream=sptr)
        e1.record(stream)
        torch.cuda.synchronize()
        msg = e0.elapsed_time(e1) / 10
        tf = 2.0 * n ** 3 / (msg * 1e-3) / 1e12
        # burst figure, the way the measured cuBLAS burst peak is taken: best of ten single launches after an idle gap
        time.sleep(0.3)
        best = float("inf")
        for _ in range(10):
            e0.record(stream)
            lib.gemm(a, b, c, dtype=cfk_b200.FP16, m=n, n=n, k=n, iterations=1, stream=sptr)
            e1.record(stream)
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        tf_burst = 2.0 * n ** 3 / (best * 1e-3) / 1e12
        cublas_burst, cublas_sustained, _ = measured_peaks()
        others["c2"] = {"workload": "gemm fp16 M=N=K=8192, fp32 accumulate, column-major C", "ms": msg, "tflops": tf,
                        "tflops_burst": tf_burst, "frac_nominal": tf / 2250.0,
                        "frac_measured_bf16_burst": tf_burst / cublas_burst,
                        "frac_measured_bf16_sustained": tf / cublas_sustained,
                        "note": "burst = best of 10 single launches after an idle gap, against the cuBLAS burst peak; "
                                "tflops = 10 back-to-back launches, against the cuBLAS sustained peak"}
        lib.check_device()
        line["other_configs"] = others

    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

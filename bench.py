#!/usr/bin/env python
"""Headline benchmark: FMHA forward TFLOP/s on B200 (and the CPU reference arm).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c4|c3|c5]

One "step" is one pass of the hot path over one batch of synthetic input: the cfk_fmha_forward calls
(one kernel launch each) that cover the workload's tensors.  The default workload is the S=8192, D=128
causal bf16 forward of the baseline (B=2, H=32): ONE problem of that size, whose 64 (batch, head) slices
are sharded over the N ranks (strong scaling; no data-path collective).  Each rank addresses its slices of
the unsharded tensors through the strided C ABI; the value is the FLOPs of the whole problem over the
slowest rank's device time.  The figure with a whole problem per rank is reported beside it
(other_configs.weak).  FLOP convention: 4*B*H*Sq*Skv*D, halved
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
    "c4": (1, 2, 32, 8192, 128, True, "fmha_fwd bf16 causal B=2 H=32 S=8192 D=128, out fp16"),
    "c3": (0, 4, 16, 4096, 128, False, "fmha_fwd fp16 B=4 H=16 S=4096 D=128, out fp16 + lse"),
    "c5": (2, 4, 16, 8192, 128, False, "fmha_fwd e4m3 B=4 H=16 S=8192 D=128, per-tensor scales, out fp16"),
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
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": desc, "accumulate": "fp32", "algorithmic_bytes_per_launch": algo_bytes_of(wl), "flop_convention": "4*B*H*S*S*D, halved for causal", "sample": sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": orc.threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "CPU restatement of the reference's unfused fp32 attention (include/utils/fmha_cutlass.hpp:154-317); "
                "the reference's own kernels are sm_90a-only and its checker needs CUTLASS, so neither runs here",
    }
    print(json.dumps(line), flush=True)


class Cudart:
    """cudaMemcpy2DAsync from the CUDA runtime torch has already loaded: a head-range shard of a [B][S][H][D] tensor
    is a pitched region (rows of head_count*D elements, pitch H*D), which one 2-D copy moves between a packed pinned
    host buffer and the unsharded device tensor."""
    H2D, D2H = 1, 2

    def __init__(self):
        import ctypes as C
        self.C = C
        self.rt = C.CDLL("libcudart.so.12")
        self.rt.cudaMemcpy2DAsync.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t,
                                              C.c_int, C.c_void_p]

    def copy2d(self, dst, dpitch, src, spitch, width, height, kind, stream):
        rc = self.rt.cudaMemcpy2DAsync(dst, dpitch, src, spitch, width, height, kind, stream)
        if rc:
            raise RuntimeError(f"cudaMemcpy2DAsync failed with {rc}")


def shard_plan(B, H, world, rank):
    from cfk_b200.sharding import sub_calls
    return sub_calls(B, H, world, rank)


def run_plan(lib, wl, plan, q, k, v, o, scales, lse=None, stream=None):
    """One step: the rank's (batch, head) slices of the unsharded tensors, one cfk_fmha_forward call per rectangular
    sub-call, addressed through a pointer offset and the unsharded strides (the reference slices a batch range the
    same way, src/fmha-pipeline/fmha_forward.cu:401-417).  Returns the number of kernel launches."""
    from cfk_b200.sharding import element_offset, strides
    dt, B, H, S, D, causal, _ = wl
    st = strides(S, H, D)
    esz = q.element_size()
    for c in plan:
        off = element_offset(c, S, H, D)
        # [B][H][S] statistics: a sub-call is whole batches, or a head range of one batch, so its own
        # [batch_count][head_count][S] block starts at (batch_begin, head_begin) of the unsharded tensor
        lse_ptr = None if lse is None else lse.data_ptr() + 4 * ((c.batch_begin * H + c.head_begin) * S)
        lib.fmha_forward(q.data_ptr() + off * esz, k.data_ptr() + off * esz, v.data_ptr() + off * esz,
                         o.data_ptr() + off * 2, dtype=dt, batch=c.batch_count, heads=c.head_count, seqlen_q=S,
                         seqlen_kv=S, head_dim=D, softmax_scale=1.0 / math.sqrt(D), causal=causal,
                         lse=lse_ptr,
                         q_descale=scales[0], k_descale=scales[1], v_descale=scales[2],
                         q_stride=st, k_stride=st, v_stride=st, o_stride=st, stream=stream)
    return len(plan)


def timed_steps(torch, stream, steps, fn):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(steps):
        fn(i)
    e1.record(stream)
    return e0, e1


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c4", choices=sorted(WORKLOADS))
    ap.add_argument("--no-extras", action="store_true", help="skip the secondary configs and the CPU baseline")
    ap.add_argument("--sustained-seconds", type=float, default=2.0)
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
    desc = desc.replace(" (per GPU)", "")
    plan = shard_plan(B, H, world, rank)
    my_slices = sum(c.batch_count * c.head_count for c in plan)
    slice_bytes = S * D * q_esz(dt)
    # Input sets: the unsharded tensors, identical on every rank (the fill is keyed by the logical index, so a shard
    # is bit-identical to the same slices of a single-GPU run); a rank touches only its slices.  When those are
    # smaller than L2, the steps rotate over several sets so that no step finds its inputs in L2.
    touched = my_slices * (3 * slice_bytes + S * D * 2)
    n_sets = max(1, min(8, -(-(256 << 20) // touched)))
    sets = []
    scales = None
    for i in range(n_sets):
        (q, k, v), scales = make_inputs(torch, lib, wl, seed=3080, device=device)
        o = torch.full((B, S, H, D), -1.0, dtype=torch.float16, device=device)
        sets.append((q, k, v, o))
    lse = torch.empty(B, H, S, dtype=torch.float32, device=device)
    stream = torch.cuda.current_stream()
    sptr = stream.cuda_stream
    total_flops = flops_of(B, H, S, D, causal)              # the whole problem, whatever the number of ranks
    my_flops = total_flops * my_slices / (B * H)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        t = torch.tensor([x], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def step(i):
        qd, kd, vd, od = sets[i % n_sets]
        return run_plan(lib, wl, plan, qd, kd, vd, od, scales, lse, stream=sptr)

    # ---- device-resident timing (value): the fixed problem, each rank its slices ----
    for i in range(args.warmup):
        step(i)
    lib.check_device()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        sampler.wait_first()
    barrier()
    t_begin = time.monotonic()
    e0, e1 = timed_steps(torch, stream, args.steps, step)
    barrier()
    t_end = time.monotonic()
    ms = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None
    lib.check_device()
    ms_max = max_over_ranks(ms)
    value = total_flops / (ms_max * 1e-3) / 1e12

    # ---- sustained: the same steps back to back for a couple of seconds, with the clocks of that region ----
    sustained = None
    if args.sustained_seconds > 0:
        n_sus = max(args.steps, int(args.sustained_seconds * 1e3 / max(ms_max, 1e-3)))
        n_sus = int(max_over_ranks(n_sus))
        sampler2 = ClockSampler(local_rank)
        if rank == 0:
            sampler2.start()
            sampler2.wait_first()
        barrier()
        t0 = time.monotonic()
        s0, s1 = timed_steps(torch, stream, n_sus, step)
        barrier()
        t1 = time.monotonic()
        sus_ms = max_over_ranks(s0.elapsed_time(s1) / n_sus)
        lib.check_device()
        if rank == 0:
            # the first 0.3 s are the clock settling under the power cap: the median is taken after them
            c2 = sampler2.stop(t0 + min(0.3, 0.25 * (t1 - t0)), t1)
            sus_tf = total_flops / (sus_ms * 1e-3) / 1e12
            sustained = {"steps": n_sus, "seconds": sus_ms * n_sus * 1e-3, "ms_per_step": sus_ms, "value": sus_tf,
                         "unit": "TFLOP/s", "clocks": c2}
            if c2.get("sm_mhz"):
                # time x clock: what the same run would show at another clock (the work per step in SM cycles)
                sustained["mcycles_per_step"] = sus_ms * 1e-3 * c2["sm_mhz"]
                sustained["value_at_max_clock"] = sus_tf * c2["sm_max_mhz"] / c2["sm_mhz"]

    # ---- end-to-end through the C ABI with host buffers (e2e): only this rank's slices travel ----
    rt = Cudart()
    esz = q_esz(dt)
    q0, k0, v0, o0 = sets[0]
    host_in = []     # per sub-call: packed pinned [batch_count][S][head_count][D] copies of Q, K, V
    host_out = [[], []]
    for c in plan:
        shp = (c.batch_count, S, c.head_count, D)
        bufs = []
        for x in (q0, k0, v0):
            h = torch.empty(shp, dtype=x.dtype, pin_memory=True)
            h.copy_(x[c.batch_begin:c.batch_begin + c.batch_count, :, c.head_begin:c.head_begin + c.head_count, :])
            bufs.append(h)
        host_in.append(bufs)
        for b in range(2):
            host_out[b].append(torch.empty(shp, dtype=torch.float16, pin_memory=True))
    h2d = sum(h.numel() * h.element_size() for bufs in host_in for h in bufs)
    d2h = sum(h.numel() * h.element_size() for h in host_out[0])
    e2e_steps = max(4, min(args.steps, 16))
    from cfk_b200.sharding import element_offset

    def copy_shard(c, dev, host, kind, st, el):
        """Packed host buffer <-> the sub-call's pitched region of the unsharded device tensor."""
        off = element_offset(c, S, H, D) * el
        width = c.head_count * D * el
        pitch = H * D * el
        if kind == Cudart.H2D:
            rt.copy2d(dev.data_ptr() + off, pitch, host.data_ptr(), width, width, c.batch_count * S, kind, st)
        else:
            rt.copy2d(host.data_ptr(), width, dev.data_ptr() + off, pitch, width, c.batch_count * S, kind, st)

    # Every step copies its Q, K, V slices from pinned host memory, runs the kernel and reads its O slices back to the
    # host.  The three stages run on three streams over two sets of device buffers, so step i+1's upload and step
    # i-1's download overlap step i's kernel (PCIe is full duplex); nothing is skipped or reused between steps.
    s_up, s_dn = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)
    if len(sets) < 2:
        sets.append(tuple(torch.empty_like(x) for x in sets[0]))
    ev_up = [torch.cuda.Event() for _ in range(2)]     # inputs of the set are on the device
    ev_run = [torch.cuda.Event() for _ in range(2)]    # the kernel has consumed the set and written its O
    ev_dn = [torch.cuda.Event() for _ in range(2)]     # O of the set has been read back

    def e2e_pipeline(n):
        for i in range(n):
            b = i & 1
            qd, kd, vd, od = sets[b]
            s_up.wait_event(ev_run[b])                 # the kernel of step i-2 no longer reads this set
            for c, bufs in zip(plan, host_in):
                for dev, host in zip((qd, kd, vd), bufs):
                    copy_shard(c, dev, host, Cudart.H2D, s_up.cuda_stream, esz)
            ev_up[b].record(s_up)
            stream.wait_event(ev_up[b])
            stream.wait_event(ev_dn[b])                # O of step i-2 has left the device
            run_plan(lib, wl, plan, qd, kd, vd, od, scales, None, stream=sptr)
            ev_run[b].record(stream)
            s_dn.wait_event(ev_run[b])
            for c, host in zip(plan, host_out[b]):
                copy_shard(c, od, host, Cudart.D2H, s_dn.cuda_stream, 2)
            ev_dn[b].record(s_dn)
        stream.wait_stream(s_dn)
        stream.wait_stream(s_up)

    e2e_pipeline(2)
    barrier()
    x0, x1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    x0.record(stream)
    e2e_pipeline(e2e_steps)
    x1.record(stream)
    barrier()
    e2e_ms = max_over_ranks(x0.elapsed_time(x1) / e2e_steps)
    e2e_value = total_flops / (e2e_ms * 1e-3) / 1e12
    lib.check_device()
    # the slices that came back are the ones the device-resident run wrote
    torch.cuda.synchronize()
    c0 = plan[0]
    e2e_equal = bool(torch.equal(host_out[(e2e_steps - 1) & 1][0],
                                 sets[(e2e_steps - 1) & 1][3][c0.batch_begin:c0.batch_begin + c0.batch_count, :,
                                                              c0.head_begin:c0.head_begin + c0.head_count, :].cpu()))

    # ---- weak scaling beside it (N > 1): every rank a whole problem of the same size ----
    weak = None
    if world > 1:
        whole = shard_plan(B, H, 1, 0)
        for i in range(3):
            run_plan(lib, wl, whole, *sets[0], scales, lse, stream=sptr)
        barrier()
        w0, w1 = timed_steps(torch, stream, 20, lambda i: run_plan(lib, wl, whole, *sets[i & 1], scales, lse, stream=sptr))
        barrier()
        weak_ms = max_over_ranks(w0.elapsed_time(w1) / 20)
        weak = {"workload": desc + ", one whole problem per GPU", "ms_per_step": weak_ms, "steps": 20,
                "tflops": world * total_flops / (weak_ms * 1e-3) / 1e12}
        lib.check_device()

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- rank 0: the JSON line; parity spot-check, CPU baseline and secondary configs (N = 1) ----
    burst, sustained_peak, peak_kind = measured_peaks()
    per_gpu = my_flops / (ms * 1e-3) / 1e12            # this GPU's own rate on its own slices
    e_a, e_b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def umma_probe(pdt, groups, reps):
        """The library's dense-UMMA probe on an operand type (one CTA per SM, operands resident in shared memory):
        the tensor-core ceiling at this run's own clocks."""
        lib.umma_peak(pdt, 2000, stream=sptr)
        torch.cuda.synchronize()
        e_a.record(stream)
        fl = 0.0
        for _ in range(reps):
            fl += lib.umma_peak(pdt, groups, stream=sptr)
        e_b.record(stream)
        torch.cuda.synchronize()
        return fl / (e_a.elapsed_time(e_b) * 1e-3) / 1e12

    probes = {}
    for pdt in sorted({dt, 1, 2}) if not args.no_extras else [dt]:
        probes[DT_NAME[pdt]] = {"burst": umma_probe(pdt, 20000, 1),
                                "sustained": umma_probe(pdt, 100000, 10 if pdt != 2 else 20)}
    lib.check_device()
    if dt == 2:
        burst, sustained_peak, peak_kind = probes["e4m3"]["burst"], probes["e4m3"]["sustained"], "live cfk_umma_peak"
    region_ms = ms * args.steps
    line = {
        "metric": "fmha_fwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_max, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": DT_NAME[dt], "data": "synthetic",
        "config": {"workload": desc, "accumulate": "fp32", "algorithmic_bytes_per_launch": algo_bytes_of(wl),
                   "flop_convention": "4*B*H*S*S*D, halved for causal",
                   "l2": ("inputs touched per step (%d MiB on this GPU) %s" %
                          (touched >> 20, "exceed the 126 MB L2" if n_sets == 1 else
                           "are smaller than the 126 MB L2: steps rotate over %d input sets (%d MiB)" % (n_sets, (n_sets * touched) >> 20))),
                   "parallelism": "the problem's %d (batch, head) slices sharded over %d GPU(s), %d per GPU, no collective"
                                  % (B * H, world, my_slices),
                   "sub_calls_per_step": len(plan)},
        "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": burst, "unit": "TFLOP/s", "frac": per_gpu / burst,
                     "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get(args.workload) if world == 1 else None,
                     "traffic_source": "one ncu capture of the same shape, not of this run: "
                                       "profiles/fmha_fwd_kernel_c3_c4_c5.md" if world == 1 else None,
                     "peak_source": f"{peak_kind} {'e4m3 UMMA' if dt == 2 else 'bf16 GEMM'} burst "
                                    f"(timed region {region_ms:.0f} ms)",
                     "umma_peak_live": {"what": "dense tcgen05.mma 128x256 from shared memory, all SMs, this run", **probes},
                     "nominal": NOMINAL[dt], "frac_nominal": per_gpu / NOMINAL[dt]},
        "sustained": sustained,
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms, "steps": e2e_steps, "output_equals_device_run": e2e_equal,
                "how": "this rank's slices only: packed pinned host buffers <-> the pitched region of the device tensor "
                       "(cudaMemcpy2DAsync); upload, kernel and download of consecutive steps overlap on three streams"},
        "gpu_launches": args.steps * len(plan),
        "clocks": clocks,
    }
    if sustained:
        sustained["frac_of_sustained_peak"] = (sustained["value"] / world) / sustained_peak
        sustained["peak_sustained"] = sustained_peak
    if weak:
        line["other_configs"] = {"weak": weak}

    if not args.no_extras and world == 1:
        from oracle.oracle import CfkOracle
        orc = CfkOracle()
        q, k, v, o = sets[0]
        # parity of the timed output: four (batch, head) slices against the CPU oracle, the corners among them
        run_plan(lib, wl, plan, q, k, v, o, scales, lse, stream=sptr)
        torch.cuda.synchronize()
        picks = sorted({(0, 0), (B - 1, H - 1), (0, H // 2), (B - 1, H // 3)})
        worst = {"max_abs": 0.0, "rel_rms": 0.0, "mismatch_pct": 0.0, "lse_max_abs": 0.0}
        where = None
        for (b, h) in picks:
            qf, kf, vf = ((x[b:b + 1, :, h:h + 1, :].float() * s).cpu().numpy() for x, s in zip((q, k, v), scales))
            ref = orc.attention(qf, kf, vf, 1.0 / math.sqrt(D), causal)
            got = o[b:b + 1, :, h:h + 1, :].float().cpu().numpy()
            cmp = orc.compare(got, ref["o"])
            if cmp["max_abs"] >= worst["max_abs"]:
                row, col = divmod(int(cmp["argmax"]), D)
                where = {"batch": b, "head": h, "row": row, "col": col}
            for kx in ("max_abs", "rel_rms", "mismatch_pct"):
                worst[kx] = max(worst[kx], cmp[kx])
            worst["lse_max_abs"] = max(worst["lse_max_abs"],
                                       float(abs(lse[b, h].cpu().numpy() - ref["lse"][0, 0]).max()))
        worst["slices_checked"] = [list(x) for x in picks]
        worst["worst_element"] = where
        worst["tolerance"] = "rel_rms <= 3e-2" if dt == 2 else "max_abs <= 2e-3"
        line["parity"] = worst
        # CPU baseline: the oracle on whole slices of the same workload, ~12 s
        cpu_sl = slices_for_cpu(torch, wl, q, k, v, scales, B * H)
        done, t_cpu, cpu_tf = cpu_attention_sample(orc, torch, wl, cpu_sl, budget_s=12.0)
        line["cpu_baseline"] = {"value": cpu_tf, "unit": "TFLOP/s", "cores": orc.threads, "kind": "port",
                                "sample": f"{done} of {B * H} (batch, head) slices, full S={S}, D={D}, "
                                          f"causal={causal}, {t_cpu:.1f} s"}
        del cpu_sl
        # secondary configs (device-resident, same timing recipe, fewer steps): bursts of ten launches, each against
        # the burst ceiling of its own operand type
        others = {}
        del q, k, v, o, lse, host_in, host_out, sets
        torch.cuda.empty_cache()
        extra = {name: WORKLOADS[name] + (False,) for name in sorted(WORKLOADS) if name != args.workload}
        extra["c5_hybrid"] = WORKLOADS["c5"][:6] + ("fmha_fwd e4m3 Q, K with fp16 V and P (the reference's FP8 mode "
                                                    "without GEMM2FP8), B=4 H=16 S=8192 D=128", True)
        for name, w2 in extra.items():
            hybrid = w2[7]
            (q2, k2, v2), sc2 = make_inputs(torch, lib, w2[:7], seed=77, device=device)
            if hybrid:
                v16 = torch.empty(v2.shape, dtype=torch.float16, device=device)
                lib.convert(v2, cfk_b200.E4M3, v16, cfk_b200.FP16, v2.numel(), sc2[2])
                v2, sc2 = v16, [sc2[0], sc2[1], 1.0]
            o2 = torch.empty(w2[1], w2[3], w2[2], w2[4], dtype=torch.float16, device=device)

            def call(n):
                lib.fmha_forward(q2, k2, v2, o2, dtype=w2[0], batch=w2[1], heads=w2[2], seqlen_q=w2[3],
                                 seqlen_kv=w2[3], head_dim=w2[4], softmax_scale=1.0 / math.sqrt(w2[4]), causal=w2[5],
                                 q_descale=sc2[0], k_descale=sc2[1], v_descale=sc2[2], iterations=n, v_fp16=hybrid,
                                 stream=sptr)
            call(3)
            torch.cuda.synchronize()
            e_a.record(stream)
            call(10)
            e_b.record(stream)
            torch.cuda.synchronize()
            ms2 = e_a.elapsed_time(e_b) / 10
            tf = flops_of(w2[1], w2[2], w2[3], w2[4], w2[5]) / (ms2 * 1e-3) / 1e12
            # the slower GEMM of the hybrid mode runs at the 16-bit rate: its ceiling is quoted against e4m3 all the same
            ceiling = probes["e4m3"]["burst"] if w2[0] == 2 else measured_peaks()[0]
            others[name] = {"workload": w2[6], "ms": ms2, "tflops": tf, "frac_nominal": tf / NOMINAL[w2[0]],
                            "frac": tf / ceiling,
                            "peak": ceiling,
                            "peak_source": ("live cfk_umma_peak e4m3 burst" if w2[0] == 2 else "measured bf16 GEMM burst"),
                            "note": "10 back-to-back launches after 3 warm-up launches (burst over burst)"}
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
        # burst figure, the way the measured cuBLAS burst peak is taken: best of ten single launches after an idle gap
        time.sleep(0.3)
        best = float("inf")
        for _ in range(10):
            e_a.record(stream)
            lib.gemm(a, b, c, dtype=cfk_b200.FP16, m=n, n=n, k=n, iterations=1, stream=sptr)
            e_b.record(stream)
            torch.cuda.synchronize()
            best = min(best, e_a.elapsed_time(e_b))
        tf_burst = 2.0 * n ** 3 / (best * 1e-3) / 1e12
        # sustained figure, the way the measured cuBLAS sustained peak is taken: back to back for two seconds
        reps = max(10, int(2000.0 / best))
        e_a.record(stream)
        lib.gemm(a, b, c, dtype=cfk_b200.FP16, m=n, n=n, k=n, iterations=reps, stream=sptr)
        e_b.record(stream)
        torch.cuda.synchronize()
        tf_sus = 2.0 * n ** 3 * reps / (e_a.elapsed_time(e_b) * 1e-3) / 1e12
        cublas_burst, cublas_sustained, _ = measured_peaks()
        others["c2"] = {"workload": "gemm fp16 M=N=K=8192, fp32 accumulate, column-major C",
                        "tflops_burst": tf_burst, "frac_burst": tf_burst / cublas_burst,
                        "tflops_sustained": tf_sus, "frac_sustained": tf_sus / cublas_sustained,
                        "sustained_seconds": e_a.elapsed_time(e_b) * 1e-3, "frac_nominal": tf_burst / 2250.0,
                        "note": "burst = best of 10 single launches after an idle gap, against the cuBLAS burst peak; "
                                "sustained = launches back to back for 2 s, against the cuBLAS sustained peak"}
        lib.check_device()
        line["other_configs"] = others

    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def q_esz(dt):
    return 1 if dt == 2 else 2


if __name__ == "__main__":
    main()

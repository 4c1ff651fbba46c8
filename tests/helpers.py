"""Input builders shared by the CPU and GPU tests (torch is used as a tensor container only)."""
import math

import numpy as np
import torch

TORCH_DT = {0: torch.float16, 1: torch.bfloat16, 2: torch.float8_e4m3fn}


def make_qkv(dtype, B, Sq, Skv, H, D, seed):
    """Seeded N(0,1) Q/K/V.  Returns (low-precision tensors, their exact float32 values, de-scales)."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Sq, H, D, generator=g)
    k = torch.randn(B, Skv, H, D, generator=g)
    v = torch.randn(B, Skv, H, D, generator=g)
    if dtype == 2:   # e4m3 with a per-tensor scale amax/448
        scales = [float(x.abs().max()) / 448.0 for x in (q, k, v)]
        low = [(x / s).to(torch.float8_e4m3fn) for x, s in zip((q, k, v), scales)]
        f32 = [l.float() * s for l, s in zip(low, scales)]
    else:
        scales = [1.0, 1.0, 1.0]
        low = [x.to(TORCH_DT[dtype]) for x in (q, k, v)]
        f32 = [l.float() for l in low]
    return low, [x.numpy() for x in f32], scales


def run_fmha(lib, low, scales, dtype, causal, out_dtype=0, p_split_keys=-1, want_stats=True, scale=None):
    """Uploads, calls cfk_fmha_forward through the C ABI, returns (O float32 numpy, stats dict)."""
    q, k, v = (x.cuda() for x in low)
    B, Sq, H, D = q.shape
    Skv = k.shape[1]
    o = torch.full((B, Sq, H, D), -1.0, device="cuda", dtype=torch.float16 if out_dtype == 0 else torch.bfloat16)
    stats = {}
    if want_stats:
        for name in ("lse", "mi", "sprime"):
            stats[name] = torch.full((B, H, Sq), -1.0, device="cuda", dtype=torch.float32)
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    lib.fmha_forward(q, k, v, o, dtype=dtype, batch=B, heads=H, seqlen_q=Sq, seqlen_kv=Skv, head_dim=D,
                     softmax_scale=scale, causal=causal, out_dtype=out_dtype, p_split_keys=p_split_keys,
                     q_descale=scales[0], k_descale=scales[1], v_descale=scales[2],
                     lse=stats.get("lse"), mi=stats.get("mi"), sprime=stats.get("sprime"))
    lib.check_device()
    return o.float().cpu().numpy(), {k2: v2.cpu().numpy() for k2, v2 in stats.items()}

"""Regenerates the committed fixtures from the numpy float64 restatement (oracle/oracle.py).

The reference project stores no golden vectors and cannot be built or imported here, so these are
outputs of the independent float64 restatement on seeded inputs rounded to fp16-representable
values (the reference's checker also runs on up-cast low-precision inputs,
src/fmha-pipeline/fmha_forward.cu:613-621).  Run from the repository root:
    python tests/golden/make_golden.py
"""
import math
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle.oracle import attention_f64, gemm_f64  # noqa: E402


def rounded(rng, shape):
    return rng.standard_normal(shape).astype(np.float16).astype(np.float32)


def main():
    rng = np.random.default_rng(3080)
    out = {}
    cases = {"c1": (1, 128, 128, 2, 64, False), "causal": (1, 128, 128, 1, 32, True), "ragged": (1, 77, 133, 1, 32, False)}
    for tag, (B, Sq, Skv, H, D, causal) in cases.items():
        q, k, v = rounded(rng, (B, Sq, H, D)), rounded(rng, (B, Skv, H, D)), rounded(rng, (B, Skv, H, D))
        scale = 1.0 / math.sqrt(D)
        r = attention_f64(q, k, v, scale, causal)
        out.update({f"{tag}_q": q.astype(np.float16), f"{tag}_k": k.astype(np.float16), f"{tag}_v": v.astype(np.float16), f"{tag}_scale": np.float32(scale),
                    f"{tag}_causal": np.int32(causal), f"{tag}_o": r["o"].astype(np.float32),
                    f"{tag}_lse": r["lse"].astype(np.float32)})
    # two more cases at a head dimension the CUDA kernels are built for, drawn from a generator of their own so that
    # the arrays above keep their values
    rng64 = np.random.default_rng(3081)
    more = {"causal64": (1, 128, 128, 1, 64, True), "ragged64": (2, 77, 133, 2, 64, False)}
    for tag, (B, Sq, Skv, H, D, causal) in more.items():
        q, k, v = rounded(rng64, (B, Sq, H, D)), rounded(rng64, (B, Skv, H, D)), rounded(rng64, (B, Skv, H, D))
        scale = 1.0 / math.sqrt(D)
        r = attention_f64(q, k, v, scale, causal)
        out.update({f"{tag}_q": q.astype(np.float16), f"{tag}_k": k.astype(np.float16), f"{tag}_v": v.astype(np.float16), f"{tag}_scale": np.float32(scale),
                    f"{tag}_causal": np.int32(causal), f"{tag}_o": r["o"].astype(np.float32),
                    f"{tag}_lse": r["lse"].astype(np.float32)})
    np.savez_compressed(os.path.join(HERE, "attention_small.npz"), **out)
    # head dimension 128 (the benchmark's), in a file of its own so that the file above keeps its bytes: a causal case
    # whose two query tiles see different numbers of key tiles, and a causal case with an offset diagonal, a ragged
    # last tile and a query block with one tile only
    rng128 = np.random.default_rng(3082)
    d128 = {}
    for tag, (B, Sq, Skv, H, D, causal) in {"causal128": (1, 256, 256, 1, 128, True), "offset128": (1, 130, 333, 1, 128, True)}.items():
        q, k, v = rounded(rng128, (B, Sq, H, D)), rounded(rng128, (B, Skv, H, D)), rounded(rng128, (B, Skv, H, D))
        scale = 1.0 / math.sqrt(D)
        r = attention_f64(q, k, v, scale, causal)
        d128.update({f"{tag}_q": q.astype(np.float16), f"{tag}_k": k.astype(np.float16), f"{tag}_v": v.astype(np.float16),
                     f"{tag}_scale": np.float32(scale), f"{tag}_causal": np.int32(causal), f"{tag}_o": r["o"].astype(np.float32),
                     f"{tag}_lse": r["lse"].astype(np.float32)})
    np.savez_compressed(os.path.join(HERE, "attention_d128.npz"), **d128)
    a = rng.uniform(-1, 1, (48, 80)).astype(np.float16).astype(np.float32)
    b = rng.uniform(-1, 1, (40, 80)).astype(np.float16).astype(np.float32)
    c_in = rng.uniform(-1, 1, (48, 40)).astype(np.float16).astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "gemm_small.npz"), a=a, b=b, c_in=c_in, alpha=np.float32(1.5),
                        beta=np.float32(-0.5), c=gemm_f64(a, b, 1.5, -0.5, c_in).astype(np.float32))


if __name__ == "__main__":
    main()

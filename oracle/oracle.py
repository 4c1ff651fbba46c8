"""Python face of the CPU oracle (test infrastructure, never the product path).

`CfkOracle` binds `libcfk_oracle.so` (built from `cfk_oracle.c` by the Makefile beside it);
`attention_f64` / `gemm_f64` are a second, independent numpy float64 restatement of the same
arithmetic used to pin the C code and to generate the committed fixtures.

PARITY UNPINNED with respect to the reference: it holds no golden vectors and its own checker
cannot be built without CUTLASS (see the header of cfk_oracle.c for the cited lines).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "libcfk_oracle.so")

DTYPE_CODES = {"fp16": 0, "bf16": 1, "e4m3": 2, "fp32": 3}


def build(force: bool = False) -> str:
    """Compile the C oracle if it is missing or older than its source."""
    src = os.path.join(_HERE, "cfk_oracle.c")
    if force or not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libcfk_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB


def _fp(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


class CfkOracle:
    def __init__(self):
        self.lib = C.CDLL(build())
        L = self.lib
        L.cfk_oracle_threads.restype = C.c_int
        L.cfk_oracle_attention.argtypes = [C.POINTER(C.c_float)] * 7 + [C.c_int] * 5 + [C.c_float] + [C.c_int] * 5
        L.cfk_oracle_gemm.argtypes = [C.POINTER(C.c_float)] * 4 + [C.c_int] * 3 + [C.c_float, C.c_float] + [C.c_int] * 3
        L.cfk_compare.argtypes = [C.POINTER(C.c_float), C.POINTER(C.c_float), C.c_int64, C.POINTER(C.c_double)]
        L.cfk_convert_from_f32.argtypes = [C.POINTER(C.c_float), C.c_void_p, C.c_int64, C.c_int]
        L.cfk_convert_to_f32.argtypes = [C.c_void_p, C.POINTER(C.c_float), C.c_int64, C.c_int]
        L.cfk_fill_f32.argtypes = [C.POINTER(C.c_float), C.c_int64, C.c_uint64, C.c_int64, C.c_int]

    @property
    def threads(self) -> int:
        return int(self.lib.cfk_oracle_threads())

    def attention(self, q, k, v, scale, causal=False, b_range=None, h_range=None, want_stats=True):
        """q:[B,Sq,H,D], k,v:[B,Skv,H,D] float32 -> dict(o, lse, row_max, inv_sum)."""
        q = np.ascontiguousarray(q, np.float32)
        k = np.ascontiguousarray(k, np.float32)
        v = np.ascontiguousarray(v, np.float32)
        B, Sq, H, D = q.shape
        Skv = k.shape[1]
        o = np.zeros_like(q)
        lse = np.zeros((B, H, Sq), np.float32)
        mx = np.zeros((B, H, Sq), np.float32)
        inv = np.zeros((B, H, Sq), np.float32)
        b0, b1 = b_range or (0, B)
        h0, h1 = h_range or (0, H)
        self.lib.cfk_oracle_attention(_fp(q), _fp(k), _fp(v), _fp(o), _fp(lse), _fp(mx), _fp(inv),
                                      B, H, Sq, Skv, D, float(scale), int(bool(causal)), b0, b1, h0, h1)
        return {"o": o, "lse": lse, "row_max": mx, "inv_sum": inv}

    def gemm(self, a, b, alpha=1.0, beta=0.0, c_in=None, c_col_major=True, m_range=None):
        """a:[M,K], b:[N,K] float32.  Returns C as an [M,N] array (a view of the chosen storage)."""
        a = np.ascontiguousarray(a, np.float32)
        b = np.ascontiguousarray(b, np.float32)
        M, K = a.shape
        N = b.shape[0]
        store = np.zeros((N, M) if c_col_major else (M, N), np.float32)
        cin = None
        if c_in is not None:
            cin = np.ascontiguousarray(c_in.T if c_col_major else c_in, np.float32)
        m0, m1 = m_range or (0, M)
        self.lib.cfk_oracle_gemm(_fp(a), _fp(b), _fp(cin) if cin is not None else None, _fp(store),
                                 M, N, K, float(alpha), float(beta), int(bool(c_col_major)), m0, m1)
        return store.T if c_col_major else store

    def compare(self, got, ref):
        got = np.ascontiguousarray(got, np.float32).ravel()
        ref = np.ascontiguousarray(ref, np.float32).ravel()
        out = (C.c_double * 5)()
        self.lib.cfk_compare(_fp(got), _fp(ref), got.size, out)
        return {"max_abs": out[0], "argmax": int(out[1]), "rel_rms": out[2],
                "mismatch_pct": out[3], "nonfinite": int(out[4])}

    def quantize(self, x, dtype: str):
        """float32 -> raw storage (uint16 for fp16/bf16, uint8 for e4m3), round-to-nearest-even."""
        x = np.ascontiguousarray(x, np.float32)
        code = DTYPE_CODES[dtype]
        out = np.empty(x.shape, {0: np.uint16, 1: np.uint16, 2: np.uint8, 3: np.float32}[code])
        self.lib.cfk_convert_from_f32(_fp(x), out.ctypes.data, x.size, code)
        return out

    def dequantize(self, raw, dtype: str):
        raw = np.ascontiguousarray(raw)
        out = np.empty(raw.shape, np.float32)
        self.lib.cfk_convert_to_f32(raw.ctypes.data, _fp(out), raw.size, DTYPE_CODES[dtype])
        return out

    def fill(self, shape, seed: int, kind: str = "normal", first_index: int = 0):
        out = np.empty(shape, np.float32)
        self.lib.cfk_fill_f32(_fp(out), out.size, seed, first_index, 0 if kind == "normal" else 1)
        return out


# ---------------------------------------------------------------------------------------------
# Independent numpy float64 restatement (same steps: scaled scores, row max, exp, inverse sum,
# normalised P times V), after include/utils/fmha_cutlass.hpp:275-314 of the reference.
# ---------------------------------------------------------------------------------------------

def attention_f64(q, k, v, scale, causal=False):
    q = np.asarray(q, np.float64)
    k = np.asarray(k, np.float64)
    v = np.asarray(v, np.float64)
    B, Sq, H, D = q.shape
    Skv = k.shape[1]
    s = np.einsum("bihd,bjhd->bhij", q, k) * scale
    if causal:
        i = np.arange(Sq)[:, None]
        j = np.arange(Skv)[None, :]
        s = np.where(j <= i + (Skv - Sq), s, -np.inf)
    mx = s.max(axis=-1, keepdims=True)
    e = np.exp(s - mx)
    sm = e.sum(axis=-1, keepdims=True)
    p = e / sm
    o = np.einsum("bhij,bjhd->bihd", p, v)
    return {"o": o, "lse": (mx + np.log(sm))[..., 0], "row_max": mx[..., 0], "inv_sum": (1.0 / sm)[..., 0]}


def gemm_f64(a, b, alpha=1.0, beta=0.0, c_in=None):
    c = alpha * (np.asarray(a, np.float64) @ np.asarray(b, np.float64).T)
    if c_in is not None and beta != 0.0:
        c = c + beta * np.asarray(c_in, np.float64)
    return c

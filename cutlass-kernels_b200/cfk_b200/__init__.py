"""ctypes binding of libcfk_b200.so for the Python test-suite and bench.

The product is the C-ABI library (declared in include/cfk_b200.h) plus the C++ shim with the
reference's launcher names (include/cfk_compat.hpp).  This module only forwards to it: it takes raw
device pointers (ints) or objects with `.data_ptr()` (torch tensors, used purely as device-memory
holders), fills the argument structs and returns the library's status code.  There is no fallback of
any kind: if the shared library is missing, importing `load()` raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "libcfk_b200.so")

FP16, BF16, E4M3, FP32 = 0, 1, 2, 3
DTYPES = {"fp16": FP16, "bf16": BF16, "e4m3": E4M3, "fp32": FP32}

STATUS_NAMES = {0: "OK", 1: "INVALID_ARG", 2: "UNSUPPORTED", 3: "DESCRIPTOR", 4: "LAUNCH", 5: "NO_DRIVER",
                6: "DEVICE_WAIT", 7: "TOO_LARGE"}

EXPORTS = ["cfk_fmha_forward", "cfk_fmha_forward_static", "cfk_gemm", "cfk_fill", "cfk_convert", "cfk_device_status",
           "cfk_last_cuda_error", "cfk_version", "cfk_selftest_umma", "cfk_umma_peak", "cfk_selftest_wait_gives_up", "cfk_selftest_wait_gives_up_static", "cfk_set_tunable", "cfk_get_tunable"]

TUNE_FMHA_EXP_EMU, TUNE_FMHA_GROUP_MB, TUNE_FMHA_KERNEL, TUNE_FMHA_GRID, TUNE_FMHA_SCHED = 0, 1, 2, 3, 4


class FmhaArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int), ("out_dtype", C.c_int), ("p_split_keys", C.c_int),
        ("batch", C.c_int), ("heads", C.c_int), ("seqlen_q", C.c_int), ("seqlen_kv", C.c_int),
        ("head_dim", C.c_int),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p),
        ("lse", C.c_void_p), ("mi", C.c_void_p), ("sprime", C.c_void_p),
        ("q_stride", C.c_int64 * 3), ("k_stride", C.c_int64 * 3), ("v_stride", C.c_int64 * 3),
        ("o_stride", C.c_int64 * 3),
        ("softmax_scale", C.c_float), ("causal", C.c_int),
        ("q_descale", C.c_float), ("k_descale", C.c_float), ("v_descale", C.c_float),
        ("iterations", C.c_int), ("v_fp16", C.c_int),
        ("s_dump", C.c_void_p),
    ]


class GemmArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int), ("m", C.c_int), ("n", C.c_int), ("k", C.c_int), ("l", C.c_int),
        ("a", C.c_void_p), ("b", C.c_void_p), ("c", C.c_void_p),
        ("alpha", C.c_float), ("beta", C.c_float), ("c_row_major", C.c_int), ("iterations", C.c_int),
        ("c_src", C.c_void_p),
    ]


def _ptr(x):
    if x is None:
        return None
    if isinstance(x, int):
        return x
    return int(x.data_ptr())


class CfkError(RuntimeError):
    def __init__(self, code, detail=""):
        super().__init__(f"cfk_b200 status {code} ({STATUS_NAMES.get(code, '?')}) {detail}")
        self.code = code


class CfkLib:
    def __init__(self, path: str = LIB_PATH):
        if not os.path.exists(path):
            raise FileNotFoundError(
                f"{path} is missing: build it with `make -C cutlass-kernels_b200` (or __graft_entry__.build()); "
                "there is no fallback path")
        self.path = path
        self.lib = C.CDLL(path)
        L = self.lib
        L.cfk_fmha_forward.argtypes = [C.POINTER(FmhaArgs), C.c_void_p]
        L.cfk_fmha_forward_static.argtypes = [C.POINTER(FmhaArgs), C.c_void_p]
        L.cfk_gemm.argtypes = [C.POINTER(GemmArgs), C.c_void_p]
        L.cfk_fill.argtypes = [C.c_void_p, C.c_int, C.c_int64, C.c_uint64, C.c_int64, C.c_int, C.c_float, C.c_float,
                               C.c_void_p]
        L.cfk_convert.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_void_p]
        L.cfk_device_status.argtypes = [C.POINTER(C.c_int)]
        L.cfk_last_cuda_error.restype = C.c_char_p
        L.cfk_selftest_umma.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p] + [C.c_int] * 5 + [C.c_void_p]
        L.cfk_umma_peak.argtypes = [C.c_int, C.c_int, C.POINTER(C.c_double), C.c_void_p]
        L.cfk_selftest_wait_gives_up.argtypes = [C.c_int, C.c_void_p]
        L.cfk_selftest_wait_gives_up_static.argtypes = [C.c_int, C.c_void_p]

    # -- raw calls (return the status code) ---------------------------------------------------
    def fmha_forward_raw(self, args: FmhaArgs, stream=None) -> int:
        return int(self.lib.cfk_fmha_forward(C.byref(args), stream))

    def fmha_forward_static_raw(self, args: FmhaArgs, stream=None) -> int:
        return int(self.lib.cfk_fmha_forward_static(C.byref(args), stream))

    def gemm_raw(self, args: GemmArgs, stream=None) -> int:
        return int(self.lib.cfk_gemm(C.byref(args), stream))

    # -- conveniences ---------------------------------------------------------------------------
    def fmha_args(self, q, k, v, o, *, dtype, batch, heads, seqlen_q, seqlen_kv, head_dim, softmax_scale,
                  causal=False, out_dtype=FP16, p_split_keys=-1, lse=None, mi=None, sprime=None,
                  q_descale=1.0, k_descale=1.0, v_descale=1.0, iterations=1,
                  q_stride=(0, 0, 0), k_stride=(0, 0, 0), v_stride=(0, 0, 0), o_stride=(0, 0, 0),
                  s_dump=None, v_fp16=False) -> FmhaArgs:
        a = FmhaArgs()
        a.dtype, a.out_dtype, a.p_split_keys = dtype, out_dtype, p_split_keys
        a.batch, a.heads, a.seqlen_q, a.seqlen_kv, a.head_dim = batch, heads, seqlen_q, seqlen_kv, head_dim
        a.q, a.k, a.v, a.o = _ptr(q), _ptr(k), _ptr(v), _ptr(o)
        a.lse, a.mi, a.sprime = _ptr(lse), _ptr(mi), _ptr(sprime)
        a.q_stride = (C.c_int64 * 3)(*q_stride)
        a.k_stride = (C.c_int64 * 3)(*k_stride)
        a.v_stride = (C.c_int64 * 3)(*v_stride)
        a.o_stride = (C.c_int64 * 3)(*o_stride)
        a.softmax_scale, a.causal = softmax_scale, int(bool(causal))
        a.q_descale, a.k_descale, a.v_descale = q_descale, k_descale, v_descale
        a.iterations = iterations
        a.s_dump = _ptr(s_dump)
        a.v_fp16 = int(bool(v_fp16))
        return a

    def fmha_forward(self, *pos, stream=None, **kw) -> None:
        rc = self.fmha_forward_raw(self.fmha_args(*pos, **kw), stream)
        if rc:
            raise CfkError(rc, self.last_error())

    def gemm(self, a, b, c, *, dtype, m, n, k, l=1, alpha=1.0, beta=0.0, c_row_major=False, iterations=1,
             c_src=None, stream=None) -> None:
        g = GemmArgs()
        g.dtype, g.m, g.n, g.k, g.l = dtype, m, n, k, l
        g.a, g.b, g.c, g.c_src = _ptr(a), _ptr(b), _ptr(c), _ptr(c_src)
        g.alpha, g.beta, g.c_row_major, g.iterations = alpha, beta, int(bool(c_row_major)), iterations
        rc = self.gemm_raw(g, stream)
        if rc:
            raise CfkError(rc, self.last_error())

    def fill(self, dst, dtype, n, seed, kind="normal", scale=1.0, value=0.0, first_index=0, stream=None) -> None:
        kinds = {"normal": 0, "uniform": 1, "const": 2, "integers": 3}
        rc = int(self.lib.cfk_fill(_ptr(dst), dtype, n, seed, first_index, kinds[kind], scale, value, stream))
        if rc:
            raise CfkError(rc, self.last_error())

    def convert(self, src, src_dtype, dst, dst_dtype, n, scale=1.0, stream=None) -> None:
        rc = int(self.lib.cfk_convert(_ptr(src), src_dtype, _ptr(dst), dst_dtype, n, scale, stream))
        if rc:
            raise CfkError(rc, self.last_error())

    def umma_peak(self, dtype, groups, stream=None) -> float:
        """Enqueues the tensor-core ceiling probe; returns the floating-point operations of the launch."""
        flops = C.c_double(0.0)
        rc = int(self.lib.cfk_umma_peak(dtype, groups, C.byref(flops), stream))
        if rc:
            raise CfkError(rc, self.last_error())
        return float(flops.value)

    def selftest_umma(self, a, b, d, n, a_fmt, b_fmt, b_mn_major, a_from_tmem, stream=None) -> int:
        return int(self.lib.cfk_selftest_umma(_ptr(a), _ptr(b), _ptr(d), n, a_fmt, b_fmt, int(b_mn_major),
                                              int(a_from_tmem), stream))

    def selftest_wait_gives_up(self, limit_ms: int, stream=None) -> int:
        """Enqueues one warp whose bounded wait runs out after `limit_ms`; returns the status code of the launch."""
        return int(self.lib.cfk_selftest_wait_gives_up(limit_ms, stream))

    def selftest_wait_gives_up_static(self, limit_ms: int, stream=None) -> int:
        """The same wait, reporting into the fixed scratch array of cfk_fmha_forward_static."""
        return int(self.lib.cfk_selftest_wait_gives_up_static(limit_ms, stream))

    def device_status(self):
        """(return code, device status word); synchronises the device and clears the word."""
        code = C.c_int(0)
        rc = int(self.lib.cfk_device_status(C.byref(code)))
        return rc, int(code.value)

    def check_device(self) -> None:
        rc, code = self.device_status()
        if rc:
            raise CfkError(rc, f"device status word {code}; {self.last_error()}")

    def last_error(self) -> str:
        return (self.lib.cfk_last_cuda_error() or b"").decode()

    def set_tunable(self, which: int, value: int) -> None:
        rc = int(self.lib.cfk_set_tunable(which, value))
        if rc:
            raise CfkError(rc, "cfk_set_tunable")

    def get_tunable(self, which: int) -> int:
        return int(self.lib.cfk_get_tunable(which))

    def version(self) -> int:
        return int(self.lib.cfk_version())


_lib = None


def load() -> CfkLib:
    global _lib
    if _lib is None:
        _lib = CfkLib()
    return _lib

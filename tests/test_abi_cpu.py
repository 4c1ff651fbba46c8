"""The C-ABI library on a box without a GPU: it loads, exports what include/cfk_b200.h declares,
and rejects bad arguments before touching the device."""
import ctypes as C
import os
import re

import pytest

import cfk_b200

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "cfk_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cfk_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(lib):
    names = declared_functions()
    assert "cfk_fmha_forward" in names and "cfk_gemm" in names
    for n in names:
        assert hasattr(lib.lib, n), f"{n} is declared in include/cfk_b200.h but not exported"
    assert sorted(cfk_b200.EXPORTS) == [n for n in names if n in cfk_b200.EXPORTS]
    assert lib.version() >= 100


def test_struct_layout_matches_header(lib):
    # sizes as the C compiler lays them out for the declarations in the header
    assert C.sizeof(cfk_b200.FmhaArgs) == 8 * 4 + 7 * 8 + 12 * 8 + 4 + 4 + 3 * 4 + 4 + (4 + 4) + 8   # v_fp16 + padding
    assert C.sizeof(cfk_b200.GemmArgs) == 5 * 4 + 4 + 3 * 8 + 4 * 4 + 8


def _args(lib, **over):
    kw = dict(dtype=cfk_b200.FP16, batch=1, heads=2, seqlen_q=128, seqlen_kv=128, head_dim=64, softmax_scale=0.125)
    kw.update(over)
    return lib.fmha_args(kw.pop("q", 0x1000), 0x2000, 0x3000, 0x4000, **kw)


@pytest.mark.parametrize("over,code", [
    (dict(batch=0), 1), (dict(seqlen_q=-1), 1), (dict(softmax_scale=0.0), 1), (dict(softmax_scale=float("nan")), 1),
    (dict(dtype=cfk_b200.FP32), 1), (dict(out_dtype=cfk_b200.E4M3), 1),
    (dict(head_dim=96), 2), (dict(head_dim=512), 2),
    (dict(p_split_keys=-2), 1),
    (dict(causal=True, seqlen_q=256, seqlen_kv=128), 2),
    (dict(q=0x1008), 1), (dict(q_stride=(128 * 2 * 64, 2 * 64 + 3, 64)), 1),
    (dict(dtype=cfk_b200.E4M3, head_dim=128, q_descale=0.0), 1),
])
def test_fmha_rejects_bad_arguments(lib, over, code):
    assert lib.fmha_forward_raw(_args(lib, **over)) == code


def test_fmha_null_pointers(lib):
    a = _args(lib)
    a.o = None
    assert lib.fmha_forward_raw(a) == 1
    assert lib.lib.cfk_fmha_forward(None, None) == 1


@pytest.mark.parametrize("over,code", [
    (dict(m=0), 1), (dict(k=12), 2), (dict(n=100), 2), (dict(dtype=cfk_b200.E4M3), 2), (dict(a=0x1004), 1),
])
def test_gemm_rejects_bad_arguments(lib, over, code):
    g = cfk_b200.GemmArgs()
    g.dtype, g.m, g.n, g.k, g.l = cfk_b200.FP16, 128, 256, 64, 1
    g.a, g.b, g.c = 0x1000, 0x2000, 0x3000
    g.alpha, g.beta, g.iterations = 1.0, 0.0, 1
    for k2, v2 in over.items():
        setattr(g, k2, v2)
    assert lib.gemm_raw(g) == code
    assert lib.lib.cfk_gemm(None, None) == 1


def test_missing_library_fails_loudly(tmp_path):
    with pytest.raises(FileNotFoundError):
        cfk_b200.CfkLib(str(tmp_path / "libcfk_b200.so"))


def test_fill_and_convert_reject_bad_arguments(lib):
    assert lib.lib.cfk_fill(None, 0, 10, 1, 0, 0, 1.0, 0.0, None) == 1
    assert lib.lib.cfk_fill(0x1000, 9, 10, 1, 0, 0, 1.0, 0.0, None) == 1
    assert lib.lib.cfk_convert(0x1000, 0, None, 1, 10, 1.0, None) == 1


@pytest.mark.parametrize("a_fmt,b_fmt", [(cfk_b200.FP16, cfk_b200.BF16), (cfk_b200.BF16, cfk_b200.FP16),
                                         (cfk_b200.FP16, cfk_b200.E4M3), (cfk_b200.E4M3, cfk_b200.BF16)])
@pytest.mark.parametrize("a_from_tmem", [0, 1])
def test_selftest_umma_refuses_mixed_operand_formats_before_any_launch(lib, a_fmt, b_fmt, a_from_tmem):
    """One MMA instruction takes A and B in one format; a mixed pair faults the tensor core, so the entry point
    refuses it on the host (this box has no device: a launch attempt would return a different code)."""
    assert lib.selftest_umma(0x1000, 0x2000, 0x3000, 128, a_fmt, b_fmt, 0, a_from_tmem) == 2


def test_selftest_umma_takes_no_descriptor_overrides(lib):
    """The descriptor fields of B are fixed to what the kernels use: the entry point has no parameter for them."""
    assert len(lib.lib.cfk_selftest_umma.argtypes) == 9
    text = open(os.path.join(ROOT, "include", "cfk_b200.h")).read()
    decl = text[text.index("int cfk_selftest_umma("):]
    decl = decl[:decl.index(";")]
    assert "lbo" not in decl and "sbo" not in decl and "step" not in decl

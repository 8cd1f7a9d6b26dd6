"""The C-ABI library loads without a GPU and exports every symbol include/flashback_b200.h
declares; argument validation (which runs before any device call) returns the documented
status codes. No compute call is made here."""

import ctypes
import re
from pathlib import Path

import pytest

from flashback_cute import _lib

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "flashback_b200.h"


def _declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(fb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = _declared_functions()
    assert {"fb_jvp_fwd", "fb_hvp_bwd", "fb_bwd_row_stats"} <= set(names)
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"


def test_binding_lists_match_header():
    assert set(_lib.EXPORTS) <= set(_declared_functions())


def test_struct_layout_matches_library():
    lib = _lib.load()
    lib.fb_abi_sizeof.restype = ctypes.c_size_t
    structs = (_lib.FbTensor, _lib.FbProblem, _lib.FbJvpArgs, _lib.FbStatsArgs, _lib.FbHvpArgs, _lib.FbBwdNoAllocArgs, _lib.FbKvScatter)
    for i, s in enumerate(structs):
        assert lib.fb_abi_sizeof(i) == ctypes.sizeof(s), s.__name__
    assert lib.fb_abi_sizeof(len(structs)) == 0


def test_binding_covers_every_declared_symbol():
    assert set(_declared_functions()) == set(_lib.EXPORTS)


def test_workspace_bytes():
    lib = _lib.load()
    lib.fb_workspace_bytes.restype = ctypes.c_size_t
    lib.fb_workspace_bytes.argtypes = [ctypes.POINTER(_lib.FbProblem), ctypes.c_int]
    pr = _lib.FbProblem(dtype=0, batch=2, heads_q=32, heads_kv=8, head_dim=128, seqlen_q=8192, seqlen_k=8192,
                        causal=1, total_q=2 * 8192, total_k=2 * 8192)
    assert lib.fb_workspace_bytes(ctypes.byref(pr), 0) == 32 * 2 * 8192 * 4
    assert lib.fb_workspace_bytes(ctypes.byref(pr), 1) == 0
    assert lib.fb_workspace_bytes(None, 0) == 0


def test_version_and_status_strings():
    lib = _lib.load()
    assert lib.fb_version() >= 100
    assert lib.fb_status_string(0) == b"ok"
    assert b"64 or 128" in lib.fb_status_string(-3)
    assert lib.fb_status_string(-12345) == b"unknown status"


def _prob(**kw):
    base = dict(dtype=0, batch=1, heads_q=2, heads_kv=2, head_dim=64, seqlen_q=8, seqlen_k=8, causal=0,
                total_q=8, total_k=8, cu_seqlens_q=None, cu_seqlens_k=None, softmax_scale=0.125, flags=0, seg_rows=0, seg_shift=0)
    base.update(kw)
    for n in ("seg_rows", "seg_shift"):  # first break / shift only
        base[n] = (ctypes.c_int32 * 4)(base[n], 0, 0, 0)
    return _lib.FbProblem(*[base[f[0]] for f in _lib.FbProblem._fields_])


@pytest.mark.parametrize(
    "kw,code",
    [
        (dict(dtype=7), -2),
        (dict(head_dim=96), -3),
        (dict(heads_q=3, heads_kv=2), -4),
        (dict(total_q=9), -5),
        (dict(batch=0), -5),
        (dict(flags=_lib.FB_FLAG_DKV_SPLIT(3)), -9),
        (dict(seqlen_q=256, seqlen_k=512, total_q=256, total_k=512, seg_rows=128, seg_shift=64), -9),            # query segments need causal
        (dict(seqlen_q=256, seqlen_k=512, total_q=256, total_k=512, causal=1, seg_rows=64, seg_shift=64), -5),   # break not on a 128-row boundary
        (dict(seqlen_q=256, seqlen_k=512, total_q=256, total_k=512, causal=1, seg_rows=384, seg_shift=64), -5),  # break beyond the query rows
        (dict(seqlen_q=256, seqlen_k=512, total_q=256, total_k=512, causal=1, seg_rows=128, seg_shift=-1), -5),
        (dict(seqlen_q=256, seqlen_k=512, total_q=256, total_k=512, causal=1, seg_rows=0, seg_shift=64), -5),    # a shift without a break
    ],
)
def test_problem_validation_codes(kw, code):
    lib = _lib.load()
    args = _lib.FbJvpArgs(prob=_prob(**kw))
    assert lib.fb_jvp_fwd(ctypes.byref(args), None) == code
    hargs = _lib.FbHvpArgs(prob=_prob(**kw))
    assert lib.fb_hvp_bwd(ctypes.byref(hargs), None) == code


def test_null_and_alignment_validation():
    lib = _lib.load()
    assert lib.fb_jvp_fwd(None, None) == -1
    args = _lib.FbJvpArgs(prob=_prob())
    assert lib.fb_jvp_fwd(ctypes.byref(args), None) == -1  # q missing
    t = _lib.FbTensor(0x1008, 128, 64)  # not 16-byte aligned
    args = _lib.FbJvpArgs(prob=_prob(), q=t, k=t, v=t)
    assert lib.fb_jvp_fwd(ctypes.byref(args), None) == -6
    t = _lib.FbTensor(0x1000, 130, 64)  # stride not a multiple of 8 elements
    args = _lib.FbJvpArgs(prob=_prob(), q=t, k=t, v=t)
    assert lib.fb_jvp_fwd(ctypes.byref(args), None) == -6


def test_mode_validation():
    lib = _lib.load()
    t = _lib.FbTensor(0x1000, 128, 64)
    # one tangent without the others
    args = _lib.FbJvpArgs(prob=_prob(), q=t, k=t, v=t, q_dot=t)
    assert lib.fb_jvp_fwd(ctypes.byref(args), None) == -9
    # directional outputs requested without tangents
    h = _lib.FbHvpArgs(prob=_prob(), q=t, k=t, v=t, dout=t, dq_dot=t)
    assert lib.fb_hvp_bwd(ctypes.byref(h), None) == -9


def test_status_to_exception_mapping():
    with pytest.raises(TypeError):
        _lib.raise_for_status(-2)
    with pytest.raises(NotImplementedError):
        _lib.raise_for_status(-3)
    with pytest.raises(ValueError):
        _lib.raise_for_status(-4)
    with pytest.raises(NotImplementedError):
        _lib.raise_for_status(-7)
    with pytest.raises(RuntimeError):
        _lib.raise_for_status(-5)


def test_no_cpu_path():
    """CPU tensors are refused loudly instead of being routed anywhere else."""
    import torch
    from flashback_cute import flashback_attn_func

    q = torch.zeros(1, 8, 2, 64, dtype=torch.bfloat16)
    with pytest.raises(NotImplementedError):
        flashback_attn_func(q, q, q)


def test_header_is_valid_c_and_links(tmp_path):
    """The public header compiles as plain C (no C++-isms) and a C program linking the library
    resolves the entry points; it runs the argument validation only (no GPU needed)."""
    import shutil
    import subprocess

    if shutil.which("gcc") is None:
        pytest.skip("gcc not available")
    src = tmp_path / "use_abi.c"
    src.write_text(
        '#include "flashback_b200.h"\n'
        "#include <stdio.h>\n"
        "int main(void) {\n"
        "  fb_jvp_args a = {0};\n"
        "  a.prob.dtype = 7;\n"
        "  int s1 = fb_jvp_fwd(&a, NULL);\n"
        "  int s2 = fb_hvp_bwd(NULL, NULL);\n"
        "  fb_bwd_noalloc_args n = {0};\n"
        "  n.prob.heads_q = 64; n.prob.total_q = FB_NOALLOC_MAX_STAT_FLOATS;\n"
        "  int s3 = fb_bwd_noalloc(&n, NULL);\n"
        '  printf("%d %d %d %d %s\\n", s1, s2, s3, fb_version(), fb_status_string(s1));\n'
        "  return 0;\n"
        "}\n"
    )
    lib_dir = _lib._LIB_PATH.parent
    exe = tmp_path / "use_abi"
    subprocess.run(
        ["gcc", "-std=c99", "-Wall", "-Werror", "-I", str(ROOT / "include"), str(src), "-o", str(exe),
         "-L", str(lib_dir), "-lflashback_b200", f"-Wl,-rpath,{lib_dir}"],
        check=True, capture_output=True, text=True,
    )
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    assert out[:3] == ["-2", "-1", "-10"]
    assert int(out[3]) >= 100

"""ctypes binding of libflashback_b200.so (C ABI declared in include/flashback_b200.h).

The library is the only compute path: if it is missing or a call fails this module raises;
nothing here falls back to PyTorch or CPU code.
"""

from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path
from typing import Optional

import torch

# FLASHBACK_LIB selects another build of the same library (e.g. the instrumented one, build.py --profile)
_LIB_PATH = Path(os.environ.get("FLASHBACK_LIB") or Path(__file__).resolve().parent / "libflashback_b200.so")
_lib = None
_lock = threading.Lock()
_launches = 0  # kernels enqueued through this module since import (launch accounting for bench.py)

FB_BF16, FB_F16, FB_F32 = 0, 1, 2
FB_FLAG_FORCE_SIMT = 1
FB_FLAG_TILE_MAJOR = 2
FB_FLAG_KV_OUT_F32 = 4       # hvp_bwd: dk, dv, dk_dot, dv_dot are float32 tensors ...
FB_FLAG_KV_ACCUMULATE = 8    # ... and results are added to their contents
FB_FLAG_SEG_KEYS = 16        # fb_problem.seg_rows / seg_shift describe the key rows (dK/dV-side kernels only)


def FB_FLAG_SCHED_GROUP(n: int) -> int:
    """Tensor-core kernels: (head, batch) pairs per scheduling group; 0 = automatic."""
    return (n & 0xFFF) << 12


def FB_FLAG_DKV_SPLIT(n: int) -> int:
    """dK/dV kernels: force the number of CTAs (1, 2, 4, 8) that share a key tile; 0 = automatic."""
    return (n & 15) << 8


# fb_problem.flags used when a caller of `problem()` passes none (tuning experiments: FLASHBACK_FLAGS=<int>)
DEFAULT_FLAGS = int(os.environ.get("FLASHBACK_FLAGS", "0"))
_DTYPES = {torch.bfloat16: FB_BF16, torch.float16: FB_F16, torch.float32: FB_F32}

FB_ERR_DTYPE, FB_ERR_HEAD_DIM, FB_ERR_HEADS, FB_ERR_ARCH = -2, -3, -4, -7


class FbTensor(ctypes.Structure):
    _fields_ = [("ptr", ctypes.c_void_p), ("row_stride", ctypes.c_int64), ("head_stride", ctypes.c_int64)]


class FbProblem(ctypes.Structure):
    _fields_ = [
        ("dtype", ctypes.c_int32), ("batch", ctypes.c_int32), ("heads_q", ctypes.c_int32), ("heads_kv", ctypes.c_int32),
        ("head_dim", ctypes.c_int32), ("seqlen_q", ctypes.c_int32), ("seqlen_k", ctypes.c_int32), ("causal", ctypes.c_int32),
        ("total_q", ctypes.c_int64), ("total_k", ctypes.c_int64),
        ("cu_seqlens_q", ctypes.c_void_p), ("cu_seqlens_k", ctypes.c_void_p),
        ("softmax_scale", ctypes.c_float), ("flags", ctypes.c_int32),
        ("seg_rows", ctypes.c_int32 * 4), ("seg_shift", ctypes.c_int32 * 4),
    ]


class FbJvpArgs(ctypes.Structure):
    _fields_ = [
        ("prob", FbProblem),
        ("q", FbTensor), ("k", FbTensor), ("v", FbTensor),
        ("q_dot", FbTensor), ("k_dot", FbTensor), ("v_dot", FbTensor),
        ("out", FbTensor), ("out_dot", FbTensor),
        ("lse", ctypes.c_void_p), ("z1", ctypes.c_void_p),
        ("dout", FbTensor), ("dout_dot", FbTensor),
        ("dpsum", ctypes.c_void_p), ("ddot", ctypes.c_void_p),
        ("lse_known", ctypes.c_int32),
    ]


class FbStatsArgs(ctypes.Structure):
    _fields_ = [
        ("prob", FbProblem),
        ("out", FbTensor), ("dout", FbTensor), ("out_dot", FbTensor), ("dout_dot", FbTensor),
        ("dpsum", ctypes.c_void_p), ("ddot", ctypes.c_void_p),
    ]


class FbHvpArgs(ctypes.Structure):
    _fields_ = [
        ("prob", FbProblem),
        ("q", FbTensor), ("k", FbTensor), ("v", FbTensor), ("dout", FbTensor),
        ("q_dot", FbTensor), ("k_dot", FbTensor), ("v_dot", FbTensor), ("dout_dot", FbTensor),
        ("lse", ctypes.c_void_p), ("dpsum", ctypes.c_void_p), ("z1", ctypes.c_void_p), ("ddot", ctypes.c_void_p),
        ("dq", FbTensor), ("dk", FbTensor), ("dv", FbTensor),
        ("dq_dot", FbTensor), ("dk_dot", FbTensor), ("dv_dot", FbTensor),
    ]


class FbBwdNoAllocArgs(ctypes.Structure):
    _fields_ = [
        ("prob", FbProblem),
        ("q", FbTensor), ("k", FbTensor), ("v", FbTensor), ("out", FbTensor), ("dout", FbTensor),
        ("lse", ctypes.c_void_p),
        ("dq", FbTensor), ("dk", FbTensor), ("dv", FbTensor),
    ]


class FbKvScatter(ctypes.Structure):
    _fields_ = [
        ("n_peers", ctypes.c_int32), ("rows_per_peer", ctypes.c_int32),
        ("row_stride", ctypes.c_int64), ("head_stride", ctypes.c_int64), ("accumulate_rows", ctypes.c_int64),
        ("dk", ctypes.c_void_p * 8), ("dv", ctypes.c_void_p * 8), ("dk_dot", ctypes.c_void_p * 8), ("dv_dot", ctypes.c_void_p * 8),
    ]


NOALLOC_MAX_STAT_FLOATS = 1 << 20

EXPORTS = (
    "fb_jvp_fwd", "fb_bwd_row_stats", "fb_hvp_bwd", "fb_bwd_noalloc", "fb_last_launch_count", "fb_check_device_status",
    "fb_status_string", "fb_last_cuda_error", "fb_version", "fb_abi_sizeof", "fb_workspace_bytes", "fb_debug_profile",
    "fb_debug_wait_timeout", "fb_hvp_bwd_scatter", "fb_sum_slots",
)


def load() -> ctypes.CDLL:
    """Load the shared library once. Raises if it has not been built."""
    global _lib
    with _lock:
        if _lib is None:
            if not _LIB_PATH.exists():
                raise RuntimeError(
                    f"{_LIB_PATH} not found: build it with `python flashback-cute_b200/build.py` "
                    "(there is no fallback path)"
                )
            lib = ctypes.CDLL(str(_LIB_PATH))
            for name, argt in (("fb_jvp_fwd", FbJvpArgs), ("fb_bwd_row_stats", FbStatsArgs), ("fb_hvp_bwd", FbHvpArgs),
                               ("fb_bwd_noalloc", FbBwdNoAllocArgs)):
                fn = getattr(lib, name)
                fn.argtypes = [ctypes.POINTER(argt), ctypes.c_void_p]
                fn.restype = ctypes.c_int
            lib.fb_hvp_bwd_scatter.argtypes = [ctypes.POINTER(FbHvpArgs), ctypes.POINTER(FbKvScatter), ctypes.c_void_p]
            lib.fb_hvp_bwd_scatter.restype = ctypes.c_int
            lib.fb_sum_slots.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                         ctypes.POINTER(ctypes.c_int64), ctypes.c_void_p, ctypes.c_void_p]
            lib.fb_sum_slots.restype = ctypes.c_int
            lib.fb_debug_wait_timeout.argtypes = [ctypes.POINTER(FbJvpArgs), ctypes.c_longlong, ctypes.c_void_p]
            lib.fb_debug_wait_timeout.restype = ctypes.c_int
            lib.fb_abi_sizeof.argtypes = [ctypes.c_int]
            lib.fb_abi_sizeof.restype = ctypes.c_size_t
            lib.fb_status_string.argtypes = [ctypes.c_int]
            lib.fb_status_string.restype = ctypes.c_char_p
            lib.fb_last_cuda_error.restype = ctypes.c_char_p
            lib.fb_last_launch_count.restype = ctypes.c_int
            lib.fb_check_device_status.restype = ctypes.c_int
            lib.fb_version.restype = ctypes.c_int
            _lib = lib
    return _lib


def launches() -> int:
    return _launches


def raise_for_status(status: int) -> None:
    """Map a C status to the exception class the reference raises for the same condition
    (flashback_cute/interface.py:362-370)."""
    if status == 0:
        return
    lib = load()
    msg = lib.fb_status_string(status).decode()
    if status == -8:
        msg += ": " + lib.fb_last_cuda_error().decode()
    if status in (FB_ERR_HEAD_DIM, FB_ERR_ARCH):
        raise NotImplementedError(msg)
    if status == FB_ERR_DTYPE:
        raise TypeError(msg)
    if status == FB_ERR_HEADS:
        raise ValueError(msg)
    raise RuntimeError(f"flashback_b200 error {status}: {msg}")


def check_device_status() -> None:
    """Synchronise and raise if a kernel's bounded wait gave up."""
    raise_for_status(load().fb_check_device_status())


def raw(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """Strip torch.func grad-tracking wrappers. Inside a `jvp` rule saved tensors, tangents and even
    freshly created tensors are wrappers without storage; the tensor underneath shares the memory
    the kernels read and write."""
    if t is None:
        return None
    ft = torch._C._functorch
    while ft.is_gradtrackingtensor(t):
        t = ft.get_unwrapped(t)
    return t


def seq_tensor(t: Optional[torch.Tensor]) -> FbTensor:
    """(B,S,H,D) or (T,H,D) tensor -> rows x heads view. Requires unit stride on D and, for 4-d
    tensors, batch stride == S * row stride (callers make tensors contiguous otherwise)."""
    if t is None:
        return FbTensor(None, 0, 0)
    t = raw(t)
    return FbTensor(t.data_ptr(), t.stride(-3), t.stride(-2))


def rows_ok(t: torch.Tensor) -> bool:
    t = raw(t)
    if t.stride(-1) != 1:
        return False
    if t.dim() == 4 and t.shape[0] > 1 and t.stride(0) != t.shape[1] * t.stride(1):
        return False
    return t.stride(-3) % 8 == 0 and t.stride(-2) % 8 == 0 and t.data_ptr() % 16 == 0


def problem(q, k, cu_q, cu_k, max_q, max_k, scale, causal, flags=None, segments=()) -> FbProblem:
    """`segments`: up to four (break row, shift) pairs, fb_problem.seg_rows / seg_shift (empty = off); they
    describe the query rows, or with FB_FLAG_SEG_KEYS in `flags` the key rows."""
    if flags is None:
        flags = DEFAULT_FLAGS
    if q.dtype not in _DTYPES:
        raise TypeError("q, k, v must share a dtype in {float16, bfloat16, float32}")
    if cu_q is None:
        B, Sq, Hq, D = q.shape
        Sk, Hkv = k.shape[1], k.shape[2]
        Tq, Tk = B * Sq, B * Sk
    else:
        Tq, Hq, D = q.shape
        Tk, Hkv = k.shape[0], k.shape[1]
        B, Sq, Sk = cu_q.numel() - 1, int(max_q), int(max_k)
    return FbProblem(
        _DTYPES[q.dtype], B, Hq, Hkv, D, Sq, Sk, int(bool(causal)), Tq, Tk,
        None if cu_q is None else raw(cu_q).data_ptr(), None if cu_k is None else raw(cu_k).data_ptr(),
        float(scale), flags,
        (ctypes.c_int32 * 4)(*[int(r) for r, _ in segments]), (ctypes.c_int32 * 4)(*[int(sh) for _, sh in segments]),
    )


def _fptr(t: Optional[torch.Tensor]):
    return None if t is None else raw(t).data_ptr()


def _stream(t: torch.Tensor):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _call(name: str, args, ref: torch.Tensor, *extra) -> None:
    global _launches
    lib = _lib or load()
    if not ref.is_cuda:
        raise RuntimeError("flashback_b200 has no CPU path: tensors must live on a CUDA device")
    fn = getattr(lib, name)
    if ref.device.index == torch.cuda.current_device():  # the common case: no device switch needed
        status = fn(ctypes.byref(args), *extra, _stream(ref))
        if status == 0:
            _launches += lib.fb_last_launch_count()
    else:
        with torch.cuda.device(ref.device):
            status = fn(ctypes.byref(args), *extra, _stream(ref))
            if status == 0:
                _launches += lib.fb_last_launch_count()
    if status != 0:
        raise_for_status(status)


def jvp_fwd(prob, q, k, v, qd, kd, vd, out, out_dot, lse, z1, dout=None, dout_dot=None, dpsum=None, ddot=None, lse_known=False):
    a = FbJvpArgs(
        prob, seq_tensor(q), seq_tensor(k), seq_tensor(v), seq_tensor(qd), seq_tensor(kd), seq_tensor(vd),
        seq_tensor(out), seq_tensor(out_dot), _fptr(lse), _fptr(z1), seq_tensor(dout), seq_tensor(dout_dot),
        _fptr(dpsum), _fptr(ddot), int(lse_known),
    )
    _call("fb_jvp_fwd", a, q)


def debug_wait_timeout(prob, q, k, v, out, lse, budget_cycles: int):
    """Test hook (fb_debug_wait_timeout): plain forward in the instantiation whose producer leaves out one
    stage's loads, so that a bounded wait runs out after `budget_cycles` and the kernels report it."""
    a = FbJvpArgs(prob, seq_tensor(q), seq_tensor(k), seq_tensor(v), seq_tensor(None), seq_tensor(None), seq_tensor(None),
                  seq_tensor(out), seq_tensor(None), _fptr(lse), None, seq_tensor(None), seq_tensor(None), None, None, 0)
    _call("fb_debug_wait_timeout", a, q, ctypes.c_longlong(int(budget_cycles)))


def bwd_row_stats(prob, out, dout, out_dot, dout_dot, dpsum, ddot):
    a = FbStatsArgs(prob, seq_tensor(out), seq_tensor(dout), seq_tensor(out_dot), seq_tensor(dout_dot), _fptr(dpsum), _fptr(ddot))
    _call("fb_bwd_row_stats", a, out)


def bwd_noalloc(prob, q, k, v, out, dout, lse, dq, dk, dv):
    """First-order backward through the entry point that allocates nothing (its dpsum scratch
    lives in a fixed array inside the library; heads_q*total_q <= NOALLOC_MAX_STAT_FLOATS)."""
    a = FbBwdNoAllocArgs(prob, seq_tensor(q), seq_tensor(k), seq_tensor(v), seq_tensor(out), seq_tensor(dout), _fptr(lse),
                         seq_tensor(dq), seq_tensor(dk), seq_tensor(dv))
    _call("fb_bwd_noalloc", a, q)


def hvp_bwd(prob, q, k, v, dout, qd, kd, vd, dout_dot, lse, dpsum, z1, ddot, dq, dk, dv, dqd, dkd, dvd):
    a = FbHvpArgs(
        prob, seq_tensor(q), seq_tensor(k), seq_tensor(v), seq_tensor(dout),
        seq_tensor(qd), seq_tensor(kd), seq_tensor(vd), seq_tensor(dout_dot),
        _fptr(lse), _fptr(dpsum), _fptr(z1), _fptr(ddot),
        seq_tensor(dq), seq_tensor(dk), seq_tensor(dv), seq_tensor(dqd), seq_tensor(dkd), seq_tensor(dvd),
    )
    _call("fb_hvp_bwd", a, q)


def kv_scatter(n_peers: int, rows_per_peer: int, row_stride: int, head_stride: int, dk=(), dv=(), dk_dot=(), dv_dot=(),
               accumulate_rows: int = 0) -> FbKvScatter:
    """Destinations of fb_hvp_bwd_scatter: per output a list of n_peers device addresses (ints), one per
    owner of a block of rows_per_peer key rows; strides in float32 elements. accumulate_rows: key rows
    below it have a local partial sum to add (0 = all rows)."""
    sc = FbKvScatter(n_peers=n_peers, rows_per_peer=rows_per_peer, row_stride=row_stride, head_stride=head_stride,
                     accumulate_rows=accumulate_rows)
    for name, ptrs in (("dk", dk), ("dv", dv), ("dk_dot", dk_dot), ("dv_dot", dv_dot)):
        arr = getattr(sc, name)
        for i, p in enumerate(ptrs):
            arr[i] = int(p)
    return sc


def hvp_bwd_scatter(prob, scatter: FbKvScatter, q, k, v, dout, qd, kd, vd, dout_dot, lse, dpsum, z1, ddot, dk, dv, dkd, dvd):
    """fb_hvp_bwd_scatter: dK/dV-side kernels only; dk, dv, dkd, dvd are the LOCAL float32 partial tensors
    (read and added when the problem's flags say accumulate), the sums go to `scatter`'s destinations."""
    global _launches
    a = FbHvpArgs(
        prob, seq_tensor(q), seq_tensor(k), seq_tensor(v), seq_tensor(dout),
        seq_tensor(qd), seq_tensor(kd), seq_tensor(vd), seq_tensor(dout_dot),
        _fptr(lse), _fptr(dpsum), _fptr(z1), _fptr(ddot),
        seq_tensor(None), seq_tensor(dk), seq_tensor(dv), seq_tensor(None), seq_tensor(dkd), seq_tensor(dvd),
    )
    lib = _lib or load()
    if not q.is_cuda:
        raise RuntimeError("flashback_b200 has no CPU path: tensors must live on a CUDA device")
    with torch.cuda.device(q.device):
        status = lib.fb_hvp_bwd_scatter(ctypes.byref(a), ctypes.byref(scatter), _stream(q))
        if status == 0:
            _launches += lib.fb_last_launch_count()
    raise_for_status(status)


def sum_slots(slots: torch.Tensor, out: torch.Tensor, valid=None, period: int = 0):
    """out = sum over s of slots[s] (float32, GPU), by the library's kernel. `slots[s]` must be a contiguous
    block shaped like `out`; the slots may be strided views (slots.stride(0) elements apart). `valid`:
    optional list of element counts - only the first valid[s] elements of every block of `period` elements
    of slot s take part (period 0: the slot is one block)."""
    global _launches
    lib = _lib or load()
    if not (slots.is_cuda and out.is_contiguous() and slots.dtype == out.dtype == torch.float32 and slots[0].is_contiguous()):
        raise ValueError("sum_slots expects float32 CUDA tensors with contiguous slots")
    n, count = slots.shape[0], out.numel()
    if slots[0].numel() != count:
        raise ValueError("every slot must have out's number of elements")
    varr = None if valid is None else (ctypes.c_int64 * n)(*[int(x) for x in valid])
    with torch.cuda.device(slots.device):
        status = lib.fb_sum_slots(slots.data_ptr(), n, slots.stride(0) if n > 1 else count, count, period, varr, out.data_ptr(), _stream(slots))
        if status == 0:
            _launches += lib.fb_last_launch_count()
    raise_for_status(status)

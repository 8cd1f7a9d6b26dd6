"""Twice-differentiable softmax attention on B200 (sm_100a).

Drop-in for the reference's `flashback_cute/interface.py`: the public entry points
`flashback_attn_func` / `flashback_attn_varlen_func` keep their names, argument order, defaults,
tensor layouts and exception types (flashback_cute/interface.py:362-409), and the autograd
structure is the same three pieces (interface.py:275-359):

  _FlashbackAttnFunc      forward = attention; backward delegates to
  _FlashbackAttnBwdFunc   forward = first-order backward; backward = the fused double backward
  _NoThirdOrderGrad       identity whose backward raises

What differs: every device step is a call through the C ABI of libflashback_b200.so (no FA4, no
CuTe-DSL, no JIT), both Functions also define `jvp` so the op works under forward-mode AD
(`torch.func.jvp`, `torch.autograd.forward_ad`), float32 inputs are accepted, and two functional
entry points expose the kernels directly: `flashback_attn_jvp` (O, O_dot in one fused pass) and
`flashback_attn_hvp` (dQ, dK, dV and their directional derivatives from dO and dO_dot).

Double backward, in the reference's notation (interface.py:7-13): with (gq, gk, gv) the
cotangents of (dq, dk, dv),  dot_dout = JVP of attention along (gq, gk, gv)  and
(dot_q, dot_k, dot_v) = directional derivative of (dq, dk, dv) along (gq, gk, gv) at fixed dout.
"""

from __future__ import annotations

import inspect
from typing import Optional

import torch

from . import _lib


_raw = _lib.raw


def _rows(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """Return `t` in a layout the kernels take (unit stride on head_dim, batch folded into rows),
    copying only if needed (the reference calls .contiguous() unconditionally, interface.py:186-188)."""
    if t is None:
        return None
    return t if _lib.rows_ok(t) else t.contiguous()


def _stat(q: torch.Tensor, cu_q) -> torch.Tensor:
    """fp32 row-statistics buffer, shape (heads_q, total_q)."""
    heads = q.shape[-2]
    total = q.shape[0] * q.shape[1] if cu_q is None else q.shape[0]
    return torch.empty(heads, total, dtype=torch.float32, device=q.device)


class _Geom:
    """Per-call geometry shared by the helpers below."""

    def __init__(self, q, k, cu_q, cu_k, max_q, max_k, scale, causal):
        self.cu_q, self.cu_k, self.max_q, self.max_k = cu_q, cu_k, max_q, max_k
        self.scale, self.causal = float(scale), bool(causal)
        self.prob = _lib.problem(q, k, cu_q, cu_k, max_q, max_k, scale, causal)
        self.empty = q.numel() == 0 or k.numel() == 0


def _forward(g: _Geom, q, k, v):
    """O and LSE (natural log, (heads_q, total_q))."""
    out = torch.empty_like(q)
    lse = _stat(q, g.cu_q)
    if g.empty:
        return out.zero_(), lse.fill_(float("-inf"))
    _lib.jvp_fwd(g.prob, q, k, v, None, None, None, out, None, lse, None)
    return out, lse


def _jvp_fused(g: _Geom, q, k, v, qd, kd, vd):
    """One pass: O, LSE, O_dot, z1."""
    out, out_dot = torch.empty_like(q), torch.empty_like(q)
    lse, z1 = _stat(q, g.cu_q), _stat(q, g.cu_q)
    if g.empty:
        return out.zero_(), lse.fill_(float("-inf")), out_dot.zero_(), z1.zero_()
    _lib.jvp_fwd(g.prob, q, k, v, qd, kd, vd, out, out_dot, lse, z1)
    return out, lse, out_dot, z1


def _jvp_lse_known(g: _Geom, q, k, v, qd, kd, vd, out, lse, dout=None, dout_dot=None):
    """O and LSE already known (the reference's K1 situation): O_dot, z1 and, with dout, the row
    statistics dpsum = rowsum(dO*O), ddot = rowsum(dO_dot*O + dO*O_dot)."""
    out_dot = torch.empty_like(q)
    z1 = _stat(q, g.cu_q)
    dpsum = ddot = None
    if dout is not None:
        dpsum, ddot = _stat(q, g.cu_q), _stat(q, g.cu_q)
    _lib.jvp_fwd(g.prob, q, k, v, qd, kd, vd, out, out_dot, lse, z1, dout, dout_dot, dpsum, ddot, lse_known=True)
    return out_dot, z1, dpsum, ddot


def _backward(g: _Geom, q, k, v, out, dout, lse):
    """First-order dq, dk, dv."""
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    if g.empty:
        return dq.zero_(), dk.zero_(), dv.zero_()
    dpsum = _stat(q, g.cu_q)
    _lib.bwd_row_stats(g.prob, out, dout, None, None, dpsum, None)
    _lib.hvp_bwd(g.prob, q, k, v, dout, None, None, None, None, lse, dpsum, None, None, dq, dk, dv, None, None, None)
    return dq, dk, dv


def _double_backward(g: _Geom, q, k, v, out, dout, lse, gdq, gdk, gdv):
    """(dot_q, dot_k, dot_v, dot_dout): grads of <(dq,dk,dv),(gdq,gdk,gdv)> w.r.t. (q,k,v,dout).
    Same contract as the reference's _double_backward (interface.py:178-272): JVP-forward kernel
    (dot_dout, z1, ddot; dpsum comes out of the same epilogue), then HVP-backward kernels."""
    if g.empty:
        return torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v), torch.zeros_like(dout)
    q, k, v, out, dout, gdq, gdk, gdv = map(_rows, (q, k, v, out, dout, gdq, gdk, gdv))
    dot_dout, z1, dpsum, ddot = _jvp_lse_known(g, q, k, v, gdq, gdk, gdv, out, lse, dout)
    dot_q, dot_k, dot_v = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    _lib.hvp_bwd(g.prob, q, k, v, dout, gdq, gdk, gdv, None, lse, dpsum, z1, ddot, None, None, None, dot_q, dot_k, dot_v)
    return dot_q, dot_k, dot_v, dot_dout


def _zeros_if_none(t, like):
    return torch.zeros_like(like) if t is None else t


class _NoThirdOrderGrad(torch.autograd.Function):
    """Identity on the double-backward results whose backward raises (the results depend on
    q/k/v/dout through saved tensors, so without this guard a third derivative would silently
    treat them as constants; same guard as interface.py:275-291)."""

    @staticmethod
    def forward(ctx, num_outputs, *tensors):
        return tuple(t.view_as(t) for t in tensors[:num_outputs])

    @staticmethod
    def backward(ctx, *grads):
        raise RuntimeError(
            "flashback_cute supports derivatives up to second order; "
            "the double-backward results cannot be differentiated again"
        )


class _FlashbackAttnBwdFunc(torch.autograd.Function):
    """(q, k, v, dout) -> (dq, dk, dv). `out` and `lse` enter as constants: the derivatives returned
    by `backward` / `jvp` are total derivatives w.r.t. (q, k, v, dout) that already include the
    dependence through O and LSE (interface.py:294-328)."""

    @staticmethod
    def forward(q, k, v, dout, out, lse, cu_q, cu_k, max_q, max_k, scale, causal):
        g = _Geom(q, k, cu_q, cu_k, max_q, max_k, scale, causal)
        return _backward(g, *map(_rows, (q, k, v, out, dout)), lse)

    @staticmethod
    def setup_context(ctx, inputs, output):
        q, k, v, dout, out, lse, cu_q, cu_k, max_q, max_k, scale, causal = inputs
        ctx.save_for_backward(q, k, v, dout, out, lse, cu_q, cu_k)
        ctx.save_for_forward(q, k, v, dout, out, lse, cu_q, cu_k)
        ctx.geom = (max_q, max_k, scale, causal)

    @staticmethod
    def backward(ctx, gdq, gdk, gdv):
        q, k, v, dout, out, lse, cu_q, cu_k = ctx.saved_tensors
        gdq, gdk, gdv = _zeros_if_none(gdq, q), _zeros_if_none(gdk, k), _zeros_if_none(gdv, v)
        with torch.no_grad():
            g = _Geom(q, k, cu_q, cu_k, *ctx.geom)
            grads = _double_backward(g, q, k, v, out, dout, lse, gdq, gdk, gdv)
        deps = (q, k, v, dout, gdq, gdk, gdv)
        if torch.is_grad_enabled() and any(t.requires_grad for t in deps):
            grads = _NoThirdOrderGrad.apply(len(grads), *grads, *deps)
        return (*grads, *((None,) * 8))

    @staticmethod
    def jvp(ctx, qd, kd, vd, doutd, *_):
        """Forward-over-reverse: directional derivative of (dq, dk, dv) along (qd, kd, vd, doutd)."""
        q, k, v, dout, out, lse, cu_q, cu_k = map(_raw, ctx.saved_tensors)
        qd, kd, vd, doutd = map(_raw, (qd, kd, vd, doutd))
        g = _Geom(q, k, cu_q, cu_k, *ctx.geom)
        qd, kd, vd = _zeros_if_none(qd, q), _zeros_if_none(kd, k), _zeros_if_none(vd, v)
        if g.empty:
            return torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
        q, k, v, out, dout, qd, kd, vd, doutd = map(_rows, (q, k, v, out, dout, qd, kd, vd, doutd))
        _, z1, dpsum, ddot = _jvp_lse_known(g, q, k, v, qd, kd, vd, out, lse, dout, doutd)
        dqd, dkd, dvd = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        _lib.hvp_bwd(g.prob, q, k, v, dout, qd, kd, vd, doutd, lse, dpsum, z1, ddot, None, None, None, dqd, dkd, dvd)
        return dqd, dkd, dvd


class _FlashbackAttnFunc(torch.autograd.Function):
    @staticmethod
    def forward(q, k, v, cu_q, cu_k, max_q, max_k, scale, causal):
        g = _Geom(q, k, cu_q, cu_k, max_q, max_k, scale, causal)
        out, lse = _forward(g, *map(_rows, (q, k, v)))
        return out, lse

    @staticmethod
    def setup_context(ctx, inputs, output):
        q, k, v, cu_q, cu_k, max_q, max_k, scale, causal = inputs
        out, lse = output
        ctx.mark_non_differentiable(lse)
        ctx.save_for_backward(q, k, v, out, lse, cu_q, cu_k)
        ctx.save_for_forward(q, k, v, out, lse, cu_q, cu_k)
        ctx.geom = (max_q, max_k, scale, causal)

    @staticmethod
    def backward(ctx, dout, _dlse):
        q, k, v, out, lse, cu_q, cu_k = ctx.saved_tensors
        dq, dk, dv = _FlashbackAttnBwdFunc.apply(q, k, v, dout, out.detach(), lse.detach(), cu_q, cu_k, *ctx.geom)
        return (dq, dk, dv, *((None,) * 6))

    @staticmethod
    def jvp(ctx, qd, kd, vd, *_):
        """Forward-mode tangent O_dot along (qd, kd, vd); O and LSE are already known."""
        q, k, v, out, lse, cu_q, cu_k = map(_raw, ctx.saved_tensors)
        qd, kd, vd = map(_raw, (qd, kd, vd))
        g = _Geom(q, k, cu_q, cu_k, *ctx.geom)
        qd, kd, vd = _zeros_if_none(qd, q), _zeros_if_none(kd, k), _zeros_if_none(vd, v)
        if g.empty:
            return torch.zeros_like(q), None
        q, k, v, out, qd, kd, vd = map(_rows, (q, k, v, out, qd, kd, vd))
        out_dot, _, _, _ = _jvp_lse_known(g, q, k, v, qd, kd, vd, out, lse)
        return out_dot, None


# torch.autograd.Function.apply binds default arguments of `forward` through inspect.signature() on every
# call when `setup_context` is defined (~30 us per apply, a quarter of a small forward's host time);
# a precomputed __signature__ makes that look-up immediate.
for _fn in (_FlashbackAttnFunc, _FlashbackAttnBwdFunc):
    _fn.forward.__signature__ = inspect.signature(_fn.forward)

_sm_major = {}  # device index -> compute capability major (looked up once per device)


def _validate(q, k, v):
    """Same checks and exception types as the reference (interface.py:362-370), with the
    architecture gate moved to sm_100 and float32 admitted."""
    if not (q.dtype == k.dtype == v.dtype) or q.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise TypeError("q, k, v must share a dtype in {float16, bfloat16, float32}")
    if not (k.shape[-1] == v.shape[-1] == q.shape[-1]) or q.shape[-1] not in (64, 128):
        raise NotImplementedError("head_dim must equal head_dim_v and be 64 or 128")
    if q.shape[-2] % k.shape[-2] != 0:
        raise ValueError("number of q heads must be divisible by number of kv heads")
    if not q.is_cuda:
        raise NotImplementedError("flashback_cute (B200 build) has no CPU path: tensors must be CUDA tensors")
    major = _sm_major.get(q.device.index)
    if major is None:
        major = _sm_major[q.device.index] = torch.cuda.get_device_capability(q.device)[0]
    if major != 10:
        raise NotImplementedError("flashback_cute (B200 build) supports only sm_100 (Blackwell) GPUs")


def flashback_attn_func(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    softmax_scale: Optional[float] = None,
    causal: bool = False,
) -> torch.Tensor:
    """Softmax attention, q (b, sq, hq, d), k/v (b, sk, hkv, d); twice differentiable, and usable
    under forward-mode AD. Causal masking is bottom-right aligned."""
    _validate(q, k, v)
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** -0.5
    return _FlashbackAttnFunc.apply(q, k, v, None, None, None, None, softmax_scale, causal)[0]


def flashback_attn_varlen_func(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    cu_seqlens_k: torch.Tensor,
    max_seqlen_q: int,
    max_seqlen_k: int,
    softmax_scale: Optional[float] = None,
    causal: bool = False,
) -> torch.Tensor:
    """Varlen softmax attention, q (total_q, hq, d), k/v (total_k, hkv, d), cu_seqlens int32 (b+1,)."""
    _validate(q, k, v)
    if cu_seqlens_q.dtype != torch.int32 or cu_seqlens_k.dtype != torch.int32:
        raise TypeError("cu_seqlens_q and cu_seqlens_k must be int32")
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** -0.5
    return _FlashbackAttnFunc.apply(
        q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale, causal
    )[0]


def flashback_attn_jvp(
    q, k, v, q_dot, k_dot, v_dot, softmax_scale: Optional[float] = None, causal: bool = False,
    cu_seqlens_q=None, cu_seqlens_k=None, max_seqlen_q=None, max_seqlen_k=None, return_stats: bool = False,
):
    """Fused JVP forward: returns (O, O_dot) in one kernel pass with online softmax; with
    return_stats also (LSE, z1), both float32 of shape (heads_q, total_q). No autograd graph."""
    _validate(q, k, v)
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** -0.5
    with torch.no_grad():
        g = _Geom(q, k, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale, causal)
        out, lse, out_dot, z1 = _jvp_fused(g, *map(_rows, (q, k, v, q_dot, k_dot, v_dot)))
    return (out, out_dot, lse, z1) if return_stats else (out, out_dot)


def flashback_attn_hvp(
    q, k, v, dout, q_dot, k_dot, v_dot, dout_dot=None, softmax_scale: Optional[float] = None, causal: bool = False,
    cu_seqlens_q=None, cu_seqlens_k=None, max_seqlen_q=None, max_seqlen_k=None, first_order: bool = True,
):
    """JVP forward followed by HVP backward, without autograd: returns
    (O, O_dot, dQ, dK, dV, dQ_dot, dK_dot, dV_dot); the first-order grads are None when
    first_order=False (the reference's double backward only needs the tangents)."""
    _validate(q, k, v)
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** -0.5
    with torch.no_grad():
        g = _Geom(q, k, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale, causal)
        q, k, v, dout, q_dot, k_dot, v_dot, dout_dot = map(_rows, (q, k, v, dout, q_dot, k_dot, v_dot, dout_dot))
        if g.empty:
            z = torch.zeros_like
            return z(q), z(q), z(q), z(k), z(v), z(q), z(k), z(v)
        out, out_dot = torch.empty_like(q), torch.empty_like(q)
        lse, z1, dpsum, ddot = (_stat(q, g.cu_q) for _ in range(4))
        _lib.jvp_fwd(g.prob, q, k, v, q_dot, k_dot, v_dot, out, out_dot, lse, z1, dout, dout_dot, dpsum, ddot)
        mk = (lambda t: torch.empty_like(t)) if first_order else (lambda t: None)
        dq, dk, dv = mk(q), mk(k), mk(v)
        dqd, dkd, dvd = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        _lib.hvp_bwd(g.prob, q, k, v, dout, q_dot, k_dot, v_dot, dout_dot, lse, dpsum, z1, ddot, dq, dk, dv, dqd, dkd, dvd)
    return out, out_dot, dq, dk, dv, dqd, dkd, dvd

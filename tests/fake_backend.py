"""Test double for the C-ABI calls, used by the CPU tests of the host logic only.

It replaces flashback_cute._lib.{jvp_fwd, bwd_row_stats, hvp_bwd} with functions that fill the
same output tensors from the CPU oracle (oracle/attention_oracle.py), so the autograd glue,
the multi-GPU drivers and the error paths can be exercised without a GPU. It lives under
tests/ and is never imported by the package.
"""

from contextlib import contextmanager
from types import SimpleNamespace

import torch

from flashback_cute import _lib, interface
from oracle import attention_oracle as orc


def _problem(q, k, cu_q, cu_k, max_q, max_k, scale, causal, flags=None, segments=()):
    return SimpleNamespace(cu_q=cu_q, cu_k=cu_k, scale=float(scale), causal=bool(causal), flags=flags or 0, segments=tuple(segments))


def _segments(prob, q, k, v, qd, kd, vd, dout, doutd):
    """fb_problem.seg_rows / seg_shift restated with plain bottom-right aligned problems: every query
    segment [lo, hi) against the keys it can see at most (hi + Sk - Sq - shift of them, which aligns its
    last row with the last of those keys); query-side results are concatenated, key-side results added."""
    Sq, Sk = q.shape[1], k.shape[1]
    bounds = [0] + [r for r, _ in prob.segments] + [Sq]
    shifts = [sh for _, sh in prob.segments] + [0]
    cut = lambda t, sl: None if t is None else t[:, sl]
    parts = []
    for lo, hi, sh in zip(bounds[:-1], bounds[1:], shifts):
        rows, keys = slice(lo, hi), slice(0, hi + Sk - Sq - sh)
        parts.append((keys.stop, orc.attention_hvp_dense(cut(q, rows), cut(k, keys), cut(v, keys), prob.scale, True, cut(qd, rows), cut(kd, keys),
                                                         cut(vd, keys), cut(dout, rows), cut(doutd, rows))))
    both = {}
    first = parts[0][1]
    for n in ("out", "out_dot", "dq", "dq_dot"):   # (B, Sq, Hq, D)
        both[n] = None if getattr(first, n) is None else torch.cat([getattr(r, n) for _, r in parts], 1)
    for n in ("lse", "z1"):                        # (B, Hq, Sq)
        both[n] = None if getattr(first, n) is None else torch.cat([getattr(r, n) for _, r in parts], 2)
    for n in ("dk", "dv", "dk_dot", "dv_dot"):     # (B, Sk, Hkv, D)
        both[n] = None
        if getattr(first, n) is not None:
            both[n] = torch.zeros((q.shape[0], Sk) + tuple(getattr(first, n).shape[2:]), dtype=getattr(first, n).dtype)
            for nk, r in parts:
                both[n][:, :nk] += getattr(r, n)
    return orc.HvpResult(**both)


def _run(prob, q, k, v, qd=None, kd=None, vd=None, dout=None, doutd=None):
    if prob.cu_q is None:
        if prob.segments:
            r = _segments(prob, q, k, v, qd, kd, vd, dout, doutd)
        else:
            r = orc.attention_hvp_dense(q, k, v, prob.scale, prob.causal, qd, kd, vd, dout, doutd)
        B, Sq, Hq, _ = q.shape
        fix = lambda s: None if s is None else s.permute(1, 0, 2).reshape(Hq, B * Sq)
        r.lse, r.z1 = fix(r.lse), fix(r.z1)
        return r
    return orc.attention_hvp_varlen(q, k, v, prob.cu_q.tolist(), prob.cu_k.tolist(), prob.scale, prob.causal, qd, kd, vd, dout, doutd)


def _put(dst, src, accumulate=False):
    if dst is not None:
        _lib.raw(dst).data_ptr()  # like the real binding: the tensor underneath must have storage
    if dst is not None and src is not None:
        src = src.to(dst.dtype).reshape(dst.shape)
        if accumulate:
            dst.add_(src)
        else:
            dst.copy_(src)


def _rowdot(a, b):
    # (..., H, D) x (..., H, D) -> (H, rows)
    s = (a.double() * b.double()).sum(-1)
    return s.reshape(-1, s.shape[-1]).t()


def jvp_fwd(prob, q, k, v, qd, kd, vd, out, out_dot, lse, z1, dout=None, dout_dot=None, dpsum=None, ddot=None, lse_known=False):
    r = _run(prob, q, k, v, qd, kd, vd)
    if not lse_known:
        _put(out, r.out)
        _put(lse, r.lse)
    _put(out_dot, r.out_dot)
    _put(z1, r.z1)
    if dout is not None:
        _put(dpsum, _rowdot(dout, r.out))
        if qd is not None:
            dd = _rowdot(dout, r.out_dot)
            if dout_dot is not None:
                dd = dd + _rowdot(dout_dot, r.out)
            _put(ddot, dd)


def bwd_row_stats(prob, out, dout, out_dot, dout_dot, dpsum, ddot):
    _put(dpsum, _rowdot(dout, out))
    if out_dot is not None:
        dd = _rowdot(dout, out_dot)
        if dout_dot is not None:
            dd = dd + _rowdot(dout_dot, out)
        _put(ddot, dd)


def _dkv_from_stats(prob, q, k, v, dout, qd, kd, vd, doutd, lse, dpsum, z1, ddot):
    """dK, dV, dK_dot, dV_dot of the given keys from the formulas of include/flashback_b200.h with the row
    statistics GIVEN (as the kernels compute them), float64; key segments place the keys in the sequence.
    Needed where the keys are a subset: the oracle proper derives its statistics from the keys it is given."""
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    G = Hq // Hkv
    f = lambda t: None if t is None else t.double().permute(0, 2, 1, 3)              # (B, H, S, D)
    fk = lambda t: None if t is None else f(t).repeat_interleave(G, dim=1)
    Q, dO, Qd, dOd = f(q), f(dout), f(qd), f(doutd)
    K, V, Kd, Vd = fk(k), fk(v), fk(kd), fk(vd)
    stat = lambda t: None if t is None else t.double().reshape(Hq, B, Sq).permute(1, 0, 2)[..., None]  # (B, Hq, Sq, 1)
    lse, dpsum, z1, ddot = stat(lse), stat(dpsum), stat(z1), stat(ddot)
    shift = torch.zeros(Sk, dtype=torch.long)
    for brk, sh in reversed(prob.segments):
        shift[:brk] = sh
    i, j = torch.arange(Sq)[:, None], torch.arange(Sk)[None, :]
    vis = j <= i + (Sk - Sq) + shift[None, :]
    c = prob.scale
    P = torch.exp(c * (Q @ K.transpose(-1, -2)) - lse) * vis
    dP = dO @ V.transpose(-1, -2)
    dS = P * (dP - dpsum)
    fold = lambda t: t.reshape(B, Hkv, G, Sk, D).sum(2).permute(0, 2, 1, 3)           # (B, Sk, Hkv, D)
    dk, dv, dkd, dvd = fold(c * (dS.transpose(-1, -2) @ Q)), fold(P.transpose(-1, -2) @ dO), None, None
    if qd is not None:
        Sd = c * (Qd @ K.transpose(-1, -2) + Q @ Kd.transpose(-1, -2))
        Pd = P * (Sd - z1)
        dPd = dO @ Vd.transpose(-1, -2)
        dvd_ = Pd.transpose(-1, -2) @ dO
        if dOd is not None:
            dPd = dPd + dOd @ V.transpose(-1, -2)
            dvd_ = dvd_ + P.transpose(-1, -2) @ dOd
        dSd = Pd * (dP - dpsum) + P * (dPd - ddot)
        dkd = fold(c * (dSd.transpose(-1, -2) @ Q + dS.transpose(-1, -2) @ Qd))
        dvd = fold(dvd_)
    return dk, dv, dkd, dvd


def hvp_bwd(prob, q, k, v, dout, qd, kd, vd, dout_dot, lse, dpsum, z1, ddot, dq, dk, dv, dqd, dkd, dvd):
    if prob.segments and prob.flags & _lib.FB_FLAG_SEG_KEYS:
        assert dq is None and dqd is None
        for dst, src in zip((dk, dv, dkd, dvd), _dkv_from_stats(prob, q, k, v, dout, qd, kd, vd, dout_dot, lse, dpsum, z1, ddot)):
            _put(dst, src)
        return
    r = _run(prob, q, k, v, qd, kd, vd, dout, dout_dot)
    acc = bool(prob.flags & _lib.FB_FLAG_KV_ACCUMULATE)  # dK/dV-side outputs added to what is there
    for dst, src in ((dq, r.dq), (dqd, r.dq_dot)):
        _put(dst, src)
    for dst, src in ((dk, r.dk), (dv, r.dv), (dkd, r.dk_dot), (dvd, r.dv_dot)):
        _put(dst, src, acc)


REAL_VALIDATE = interface._validate


@contextmanager
def installed():
    saved = {n: getattr(_lib, n) for n in ("jvp_fwd", "bwd_row_stats", "hvp_bwd", "problem", "rows_ok")}
    saved_validate = interface._validate
    _lib.jvp_fwd, _lib.bwd_row_stats, _lib.hvp_bwd, _lib.problem = jvp_fwd, bwd_row_stats, hvp_bwd, _problem
    _lib.rows_ok = lambda t: t.data_ptr() >= 0 and t.is_contiguous()  # data_ptr: wrappers without storage must not get here
    interface._validate = lambda q, k, v: None
    try:
        yield
    finally:
        for n, f in saved.items():
            setattr(_lib, n, f)
        interface._validate = saved_validate

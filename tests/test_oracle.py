"""Pins oracle/attention_oracle.py against the golden vectors in tests/golden/, which are
outputs of the reference's own eager oracle (see tests/golden/make_golden.py)."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc

GOLDEN = Path(__file__).resolve().parent / "golden"
DENSE = sorted(GOLDEN.glob("dense_*.npz"))
VARLEN = sorted(GOLDEN.glob("varlen_*.npz"))
TOL = 1e-11  # float64 closed form vs float64 autograd


def _t(z, name):
    return torch.from_numpy(z[name])


def _close(a, b, name):
    err = (a - b).abs().max().item()
    ref = max(b.abs().max().item(), 1.0)
    assert err <= TOL * ref, f"{name}: {err:.3e}"


def _check(z, res_db, res_full):
    # reference double backward: tangents = (gq,gk,gv), dout_dot = 0
    for mine, gold in (("out", "out"), ("dq", "dq"), ("dk", "dk"), ("dv", "dv"), ("dq_dot", "dot_q"),
                       ("dk_dot", "dot_k"), ("dv_dot", "dot_v"), ("out_dot", "dot_dout")):
        _close(getattr(res_db, mine), _t(z, gold), gold)
    _close(res_db.out_dot, _t(z, "out_dot"), "out_dot(jvp)")
    # forward-over-reverse with a non-zero dout tangent
    for mine, gold in (("dq", "hvp_dq"), ("dk", "hvp_dk"), ("dv", "hvp_dv"), ("dq_dot", "hvp_dq_dot"),
                       ("dk_dot", "hvp_dk_dot"), ("dv_dot", "hvp_dv_dot")):
        _close(getattr(res_full, mine), _t(z, gold), gold)


def test_golden_files_present():
    assert len(DENSE) == 5 and len(VARLEN) == 2


@pytest.mark.parametrize("path", DENSE, ids=lambda p: p.stem)
def test_closed_form_matches_reference_dense(path):
    z = np.load(path)
    args = [_t(z, n) for n in ("q", "k", "v")]
    kw = dict(q_dot=_t(z, "q_dot"), k_dot=_t(z, "k_dot"), v_dot=_t(z, "v_dot"), dout=_t(z, "dout"))
    scale, causal = float(z["scale"]), bool(z["causal"])
    res_db = orc.attention_hvp_dense(*args, scale, causal, **kw, row_block=16)
    res_full = orc.attention_hvp_dense(*args, scale, causal, **kw, dout_dot=_t(z, "dout_dot"), row_block=7)
    _check(z, res_db, res_full)


@pytest.mark.parametrize("path", VARLEN, ids=lambda p: p.stem)
def test_closed_form_matches_reference_varlen(path):
    z = np.load(path)
    args = [_t(z, n) for n in ("q", "k", "v")]
    kw = dict(q_dot=_t(z, "q_dot"), k_dot=_t(z, "k_dot"), v_dot=_t(z, "v_dot"), dout=_t(z, "dout"))
    scale, causal = float(z["scale"]), bool(z["causal"])
    cu_q, cu_k = z["cu_q"].tolist(), z["cu_k"].tolist()
    res_db = orc.attention_hvp_varlen(*args, cu_q, cu_k, scale, causal, **kw)
    res_full = orc.attention_hvp_varlen(*args, cu_q, cu_k, scale, causal, **kw, dout_dot=_t(z, "dout_dot"))
    _check(z, res_db, res_full)


@pytest.mark.parametrize("path", DENSE, ids=lambda p: p.stem)
def test_eager_restatement_matches_reference(path):
    """The autograd-based eager restatement (timed as the CPU baseline) gives the same eight
    outputs as the reference's double_backward."""
    z = np.load(path)
    scale, causal = float(z["scale"]), bool(z["causal"])
    leaves = [_t(z, n).clone().requires_grad_() for n in ("q", "k", "v", "dout")]
    fn = lambda q, k, v: orc.eager_attention(q, k, v, causal, scale, True)
    res = orc.eager_double_backward(fn, *leaves, _t(z, "q_dot"), _t(z, "k_dot"), _t(z, "v_dot"))
    for got, name in zip(res, ("out", "dq", "dk", "dv", "dot_q", "dot_k", "dot_v", "dot_dout")):
        _close(got.detach(), _t(z, name), name)


def test_lse_and_fully_masked_rows():
    """Sq > Sk causal: leading rows see no key -> out 0, lse -inf, all their grads 0."""
    z = np.load(GOLDEN / "dense_gqa_causal_sq_gt_sk.npz")
    q, k, v = (_t(z, n) for n in ("q", "k", "v"))
    res = orc.attention_hvp_dense(q, k, v, float(z["scale"]), True)
    n_masked = q.shape[1] - k.shape[1]
    assert torch.all(res.out[:, :n_masked] == 0)
    assert torch.all(torch.isinf(res.lse[:, :, :n_masked]))
    assert torch.all(torch.isfinite(res.lse[:, :, n_masked:]))

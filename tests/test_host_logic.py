"""CPU tests of the host side (autograd glue mirroring flashback_cute/interface.py:275-409):
the double-backward chain, forward-mode rules, third-order guard, empty inputs and argument
validation. Device calls are replaced by tests/fake_backend.py; the parity of the real kernels
is tested in the `gpu`-marked files."""

import itertools

import pytest
import torch

from flashback_cute import flashback_attn_func, flashback_attn_varlen_func, flashback_attn_hvp, flashback_attn_jvp, interface
from oracle import attention_oracle as orc
from tests import fake_backend

NAMES = ("out", "dq", "dk", "dv", "dot_q", "dot_k", "dot_v", "dot_dout")


def _inputs(B=2, Sq=12, Sk=20, Hq=4, Hkv=2, D=8, seed=0):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    return r(B, Sq, Hq, D), r(B, Sk, Hkv, D), r(B, Sk, Hkv, D), r(B, Sq, Hq, D), r(B, Sq, Hq, D), r(B, Sk, Hkv, D), r(B, Sk, Hkv, D)


@pytest.fixture(autouse=True)
def _fake():
    with fake_backend.installed():
        yield


@pytest.mark.parametrize("causal", [False, True])
def test_double_backward_chain_matches_eager(causal):
    q, k, v, dout, gq, gk, gv = _inputs()
    scale = 0.3
    leaves = lambda: [t.clone().requires_grad_() for t in (q, k, v, dout)]
    got = orc.eager_double_backward(lambda a, b, c: flashback_attn_func(a, b, c, scale, causal), *leaves(), gq, gk, gv)
    ref = orc.eager_double_backward(lambda a, b, c: orc.eager_attention(a, b, c, causal, scale, True), *leaves(), gq, gk, gv)
    for n, a, b in zip(NAMES, got, ref):
        assert a.shape == b.shape, n
        assert torch.allclose(a, b, atol=1e-10, rtol=1e-10), n


def test_varlen_double_backward_chain():
    lens_q, lens_k = [5, 9, 1], [7, 9, 3]
    cu_q = torch.tensor([0, *itertools.accumulate(lens_q)], dtype=torch.int32)
    cu_k = torch.tensor([0, *itertools.accumulate(lens_k)], dtype=torch.int32)
    g = torch.Generator().manual_seed(1)
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    q, k, v = r(15, 4, 8), r(19, 2, 8), r(19, 2, 8)
    dout, gq, gk, gv = r(15, 4, 8), r(15, 4, 8), r(19, 2, 8), r(19, 2, 8)
    leaves = lambda: [t.clone().requires_grad_() for t in (q, k, v, dout)]
    fn = lambda a, b, c: flashback_attn_varlen_func(a, b, c, cu_q, cu_k, 9, 9, 0.35, True)
    rf = lambda a, b, c: orc.eager_attention_varlen(a, b, c, cu_q, cu_k, True, 0.35, True)
    got = orc.eager_double_backward(fn, *leaves(), gq, gk, gv)
    ref = orc.eager_double_backward(rf, *leaves(), gq, gk, gv)
    for n, a, b in zip(NAMES, got, ref):
        assert torch.allclose(a, b, atol=1e-10, rtol=1e-10), n


def test_forward_mode_jvp_rule():
    q, k, v, _, gq, gk, gv = _inputs()
    fn = lambda a, b, c: flashback_attn_func(a, b, c, 0.3, True)
    rf = lambda a, b, c: orc.eager_attention(a, b, c, True, 0.3, True)
    out, out_dot = torch.func.jvp(fn, (q, k, v), (gq, gk, gv))
    ro, rd = torch.func.jvp(rf, (q, k, v), (gq, gk, gv))
    assert torch.allclose(out, ro, atol=1e-10) and torch.allclose(out_dot, rd, atol=1e-10)


def test_forward_over_reverse_rule():
    """jvp of the first backward (the HVP path with a non-zero dout tangent)."""
    q, k, v, dout, gq, gk, gv = _inputs()
    g = torch.Generator().manual_seed(9)
    doutd = torch.randn(dout.shape, generator=g, dtype=torch.float64)

    def vjp_of(f):
        def inner(a, b, c, d):
            _, pull = torch.func.vjp(f, a, b, c)
            return pull(d)
        return inner

    fn = lambda a, b, c: flashback_attn_func(a, b, c, 0.3, False)
    rf = lambda a, b, c: orc.eager_attention(a, b, c, False, 0.3, True)
    got_p, got_t = torch.func.jvp(vjp_of(fn), (q, k, v, dout), (gq, gk, gv, doutd))
    ref_p, ref_t = torch.func.jvp(vjp_of(rf), (q, k, v, dout), (gq, gk, gv, doutd))
    for a, b in zip((*got_p, *got_t), (*ref_p, *ref_t)):
        assert torch.allclose(a, b, atol=1e-10, rtol=1e-10)


def test_functional_entry_points():
    q, k, v, dout, gq, gk, gv = _inputs()
    r = orc.attention_hvp_dense(q, k, v, 0.3, True, gq, gk, gv, dout)
    out, out_dot = flashback_attn_jvp(q, k, v, gq, gk, gv, 0.3, True)
    assert torch.allclose(out, r.out) and torch.allclose(out_dot, r.out_dot)
    res = flashback_attn_hvp(q, k, v, dout, gq, gk, gv, None, 0.3, True)
    for a, b in zip(res, (r.out, r.out_dot, r.dq, r.dk, r.dv, r.dq_dot, r.dk_dot, r.dv_dot)):
        assert torch.allclose(a, b, atol=1e-12)
    res = flashback_attn_hvp(q, k, v, dout, gq, gk, gv, None, 0.3, True, first_order=False)
    assert res[2] is None and res[3] is None and res[4] is None


def test_third_order_raises():
    q, k, v, dout, gq, gk, gv = _inputs(B=1, Sq=6, Sk=6)
    ql, kl, vl, dl = [t.clone().requires_grad_() for t in (q, k, v, dout)]
    out = flashback_attn_func(ql, kl, vl, 0.3, False)
    dq, dk, dv = torch.autograd.grad(out, (ql, kl, vl), dl, create_graph=True)
    dots = torch.autograd.grad((dq, dk, dv), (ql, kl, vl, dl), (gq, gk, gv), create_graph=True)
    with pytest.raises(RuntimeError, match="second order"):
        torch.autograd.grad(dots[0].sum(), ql)


def test_empty_inputs_return_zeros():
    q, k, v, dout, gq, gk, gv = _inputs(Sk=0)
    ql, kl, vl, dl = [t.clone().requires_grad_() for t in (q, k, v, dout)]
    res = orc.eager_double_backward(lambda a, b, c: flashback_attn_func(a, b, c, 0.3, False), ql, kl, vl, dl, gq, gk, gv)
    assert all(torch.all(t == 0) for t in res)
    assert res[0].shape == q.shape and res[2].shape == k.shape


def test_non_contiguous_inputs_are_accepted():
    q, k, v, dout, gq, gk, gv = _inputs()
    qt = q.transpose(1, 2).contiguous().transpose(1, 2)  # (B,S,H,D) view with permuted strides
    assert not qt.is_contiguous()
    a = flashback_attn_func(qt, k, v, 0.3, True)
    b = flashback_attn_func(q, k, v, 0.3, True)
    assert torch.equal(a, b)


def test_validate_exceptions_match_reference():
    """Exception classes of flashback_cute/interface.py:362-370, through the real _validate."""
    validate = fake_backend.REAL_VALIDATE
    bf = lambda *s: torch.zeros(*s, dtype=torch.bfloat16)
    with pytest.raises(TypeError):
        validate(bf(1, 4, 2, 64), bf(1, 4, 2, 64).half(), bf(1, 4, 2, 64))
    with pytest.raises(TypeError):
        validate(bf(1, 4, 2, 64).double(), bf(1, 4, 2, 64).double(), bf(1, 4, 2, 64).double())
    with pytest.raises(NotImplementedError):
        validate(bf(1, 4, 2, 96), bf(1, 4, 2, 96), bf(1, 4, 2, 96))
    with pytest.raises(ValueError):
        validate(bf(1, 4, 3, 64), bf(1, 4, 2, 64), bf(1, 4, 2, 64))
    with pytest.raises(NotImplementedError):  # valid shapes but a CPU tensor: there is no CPU path
        validate(bf(1, 4, 2, 64), bf(1, 4, 2, 64), bf(1, 4, 2, 64))


def test_varlen_cu_seqlens_dtype_check():
    q = torch.zeros(4, 2, 8, dtype=torch.float64)
    cu = torch.tensor([0, 4], dtype=torch.int64)
    with pytest.raises(TypeError, match="int32"):
        flashback_attn_varlen_func(q, q, q, cu, cu, 4, 4)

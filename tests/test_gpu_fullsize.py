"""Full-size checks on the three single-GPU benchmark configurations (causal MHA B4 H16 S2048 D128;
causal GQA B2 Hq32 Hkv8 S8192 D128, the bench workload; non-causal MHA B8 H32 S4096 D64; all bf16)
through size-independent properties, plus a sampled comparison against the float64 oracle.

Properties used:
  * scale invariance of attention in (Q, K): <Q, dQ> = <K, dK> per (batch, kv-head group), and its
    derivative along the tangent direction: <Qd,dQ> + <Q,dQd> = <Kd,dK> + <K,dKd>;
  * linearity of the directional derivatives in the tangents;
  * rows of P sum to one: with V = 1, O = 1 and O_dot = 0 whatever Q, K and their tangents are.
"""

import collections

import pytest
import torch

from flashback_cute import _lib, flashback_attn_hvp, flashback_attn_jvp
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu
if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

DEV = "cuda"
Cfg = collections.namedtuple("Cfg", "B HQ HKV S D CAUSAL")
CONFIGS = {
    "causal_mha_s2048_d128": Cfg(4, 16, 16, 2048, 128, True),
    "causal_gqa_s8192_d128": Cfg(2, 32, 8, 8192, 128, True),
    "noncausal_mha_s4096_d64": Cfg(8, 32, 32, 4096, 64, False),
}


@pytest.fixture(scope="module", params=list(CONFIGS), ids=list(CONFIGS))
def problem(request):
    c = CONFIGS[request.param]
    g = torch.Generator(device=DEV).manual_seed(0)
    r = lambda h, std=1.0: (torch.randn(c.B, c.S, h, c.D, generator=g, device=DEV, dtype=torch.float32) * std).to(torch.bfloat16)
    x = dict(q=r(c.HQ), k=r(c.HKV), v=r(c.HKV), qd=r(c.HQ, 0.1), kd=r(c.HKV, 0.1), vd=r(c.HKV, 0.1), do=r(c.HQ), dod=r(c.HQ))
    res = flashback_attn_hvp(x["q"], x["k"], x["v"], x["do"], x["qd"], x["kd"], x["vd"], x["dod"], c.D ** -0.5, c.CAUSAL)
    torch.cuda.synchronize()
    _lib.check_device_status()
    yield c, x, res
    del x, res
    torch.cuda.empty_cache()


def _inner(c, a, b):
    """<a, b> per (batch, kv-head group): q-like tensors fold their G heads into the group."""
    p = (a.double() * b.double()).sum((1, 3))  # (B, H)
    return p.reshape(c.B, c.HKV, -1).sum(-1)


def test_all_outputs_finite(problem):
    _, _, res = problem
    for t in res:
        assert torch.isfinite(t).all()


def test_scale_invariance_identity(problem):
    c, x, (o, od, dq, dk, dv, dqd, dkd, dvd) = problem
    lhs, rhs = _inner(c, x["q"], dq), _inner(c, x["k"], dk)
    mag = (x["q"].double().abs() * dq.double().abs()).sum((1, 3)).reshape(c.B, c.HKV, -1).sum(-1)
    assert ((lhs - rhs).abs() / mag).max().item() < 2e-3
    lhs2 = _inner(c, x["qd"], dq) + _inner(c, x["q"], dqd)
    rhs2 = _inner(c, x["kd"], dk) + _inner(c, x["k"], dkd)
    mag2 = (x["q"].double().abs() * dqd.double().abs()).sum((1, 3)).reshape(c.B, c.HKV, -1).sum(-1)
    assert ((lhs2 - rhs2).abs() / mag2).max().item() < 2e-3


def test_tangent_linearity(problem):
    c, x, res = problem
    res2 = flashback_attn_hvp(x["q"], x["k"], x["v"], x["do"], 2 * x["qd"], 2 * x["kd"], 2 * x["vd"], 2 * x["dod"], c.D ** -0.5, c.CAUSAL, first_order=False)
    for i in (1, 5, 6, 7):
        a, b = res[i].float() * 2, res2[i].float()
        assert (a - b).abs().max().item() <= 2e-2 * b.abs().max().item()


def test_rows_of_p_sum_to_one(problem):
    c, x, _ = problem
    ones = torch.ones_like(x["v"])
    o, od = flashback_attn_jvp(x["q"], x["k"], ones, x["qd"], x["kd"], torch.zeros_like(ones), c.D ** -0.5, c.CAUSAL)
    assert (o.float() - 1).abs().max().item() < 1e-2
    assert od.float().abs().max().item() < 2e-2


RATIO = 2.0  # kernel error may be at most RATIO x the eager same-dtype error, both against float64
NAMES = ("out", "out_dot", "dq", "dk", "dv", "dq_dot", "dk_dot", "dv_dot")


def _gate(name, got, want, eager, where):
    err = (got.double() - want).abs().max().item()
    err_pt = (eager.double() - want).abs().max().item()
    assert err <= RATIO * err_pt, f"{where} {name}: max err {err:.3e} > {RATIO} x eager bf16 err {err_pt:.3e}"


@pytest.mark.parametrize("group", [(0, 0), (-1, -1)], ids=["first_group", "last_group"])
def test_sampled_groups_meet_the_tolerance(problem, group):
    """Two (batch, kv-head) groups with all of their G query heads, all rows, all eight outputs:
    max|kernel - float64| <= 2 x max|eager bf16 - float64|. The float64 side is the closed form,
    evaluated on the GPU 512 query rows at a time; the eager side is forward-over-reverse autograd of
    the eager bf16 attention on the same group (one S x S score matrix per head fits at S = 8192)."""
    c, x, res = problem
    b, hk = group[0] % c.B, group[1] % c.HKV
    G = c.HQ // c.HKV
    qs = slice(hk * G, (hk + 1) * G)
    pick_q = lambda t: t[b:b + 1, :, qs]
    pick_k = lambda t: t[b:b + 1, :, hk:hk + 1]
    scale = c.D ** -0.5
    ref = orc.attention_hvp_dense(
        pick_q(x["q"]), pick_k(x["k"]), pick_k(x["v"]), scale, c.CAUSAL,
        pick_q(x["qd"]), pick_k(x["kd"]), pick_k(x["vd"]), pick_q(x["do"]), pick_q(x["dod"]), row_block=512,
    )
    low = orc.eager_hvp(pick_q(x["q"]), pick_k(x["k"]), pick_k(x["v"]), pick_q(x["do"]), pick_q(x["qd"]), pick_k(x["kd"]),
                        pick_k(x["vd"]), pick_q(x["dod"]), c.CAUSAL, scale, False)
    for n, got, lp in zip(NAMES, res, low):
        want = getattr(ref, n)
        mine = pick_q(got) if want.shape[2] == G else pick_k(got)
        _gate(n, mine, want, lp, f"group {(b, hk)}")
    del low, ref
    torch.cuda.empty_cache()


def test_long_context_properties_s65536():
    """The long-context configuration's sequence length (S = 65536, D = 128, causal), two heads:
    rows of P sum to one, the scale-invariance identity holds, and the last 256 query rows meet the
    tolerance against the float64 closed form evaluated against all 65536 keys: O, O_dot, dQ, dQ_dot
    of those rows, and dK, dV, dK_dot, dV_dot of the last 256 KEYS (under the causal mask no earlier
    query sees them, so the same query chunk determines them completely)."""
    S, H, D = 65536, 2, 128
    g = torch.Generator(device=DEV).manual_seed(3)
    r = lambda std=1.0: (torch.randn(1, S, H, D, generator=g, device=DEV, dtype=torch.float32) * std).to(torch.bfloat16)
    q, k, v, qd, kd, vd, do, dod = r(), r(), r(), r(0.1), r(0.1), r(0.1), r(), r()
    scale = D ** -0.5
    o, od = flashback_attn_jvp(q, k, torch.ones_like(v), qd, kd, torch.zeros_like(v), scale, True)
    assert (o.float() - 1).abs().max().item() < 1e-2 and od.float().abs().max().item() < 2e-2
    res = flashback_attn_hvp(q, k, v, do, qd, kd, vd, dod, scale, True)
    torch.cuda.synchronize()
    _lib.check_device_status()
    for t in res:
        assert torch.isfinite(t).all()
    inner = lambda a, b: (a.double() * b.double()).sum((1, 3))
    lhs, rhs = inner(q, res[2]), inner(k, res[3])
    mag = (q.double().abs() * res[2].double().abs()).sum((1, 3))
    assert ((lhs - rhs).abs() / mag).max().item() < 2e-3
    # a query chunk [a, S) against keys [0, S) is masked exactly as in the full problem because the
    # causal mask is bottom-right aligned
    a = S - 256
    ref = orc.attention_hvp_dense(q[:, a:], k, v, scale, True, qd[:, a:], kd, vd, do[:, a:], dod[:, a:], row_block=64)
    low = orc.eager_hvp(q[:, a:], k, v, do[:, a:], qd[:, a:], kd, vd, dod[:, a:], True, scale, False)
    for n, got, lp in zip(NAMES, res, low):
        want = getattr(ref, n)
        _gate(n, got[:, a:], want[:, a:] if want.shape[1] == S else want, lp[:, a:] if lp.shape[1] == S else lp, "S=65536 tail")


@pytest.mark.parametrize("rank", [0, 5])
def test_long_context_rank_share_equals_the_unsharded_rows(rank):
    """The long-context configuration's sequence length with the 8-GPU partition (S = 65536, D = 128, causal,
    two heads, four zig-zag chunks per rank): what one rank computes is bit for bit the unsharded result
    restricted to its rows - O, O_dot, dQ, dQ_dot of its query chunks run as ONE problem (query segments), and
    dK, dV, dK_dot, dV_dot of the keys of its chunks against all queries (key segments, one CTA per key tile on
    both sides so that the sums are formed in the same order). The unsharded result itself is gated against
    the float64 closed form in test_long_context_properties_s65536."""
    from flashback_cute import parallel as P

    S, H, D, world = 65536, 2, 128, 8
    g = torch.Generator(device=DEV).manual_seed(4)
    r = lambda std=1.0: (torch.randn(1, S, H, D, generator=g, device=DEV, dtype=torch.float32) * std).to(torch.bfloat16)
    q, k, v, qd, kd, vd, do, dod = r(), r(), r(), r(0.1), r(0.1), r(0.1), r(), r()
    scale, N = D ** -0.5, None
    one_cta = _lib.FB_FLAG_DKV_SPLIT(1)

    def step(prob, q_, k_, v_, do_, qd_, kd_, vd_, dod_, st, key_side_only=False):
        out = {n: torch.empty_like(q_) for n in ("out", "out_dot", "dq", "dq_dot")}
        out.update({n: torch.empty_like(k_) for n in ("dk", "dv", "dk_dot", "dv_dot")})
        if not key_side_only:
            _lib.jvp_fwd(prob, q_, k_, v_, qd_, kd_, vd_, out["out"], out["out_dot"], st[0], st[1], do_, dod_, st[2], st[3])
        _lib.hvp_bwd(prob, q_, k_, v_, do_, qd_, kd_, vd_, dod_, st[0], st[2], st[1], st[3],
                     N if key_side_only else out["dq"], out["dk"], out["dv"], N if key_side_only else out["dq_dot"], out["dk_dot"], out["dv_dot"])
        return out

    st_full = [torch.empty(H, S, dtype=torch.float32, device=DEV) for _ in range(4)]  # lse, z1, dpsum, ddot
    full = step(_lib.problem(q, k, N, N, N, N, scale, True, flags=one_cta), q, k, v, do, qd, kd, vd, dod, st_full)
    chunks = P.zigzag_chunks(S, rank, world, 4)
    loc = lambda t: P.zigzag_local(t, chunks).contiguous()
    b1 = chunks[-1][1]
    st_loc = [torch.empty(H, S // world, dtype=torch.float32, device=DEV) for _ in range(4)]
    mine = step(_lib.problem(loc(q), k[:, :b1], N, N, N, N, scale, True, flags=one_cta, segments=P.zigzag_segments(chunks)),
                loc(q), k[:, :b1], v[:, :b1], loc(do), loc(qd), kd[:, :b1], vd[:, :b1], loc(dod), st_loc)
    own = step(_lib.problem(q, loc(k), N, N, N, N, scale, True, flags=one_cta | _lib.FB_FLAG_SEG_KEYS, segments=P.zigzag_key_segments(chunks, S)),
               q, loc(k), loc(v), do, qd, loc(kd), loc(vd), dod, st_full, key_side_only=True)
    torch.cuda.synchronize()
    _lib.check_device_status()
    for n in ("out", "out_dot", "dq", "dq_dot"):
        assert torch.equal(mine[n], P.zigzag_local(full[n], chunks)), n
    for i, n in enumerate(("lse", "z1", "dpsum", "ddot")):
        assert torch.equal(st_loc[i], torch.cat([st_full[i][:, a:b] for a, b in chunks], 1)), n
    for n in ("dk", "dv", "dk_dot", "dv_dot"):
        assert torch.equal(own[n], P.zigzag_local(full[n], chunks)), n


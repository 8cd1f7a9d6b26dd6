"""Generate tests/golden/*.npz from the reference's own eager oracle.

Run in a container where the reference checkout is present:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's tests/reference.py UNMODIFIED (attention_ref,
attention_ref_varlen, double_backward) and records, in float64, for a handful of small
seeded cases: the eight outputs of double_backward (tests/reference.py:57-66), the
forward-mode tangent torch.func.jvp(attention_ref), and the directional derivative of the
VJP (dq, dk, dv) along (q_dot, k_dot, v_dot, dout_dot) computed by torch.func.jvp of the
VJP. Inputs are stored next to the outputs so the fixtures do not depend on the RNG.
The fixtures are what pins oracle/attention_oracle.py; they are small (float64, S <= 44).
"""

import importlib.util
import itertools
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent

# name, B, Sq, Sk, Hq, Hkv, D, causal
DENSE_CASES = [
    ("mha_noncausal", 2, 24, 24, 2, 2, 8, False),
    ("mha_causal", 2, 32, 32, 2, 2, 8, True),
    ("gqa_causal_sq_lt_sk", 1, 19, 41, 6, 2, 8, True),
    ("gqa_causal_sq_gt_sk", 1, 44, 17, 4, 2, 8, True),  # fully masked leading rows
    ("mqa_noncausal_ragged", 1, 21, 35, 4, 1, 16, False),
]
# name, lens_q, lens_k, Hq, Hkv, D, causal
VARLEN_CASES = [
    ("noncausal", [9, 24, 1, 15], [11, 24, 7, 30], 4, 2, 8, False),
    ("causal", [9, 24, 1, 15], [11, 24, 7, 30], 4, 4, 8, True),
]


def load_reference(root: Path):
    spec = importlib.util.spec_from_file_location("flashback_reference_oracle", root / "tests" / "reference.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def hvp_of_vjp(fn, q, k, v, dout, qd, kd, vd, doutd):
    """Directional derivative of (q,k,v,dout) -> VJP(dout) along (qd,kd,vd,doutd)."""

    def vjp_fn(q_, k_, v_, do_):
        _, pull = torch.func.vjp(fn, q_, k_, v_)
        return pull(do_)

    (dq, dk, dv), (dqd, dkd, dvd) = torch.func.jvp(vjp_fn, (q, k, v, dout), (qd, kd, vd, doutd))
    return dq, dk, dv, dqd, dkd, dvd


def record(ref, fn, q, k, v):
    g = torch.Generator().manual_seed(1234)
    rn = lambda t: torch.randn(t.shape, generator=g, dtype=torch.float64)
    dout, gq, gk, gv, doutd = rn(q), rn(q), rn(k), rn(v), rn(q)
    leaves = [t.clone().requires_grad_() for t in (q, k, v, dout)]
    out, dq, dk, dv, dot_q, dot_k, dot_v, dot_dout = ref.double_backward(fn, *leaves, gq, gk, gv)
    _, out_dot = torch.func.jvp(fn, (q, k, v), (gq, gk, gv))
    h = hvp_of_vjp(fn, q, k, v, dout, gq, gk, gv, doutd)
    arrs = dict(
        q=q, k=k, v=v, dout=dout, q_dot=gq, k_dot=gk, v_dot=gv, dout_dot=doutd,
        out=out, dq=dq, dk=dk, dv=dv, dot_q=dot_q, dot_k=dot_k, dot_v=dot_v, dot_dout=dot_dout,
        out_dot=out_dot, hvp_dq=h[0], hvp_dk=h[1], hvp_dv=h[2], hvp_dq_dot=h[3], hvp_dk_dot=h[4], hvp_dv_dot=h[5],
    )
    return {n: t.detach().numpy() for n, t in arrs.items()}


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py /path/to/reference")
    root = Path(sys.argv[1])
    ref = load_reference(root)
    for name, B, Sq, Sk, Hq, Hkv, D, causal in DENSE_CASES:
        g = torch.Generator().manual_seed(0)
        q = torch.randn(B, Sq, Hq, D, generator=g, dtype=torch.float64)
        k = torch.randn(B, Sk, Hkv, D, generator=g, dtype=torch.float64)
        v = torch.randn(B, Sk, Hkv, D, generator=g, dtype=torch.float64)
        scale = D ** -0.5
        fn = lambda q_, k_, v_: ref.attention_ref(q_, k_, v_, causal, scale, True)
        arrs = record(ref, fn, q, k, v)
        np.savez_compressed(HERE / f"dense_{name}.npz", causal=causal, scale=scale, **arrs)
        print("wrote", name)
    for name, lens_q, lens_k, Hq, Hkv, D, causal in VARLEN_CASES:
        g = torch.Generator().manual_seed(0)
        cu_q = torch.tensor([0, *itertools.accumulate(lens_q)], dtype=torch.int32)
        cu_k = torch.tensor([0, *itertools.accumulate(lens_k)], dtype=torch.int32)
        q = torch.randn(sum(lens_q), Hq, D, generator=g, dtype=torch.float64)
        k = torch.randn(sum(lens_k), Hkv, D, generator=g, dtype=torch.float64)
        v = torch.randn(sum(lens_k), Hkv, D, generator=g, dtype=torch.float64)
        scale = D ** -0.5
        fn = lambda q_, k_, v_: ref.attention_ref_varlen(q_, k_, v_, cu_q, cu_k, causal, scale, True)
        arrs = record(ref, fn, q, k, v)
        np.savez_compressed(
            HERE / f"varlen_{name}.npz", causal=causal, scale=scale, cu_q=cu_q.numpy(), cu_k=cu_k.numpy(), **arrs
        )
        print("wrote", name)


if __name__ == "__main__":
    main()

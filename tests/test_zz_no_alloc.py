"""The allocation-free backward entry point (fb_bwd_noalloc) gives the same dq, dk, dv as the
ordinary two-call route (fb_bwd_row_stats + fb_hvp_bwd with a caller-allocated dpsum vector).

Some hosts of this library cannot allocate device memory at call time (a runtime that planned all
of its buffers up front, a latency-critical callback, a C host without a device allocator); for
them the scratch vector lives in a fixed array inside the library. This file is named so that
pytest collects it last: a run that stops at the first failure has then already run every other
test. It calls the entry point twice in a row (the array is shared between calls and keeps the
previous call's contents) on two different problems, and checks the size limit is enforced.
"""

import ctypes

import pytest
import torch

from flashback_cute import _lib, interface as I

pytestmark = pytest.mark.gpu
if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

DEV = "cuda"


def _problem(B, Sq, Sk, Hq, Hkv, D, causal, dtype, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    r = lambda s, h: torch.randn(B, s, h, D, generator=g, device=DEV, dtype=torch.float32).to(dtype)
    q, k, v, dout = r(Sq, Hq), r(Sk, Hkv), r(Sk, Hkv), r(Sq, Hq)
    geom = I._Geom(q, k, None, None, None, None, D ** -0.5, causal)
    out, lse = I._forward(geom, q, k, v)
    return geom, q, k, v, out, dout, lse


def _both_routes(geom, q, k, v, out, dout, lse):
    ref = I._backward(geom, q, k, v, out, dout, lse)  # caller-allocated dpsum, two C calls
    got = tuple(torch.empty_like(t) for t in (q, k, v))
    n0 = _lib.launches()
    _lib.bwd_noalloc(geom.prob, q, k, v, out, dout, lse, *got)
    # the call reports its row-statistics launch together with the backward's kernels (dQ; dK, dV)
    assert _lib.launches() - n0 >= 3
    torch.cuda.synchronize()
    _lib.check_device_status()
    return ref, got


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_noalloc_matches_two_call_route_twice_in_a_row(dtype):
    # Same kernels, same inputs, same summation order: the tolerance of the parity tests would do,
    # and in fact the results are bit-identical.
    first = _problem(2, 200, 264, 4, 2, 128, True, dtype, seed=1)
    second = _problem(1, 384, 384, 8, 8, 64, False, dtype, seed=2)  # different sizes: stale scratch contents must not matter
    for prob in (first, second, first):
        ref, got = _both_routes(*prob)
        for name, a, b in zip(("dq", "dk", "dv"), got, ref):
            assert torch.isfinite(a).all(), name
            assert torch.equal(a, b), f"{name}: max diff {(a.float() - b.float()).abs().max().item():.3e}"


def test_noalloc_rejects_oversized_problems():
    lib = _lib.load()
    limit = _lib.NOALLOC_MAX_STAT_FLOATS
    heads, rows = 32, limit // 32 + 8
    t = _lib.FbTensor(0x1000, heads * 128, 128)
    prob = _lib.FbProblem(0, 1, heads, heads, 128, rows, rows, 0, rows, rows, None, None, 0.1, 0)
    args = _lib.FbBwdNoAllocArgs(prob, t, t, t, t, t, 0x1000, t, t, t)
    assert lib.fb_bwd_noalloc(ctypes.byref(args), None) == -10  # FB_ERR_TOO_LARGE, before any device work
    assert b"maximum" in lib.fb_status_string(-10)

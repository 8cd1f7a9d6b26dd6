"""Autograd-pipeline benchmark in the shape of the reference's bench/bench_double_backward.py:
median ms and peak allocated GB of three pipelines, through the public autograd API, next to a
naive eager attention on the same GPU.

  fwd             out = f(q, k, v)                                   (no autograd tape)
  fwd+bwd         grad(f(q, k, v).sum(), (q, k, v))
  fwd+bwd+bwdbwd  bck = grad(f(q, k, v).sum(), (q, k, v), create_graph=True)
                  grad(sum(t.sum() for t in bck), (q, k, v))

Run from the repo root on a B200:  python flashback-cute_b200/bench_pipelines.py [--causal]
"""

import argparse
import statistics
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))

import torch  # noqa: E402

from flashback_cute import flashback_attn_func  # noqa: E402

PIPELINES = ("fwd", "fwd+bwd", "fwd+bwd+bwdbwd")
DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


def naive_attention(q, k, v, causal, scale):
    """Eager attention with S x S intermediates: matmuls in the input dtype, softmax in float32."""
    s = scale * torch.einsum("bqhd,bkhd->bhqk", q, k).float()
    if causal:
        sq, sk = q.shape[1], k.shape[1]
        row = torch.arange(sq, device=q.device)[:, None]
        col = torch.arange(sk, device=q.device)[None, :]
        s = s.masked_fill(col > row + (sk - sq), float("-inf"))
    return torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1).to(q.dtype), v)


def run_pipeline(name, fn, q, k, v):
    if name == "fwd":
        with torch.no_grad():
            fn(q, k, v)
    elif name == "fwd+bwd":
        torch.autograd.grad(fn(q, k, v).sum(), (q, k, v))
    else:
        bck = torch.autograd.grad(fn(q, k, v).sum(), (q, k, v), create_graph=True)
        torch.autograd.grad(sum(t.sum() for t in bck), (q, k, v))


def measure(name, fn, q, k, v, warmup=3, iters=10):
    """(median ms, peak allocated GB) or None on out-of-memory."""
    try:
        for _ in range(warmup):
            run_pipeline(name, fn, q, k, v)
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        times = []
        for _ in range(iters):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            run_pipeline(name, fn, q, k, v)
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        return statistics.median(times), torch.cuda.max_memory_allocated() / 2**30
    except torch.OutOfMemoryError:
        torch.cuda.empty_cache()
        return None


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--hdim", type=int, nargs="+", default=[64, 128])
    ap.add_argument("--seqlens", type=int, nargs="+", default=[512, 1024, 2048, 4096, 8192])
    ap.add_argument("--dtype", choices=sorted(DTYPES), default="bf16")
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--naive-max-seqlen", type=int, default=4096, help="skip the naive method above this length")
    args = ap.parse_args()
    dtype = DTYPES[args.dtype]
    print(f"batch={args.batch} heads={args.heads} dtype={args.dtype} causal={args.causal} ({torch.cuda.get_device_name()})")
    header = f"{'method':<15}{'hdim':>5}{'seqlen':>7}" + "".join(f"{p + ' ms':>21}{'GB':>7}" for p in PIPELINES)
    print(header)
    print("-" * len(header))
    for hdim in args.hdim:
        scale = hdim ** -0.5
        methods = {
            "flashback_b200": lambda q, k, v: flashback_attn_func(q, k, v, softmax_scale=scale, causal=args.causal),
            "naive": lambda q, k, v: naive_attention(q, k, v, args.causal, scale),
        }
        for method, fn in methods.items():
            for seqlen in args.seqlens:
                if method == "naive" and seqlen > args.naive_max_seqlen:
                    continue
                torch.manual_seed(0)
                q, k, v = [torch.randn(args.batch, seqlen, args.heads, hdim, device="cuda", dtype=dtype, requires_grad=True) for _ in range(3)]
                row = f"{method:<15}{hdim:>5}{seqlen:>7}"
                for pipeline in PIPELINES:
                    res = measure(pipeline, fn, q, k, v)
                    row += f"{'OOM':>21}{'-':>7}" if res is None else f"{res[0]:>21.3f}{res[1]:>7.2f}"
                print(row, flush=True)
                del q, k, v
                torch.cuda.empty_cache()


if __name__ == "__main__":
    main()

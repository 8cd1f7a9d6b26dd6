"""Benchmark of the attention JVP-forward + HVP-backward hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --pipelines [--causal]        autograd pipelines table (fwd / fwd+bwd / fwd+bwd+bwdbwd)

One "step" = one JVP-forward pass (O, LSE, O_dot, row statistics) followed by one HVP-backward
pass (dQ, dK, dV and their directional derivatives from dO and dO_dot) over one batch of
synthetic inputs with the shapes and value distributions of the named workload
(default: causal GQA bf16, B=2, Hq=32, Hkv=8, S=8192, D=128).

N > 1 (default workload): STRONG scaling. The one problem is partitioned by (batch, kv-head) groups,
16 / N groups per GPU, no communication; every rank draws the full tensors from the same seed and
runs the kernels on strided views of its groups. `value` = FLOPs of the whole problem / the slowest
rank's time. The line also carries `weak_replicas` (every rank runs the whole problem, the mode that
cannot lose to imbalance) and `long_context` (the S=65536 workload on the same N GPUs: query blocks
sharded; by default every GPU gathers all query-side rows and computes the complete dK/dV of its own
keys, and under `partial_sum_exchange` the same step with the partial dK/dV summed over NVLink instead;
results checked against the float64 oracle first).

Rank 0 prints ONE JSON line. FLOP accounting: one unit = 2*B*Hq*S^2*D flop (halved when causal)
per S x S x D matmul. `value` counts the matmuls the maths needs (6 for the fused JVP forward,
15 for the HVP backward with dO_dot); `executed_tflops` and `roofline` count the matmuls the
kernels actually execute (the backward recomputes the S-like tiles in its dQ and dK/dV passes).

--impl reference times the CPU eager restatement of the reference's tests/reference.py path
(oracle/attention_oracle.py, forward-mode over reverse-mode autograd) on the host cores, on a
bounded sample of the same workload: one (batch, q-head) slice at the workload's sequence length.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "flashback-cute_b200"))

import torch  # noqa: E402

WORKLOADS = {
    # name: (B, Hq, Hkv, S, D, causal)
    "causal_gqa_s8192_d128": (2, 32, 8, 8192, 128, True),
    "causal_mha_s2048_d128": (4, 16, 16, 2048, 128, True),
    "noncausal_mha_s4096_d64": (8, 32, 32, 4096, 64, False),
    # long context: query blocks sharded across the GPUs, NCCL reduce-scatter of partial dK/dV (strong scaling)
    "long_causal_s65536_d128": (1, 16, 16, 65536, 128, True),
}
LONG = "long_causal_s65536_d128"
DEFAULT_WORKLOAD = "causal_gqa_s8192_d128"
UNITS_JVP, UNITS_HVP = 6, 15                      # matmuls the maths needs per step
EXEC_UNITS = {"jvp_fwd": 6, "hvp_dq": 9, "hvp_dkv_first": 4, "hvp_dkv_dot": 10}  # matmuls executed per kernel
METRIC = "JVP-fwd + HVP-bwd TFLOP/s (useful matmuls)"


def unit_flops(B, Hq, S, D, causal):
    f = 2.0 * B * Hq * S * S * D
    return f / 2 if causal else f


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(burst=d["bf16_tflops"], sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]), hbm=d["hbm_gbs"], src="measured")
    return dict(burst=1590.0, sustained=1400.0, hbm=6650.0, src="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi. The process is started early (it takes a
    few hundred ms to produce its first line) and only the samples taken inside the window marked by
    begin() / stop() are kept; the window is the warm-up plus the timed region, which run the same load
    back to back (on 8 GPUs the timed region alone lasts tens of ms, less than one sampling period)."""

    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.index, self.rows, self.proc, self.t_begin = index, [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.monotonic(), [x.strip() for x in line.split(",")]))

    def begin(self):
        self.t_begin = time.monotonic()

    def stop(self):
        if self.proc is None:
            return None
        t_end = time.monotonic()
        time.sleep(0.05)  # let the reader thread take in the last lines
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        ok = [(t, r) for t, r in self.rows if len(r) == 6 and r[0].isdigit()]
        rows = [r for t, r in ok if (self.t_begin or 0) <= t <= t_end + 0.03]
        if not rows:
            return None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in rows for n, v in zip(names, r[2:]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(int(r[0]) for r in rows), "sm_max_mhz": int(rows[0][1]), "reasons": reasons, "samples": len(rows),
                "window": "warm-up + timed region"}


def make_inputs(shape, device, seed, dtype=torch.bfloat16):
    """Q,K,V ~ N(0,1); tangents ~ N(0, 0.1^2); dO, dO_dot ~ N(0,1); drawn in this fixed order."""
    B, Hq, Hkv, S, D, _ = shape
    g = torch.Generator(device=device).manual_seed(seed)
    def rn(h, std=1.0):
        return (torch.randn(B, S, h, D, generator=g, device=device, dtype=torch.float32) * std).to(dtype)
    return dict(q=rn(Hq), k=rn(Hkv), v=rn(Hkv), q_dot=rn(Hq, 0.1), k_dot=rn(Hkv, 0.1), v_dot=rn(Hkv, 0.1), dout=rn(Hq), dout_dot=rn(Hq))


# ------------------------------------------------------------------------------------------------
# reference arm / CPU baseline: eager forward-over-reverse on the host cores
# ------------------------------------------------------------------------------------------------
def cpu_step(shape, sample):
    """One (batch, q-head) slice of the workload through the eager CPU restatement."""
    from oracle import attention_oracle as orc

    _, _, _, _, D, causal = shape
    t0 = time.perf_counter()
    orc.eager_hvp(sample["q"], sample["k"], sample["v"], sample["dout"], sample["q_dot"], sample["k_dot"], sample["v_dot"],
                  sample["dout_dot"], causal, D ** -0.5, False)
    return time.perf_counter() - t0


def use_all_host_threads():
    """torchrun exports OMP_NUM_THREADS=1; the CPU legs should use every core this process may run on."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def cpu_sample(shape, seed=0):
    B, Hq, Hkv, S, D, causal = shape
    return make_inputs((1, 1, 1, S, D, causal), "cpu", seed, dtype=torch.float32)


def run_reference(args, shape, rank):
    if rank != 0:
        return
    B, Hq, Hkv, S, D, causal = shape
    use_all_host_threads()
    sample = cpu_sample(shape)
    small = cpu_sample((1, 1, 1, 256, D, causal))
    cpu_step(shape, small)
    for _ in range(args.warmup):
        cpu_step(shape, sample)
    times = [cpu_step(shape, sample) for _ in range(args.steps)]
    ms = 1e3 * sum(times) / len(times)
    flops = (UNITS_JVP + UNITS_HVP) * unit_flops(1, 1, S, D, causal)
    val = flops / (ms * 1e-3) / 1e12
    cores = torch.get_num_threads()
    desc = f"1 (batch, q-head) slice of {args.workload} at S={S}, float32, eager forward-over-reverse (oracle port of tests/reference.py)"
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "B": B, "Hq": Hq, "Hkv": Hkv, "S": S, "D": D, "causal": causal},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
class Step:
    """The four kernel calls of one step on a (view of a) problem, with caller-owned outputs."""

    def __init__(self, x, scale, causal):
        from flashback_cute import _lib, interface as I

        self.lib, self.x = _lib, x
        q, k = x["q"], x["k"]
        self.prob = _lib.problem(q, k, None, None, None, None, scale, causal)
        shp_q, shp_k = q.shape, k.shape
        mk = lambda shp: torch.empty(shp, dtype=q.dtype, device=q.device)
        self.out, self.out_dot, self.dq, self.dqd = (mk(shp_q) for _ in range(4))
        self.dk, self.dv, self.dkd, self.dvd = (mk(shp_k) for _ in range(4))
        self.lse, self.z1, self.dpsum, self.ddot = (torch.empty(shp_q[2], shp_q[0] * shp_q[1], dtype=torch.float32, device=q.device) for _ in range(4))
        D = q.shape[-1]
        names = ["jvp_fwd", "hvp_dq"] + (["hvp_dkv_all"] if D == 64 else ["hvp_dkv_first", "hvp_dkv_dot"])
        self.kernels = [(n, getattr(self, "k_" + n)) for n in names]
        # head_dim 64: dK, dV and their tangents come out of one launch (6 S-like + 6 output GEMMs)
        self.exec_units = {"jvp_fwd": 6, "hvp_dq": 9, "hvp_dkv_all": 12} if D == 64 else dict(EXEC_UNITS)

    def _bwd(self, *outs):
        x = self.x
        self.lib.hvp_bwd(self.prob, x["q"], x["k"], x["v"], x["dout"], x["q_dot"], x["k_dot"], x["v_dot"], x["dout_dot"],
                         self.lse, self.dpsum, self.z1, self.ddot, *outs)

    def k_jvp_fwd(self):
        x = self.x
        self.lib.jvp_fwd(self.prob, x["q"], x["k"], x["v"], x["q_dot"], x["k_dot"], x["v_dot"], self.out, self.out_dot, self.lse, self.z1,
                         x["dout"], x["dout_dot"], self.dpsum, self.ddot)

    def k_hvp_dq(self):
        self._bwd(self.dq, None, None, self.dqd, None, None)

    def k_hvp_dkv_first(self):
        self._bwd(None, self.dk, self.dv, None, None, None)

    def k_hvp_dkv_dot(self):
        self._bwd(None, None, None, None, self.dkd, self.dvd)

    def k_hvp_dkv_all(self):
        self._bwd(None, self.dk, self.dv, None, self.dkd, self.dvd)

    def run(self, events=None):
        for i, (_, fn) in enumerate(self.kernels):
            if events is not None:
                events[i].record()
            fn()
        if events is not None:
            events[len(self.kernels)].record()


def timed_steps(step: Step, steps: int, barrier):
    """(total ms of `steps` steps, mean ms per kernel) with CUDA events on the launching stream."""
    n = len(step.kernels)
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(n + 1)] for _ in range(steps)]
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record()
    for s in range(steps):
        step.run(evs[s])
    t1.record()
    barrier()
    kern = {name: sum(e[i].elapsed_time(e[i + 1]) for e in evs) / steps for i, (name, _) in enumerate(step.kernels)}
    return t0.elapsed_time(t1), kern


def run_kernels_only(args, shape):
    """--kernels-only: warm-up + K steps of the four kernel calls on one GPU and their mean times, nothing
    else (no copies, no CPU leg). The command `ncu` captures are taken from; --shape picks a reduced case."""
    from flashback_cute import _lib

    B, Hq, Hkv, S, D, causal = shape
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[args.dtype]  # fp32: the CUDA-core kernels
    step = Step(make_inputs(shape, dev, seed=0, dtype=dtype), D ** -0.5, causal)
    for _ in range(args.warmup):
        step.run()
    total_ms, kern_ms = timed_steps(step, args.steps, torch.cuda.synchronize)
    _lib.check_device_status()
    F = unit_flops(B, Hq, S, D, causal)
    print(json.dumps({"shape": dict(B=B, Hq=Hq, Hkv=Hkv, S=S, D=D, causal=causal), "dtype": args.dtype, "steps": args.steps,
                      "ms_per_step": total_ms / args.steps, "flags": _lib.DEFAULT_FLAGS,
                      "kernels": {n: {"ms": round(ms, 4), "executed_units": step.exec_units[n],
                                      "tflops": round(step.exec_units[n] * F / (ms * 1e-3) / 1e12, 1)} for n, ms in kern_ms.items()},
                      "useful_tflops": (UNITS_JVP + UNITS_HVP) * F / (total_ms / args.steps * 1e-3) / 1e12}), flush=True)


def run_rank_share(args, shape):
    """--rank-share R/N (long-context workload, ONE GPU): the kernels rank R of an N-rank job runs in a step,
    each timed in steady state (>= 0.3 s of the same kernel first), against the unsharded kernels / N. Query side:
    the rank's zig-zag chunks as one problem (query segments). Key side, both ways: partial sums over the keys the
    rank's queries see (float32 outputs, head groups of a quarter) and key ownership (the keys of the rank's own
    chunks against all query rows, key segments). No communication: what the numbers leave out is the exchange."""
    from flashback_cute import _lib, parallel as P

    B, Hq, Hkv, S, D, causal = shape
    R, N = (int(t) for t in args.rank_share.split("/"))
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    x = make_inputs(shape, dev, seed=0)
    scale, NONE, G = D ** -0.5, None, Hq // Hkv

    def steady(fn, n):
        t0 = time.monotonic()
        while time.monotonic() - t0 < 0.3:
            fn()
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    def kernels(q, k, v, do, qd, kd, vd, dod, st, flags, segments, n, kv_dtype=None, hg=None):
        """ms of JVP-fwd, dQ, first-order dK/dV, tangent dK/dV (the last two over head groups of hg)."""
        prob = _lib.problem(q, k, NONE, NONE, NONE, NONE, scale, True, flags=flags, segments=segments)
        out = {m: torch.empty_like(q) for m in ("o", "od", "dq", "dqd")}
        hg = hg or Hkv
        kout = {m: torch.empty((1, k.shape[1], hg, D), dtype=kv_dtype or k.dtype, device=dev) for m in ("dk", "dv", "dkd", "dvd")}
        res = {}
        if not (flags & _lib.FB_FLAG_SEG_KEYS):
            res["jvp_fwd"] = steady(lambda: _lib.jvp_fwd(prob, q, k, v, qd, kd, vd, out["o"], out["od"], st[0], st[1], do, dod, st[2], st[3]), n)
            res["hvp_dq"] = steady(lambda: _lib.hvp_bwd(prob, q, k, v, do, qd, kd, vd, dod, st[0], st[2], st[1], st[3], out["dq"], NONE, NONE, out["dqd"], NONE, NONE), n)

        def dkv(tangents):
            for h0 in range(0, Hkv, hg):
                hk, hq = slice(h0, h0 + hg), slice(h0 * G, (h0 + hg) * G)
                kf = flags | (_lib.FB_FLAG_KV_OUT_F32 if kv_dtype == torch.float32 else 0)
                pk = _lib.problem(q[:, :, hq], k[:, :, hk], NONE, NONE, NONE, NONE, scale, True, flags=kf, segments=segments)
                a = (q[:, :, hq], k[:, :, hk], v[:, :, hk], do[:, :, hq], qd[:, :, hq], kd[:, :, hk], vd[:, :, hk], dod[:, :, hq],
                     st[0][hq], st[2][hq], st[1][hq], st[3][hq])
                if tangents:
                    _lib.hvp_bwd(pk, *a, NONE, NONE, NONE, NONE, kout["dkd"], kout["dvd"])
                else:
                    _lib.hvp_bwd(pk, *a, NONE, kout["dk"], kout["dv"], NONE, NONE, NONE)
        res["hvp_dkv_first"] = steady(lambda: dkv(False), n)
        res["hvp_dkv_dot"] = steady(lambda: dkv(True), n)
        return res

    full = (x["q"], x["k"], x["v"], x["dout"], x["q_dot"], x["k_dot"], x["v_dot"], x["dout_dot"])
    st_full = [torch.empty(Hq, S, dtype=torch.float32, device=dev) for _ in range(4)]  # lse, z1, dpsum, ddot of all rows
    whole = kernels(*full, st_full, 0, (), 3)
    per = P.default_chunks_per_rank(S, N)
    chunks = P.zigzag_chunks(S, R, N, per)
    b1 = chunks[-1][1]
    loc = lambda t: P.zigzag_local(t, chunks).contiguous()
    ql, dol, qdl, dodl = loc(x["q"]), loc(x["dout"]), loc(x["q_dot"]), loc(x["dout_dot"])
    seen = [t[:, :b1] for t in (x["k"], x["v"], x["k_dot"], x["v_dot"])]
    st_loc = [torch.empty(Hq, S // N, dtype=torch.float32, device=dev) for _ in range(4)]
    hg = max(1, Hkv // 4)
    sums = kernels(ql, seen[0], seen[1], dol, qdl, seen[2], seen[3], dodl, st_loc, 0, P.zigzag_segments(chunks), 10, torch.float32, hg)
    own = [loc(t) for t in (x["k"], x["v"], x["k_dot"], x["v_dot"])]
    owner = kernels(x["q"], own[0], own[1], x["dout"], x["q_dot"], own[2], own[3], x["dout_dot"], st_full, _lib.FB_FLAG_SEG_KEYS,
                    P.zigzag_key_segments(chunks, S), 10)
    _lib.check_device_status()
    r3 = lambda d: {n: round(v, 3) for n, v in d.items()}
    q_side = sums["jvp_fwd"] + sums["hvp_dq"]
    print(json.dumps({
        "workload": LONG, "rank": R, "ranks": N, "query_chunks": chunks,
        "unsharded_ms_over_ranks": r3({n: v / N for n, v in whole.items()}), "unsharded_sum_ms_over_ranks": round(sum(whole.values()) / N, 3),
        "query_side_ms": r3({n: sums[n] for n in ("jvp_fwd", "hvp_dq")}),
        "key_side_partial_sums_ms": r3({n: sums[n] for n in ("hvp_dkv_first", "hvp_dkv_dot")}),
        "key_side_own_keys_ms": r3(owner),
        "step_partial_sums_ms": round(q_side + sums["hvp_dkv_first"] + sums["hvp_dkv_dot"], 3),
        "step_own_keys_ms": round(q_side + sum(owner.values()), 3),
    }), flush=True)


def run_ours(args, shape, rank, world, local_rank):
    import torch.distributed as dist
    from flashback_cute import _lib, flashback_attn_hvp, parallel

    B, Hq, Hkv, S, D, causal = shape
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    scale = D ** -0.5

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(vals):
        t = torch.tensor(vals, device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    # Strong scaling: the same full tensors on every rank (same seed), this rank's (batch, kv-head) groups as views.
    full = make_inputs(shape, dev, seed=0)
    bs, hs = parallel.group_slices(B, Hkv, rank, world)
    mine = {n: parallel.shard_by_group(t, bs, hs, Hkv) for n, t in full.items()}
    Bs, Hq_s, Hkv_s = mine["q"].shape[0], mine["q"].shape[2], mine["k"].shape[2]
    step = Step(mine, scale, causal)

    step.run()  # first call: one-time set-up in the library
    barrier()
    if sampler:
        sampler.begin()
    # warm-up: at least 3 steps, and at least ~0.3 s of the same load so that clocks and the clock samples settle
    t_w = time.monotonic()
    n_w = 0
    while n_w < max(args.warmup, 3) or time.monotonic() - t_w < 0.3:
        step.run()
        n_w += 1
        if n_w % 8 == 0:
            torch.cuda.synchronize()
    barrier()
    _lib.check_device_status()
    launches0 = _lib.launches()
    total_ms, kern_ms = timed_steps(step, args.steps, barrier)
    clocks = sampler.stop() if sampler else None
    launches = _lib.launches() - launches0
    _lib.check_device_status()

    # The reference's own double backward (K1 + K2: O and LSE known, tangents only, dO_dot = 0), timed
    # separately for information: 5 + 10 matmul units needed, 5 + 15 executed. This rank's share.
    x = mine

    def k1():
        _lib.jvp_fwd(step.prob, x["q"], x["k"], x["v"], x["q_dot"], x["k_dot"], x["v_dot"], step.out, step.out_dot, step.lse, step.z1,
                     x["dout"], None, step.dpsum, step.ddot, lse_known=True)

    def k2():
        _lib.hvp_bwd(step.prob, x["q"], x["k"], x["v"], x["dout"], x["q_dot"], x["k_dot"], x["v_dot"], None, step.lse, step.dpsum, step.z1,
                     step.ddot, None, None, None, step.dqd, step.dkd, step.dvd)

    _lib.jvp_fwd(step.prob, x["q"], x["k"], x["v"], None, None, None, step.out, None, step.lse, None)  # O, LSE for K1
    for _ in range(2):
        k1(); k2()
    db_ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    db_k1 = db_k2 = 0.0
    db_steps = 5
    for _ in range(db_steps):
        db_ev[0].record(); k1(); db_ev[1].record(); k2(); db_ev[2].record()
        torch.cuda.synchronize()
        db_k1 += db_ev[0].elapsed_time(db_ev[1]) / db_steps
        db_k2 += db_ev[1].elapsed_time(db_ev[2]) / db_steps

    # End to end through the public API with HOST buffers: every step copies this rank's eight input
    # shards from pinned host memory and its eight results back. The three legs of consecutive steps
    # overlap on three streams (copy-in of step i+1 and copy-out of step i-1 run under the kernels of
    # step i), with two device input sets; each step's copies are inside the timed region.
    host = {n: t.contiguous().cpu().pin_memory() for n, t in mine.items()}
    dev_in = [{n: torch.empty(t.shape, dtype=t.dtype, device=dev) for n, t in host.items()} for _ in range(2)]
    host_out = None
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    s_comp = torch.cuda.current_stream(dev)
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_free = [torch.cuda.Event() for _ in range(2)]
    e2e_i = 0

    def e2e_step():
        nonlocal host_out, e2e_i
        j = e2e_i % 2
        d = dev_in[j]
        with torch.cuda.stream(s_in):
            if e2e_i >= 2:
                s_in.wait_event(ev_free[j])  # the kernels that read this input set two steps ago are done
            for n, t in host.items():
                d[n].copy_(t, non_blocking=True)
            ev_in[j].record(s_in)
        s_comp.wait_event(ev_in[j])
        res = flashback_attn_hvp(d["q"], d["k"], d["v"], d["dout"], d["q_dot"], d["k_dot"], d["v_dot"], d["dout_dot"], scale, causal)
        ev_free[j].record(s_comp)
        if host_out is None:
            host_out = [torch.empty(r.shape, dtype=r.dtype, pin_memory=True) for r in res]
        done = torch.cuda.Event()
        done.record(s_comp)
        with torch.cuda.stream(s_out):
            s_out.wait_event(done)
            for h, r in zip(host_out, res):
                r.record_stream(s_out)
                h.copy_(r, non_blocking=True)
        e2e_i += 1

    e2e_steps = max(4, args.steps)  # the pipeline's fill and drain (one copy-in, one copy-out) are inside the timed region
    for _ in range(3):
        e2e_step()
    s_comp.wait_stream(s_out)
    barrier()
    # three repeats of the timed loop; the median repeat is reported (host-side copies on a shared
    # machine are noisy) and all three are listed
    e2e_repeats = []
    for _ in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(e2e_steps):
            e2e_step()
        s_comp.wait_stream(s_in)
        s_comp.wait_stream(s_out)
        e1.record()
        barrier()
        e2e_repeats.append(e0.elapsed_time(e1) / e2e_steps)
    e2e_repeats = [max_over_ranks([r])[0] for r in e2e_repeats]
    e2e_ms = sorted(e2e_repeats)[1]
    h2d = sum(t.numel() * t.element_size() for t in host.values())
    d2h = sum(t.numel() * t.element_size() for t in host_out)
    del host, dev_in, host_out
    torch.cuda.empty_cache()

    # Secondary, N > 1 only: weak scaling of replicas (every rank runs the WHOLE problem).
    weak = None
    if world > 1:
        rep = Step(full, scale, causal)
        for _ in range(3):
            rep.run()
        w_steps = max(5, args.steps // 2)
        w_ms, _ = timed_steps(rep, w_steps, barrier)
        w_ms = max_over_ranks([w_ms])[0] / w_steps
        weak = {"note": "every rank runs the whole problem (no partition): aggregate over the N replicas", "ms_per_step": w_ms,
                "value": world * (UNITS_JVP + UNITS_HVP) * unit_flops(B, Hq, S, D, causal) / (w_ms * 1e-3) / 1e12, "unit": "TFLOP/s"}
        del rep
    del step, full, mine
    torch.cuda.empty_cache()

    # Secondary, N > 1 only: the long-context workload on the same GPUs (query-block sharding + reduce-scatter).
    long_ctx = None
    if world > 1 and not args.no_long:
        long_ctx = long_context_run(WORKLOADS[LONG], rank, world, dev, steps=3, warmup=2, check=True, exchange=args.exchange)
        if args.exchange is None:  # ... and the same step with the partial sums reduce-scattered over NVLink (copy-engine exchange)
            long_ctx["partial_sum_exchange"] = long_context_run(WORKLOADS[LONG], rank, world, dev, steps=3, warmup=2, check=True, exchange="copy")

    # max over ranks
    stats = max_over_ranks([total_ms, *kern_ms.values(), db_k1, db_k2])
    total_ms = stats[0]
    kern_ms = {n: stats[1 + i] for i, n in enumerate(kern_ms)}
    db_k1, db_k2 = stats[-2], stats[-1]
    if rank != 0:
        return

    F = unit_flops(B, Hq, S, D, causal)   # one matmul unit of the WHOLE problem
    Fr = F / world                        # ... of one rank's share
    ms_per_step = total_ms / args.steps
    exec_units = {"jvp_fwd": 6, "hvp_dq": 9, "hvp_dkv_all": 12} if D == 64 else dict(EXEC_UNITS)
    useful = (UNITS_JVP + UNITS_HVP) * F
    executed = sum(exec_units.values()) * F
    value = useful / (ms_per_step * 1e-3) / 1e12
    pk = peaks()
    per_kernel = {}
    for n, ms in kern_ms.items():
        tf = exec_units[n] * Fr / (ms * 1e-3) / 1e12  # per GPU
        per_kernel[n] = {"ms": round(ms, 4), "executed_units": exec_units[n], "tflops_per_gpu": round(tf, 1),
                         "frac_of_burst_peak": round(tf / pk["burst"], 4), "frac_of_sustained_peak": round(tf / pk["sustained"], 4),
                         "frac_of_nominal_2250": round(tf / 2250.0, 4)}
    dom = max(kern_ms, key=kern_ms.get)
    dom_tf = per_kernel[dom]["tflops_per_gpu"]
    hvp_ms = sum(ms for n, ms in kern_ms.items() if n.startswith("hvp_"))
    hvp_exec = sum(u for n, u in exec_units.items() if n.startswith("hvp_"))
    traffic_file = ROOT / "profiles" / "dram_traffic.json"
    traffic = None
    if traffic_file.exists() and world == 1:
        traffic = json.loads(traffic_file.read_text()).get(args.workload, {}).get(dom)

    # CPU baseline: bounded sample on this box's host cores
    use_all_host_threads()
    sample = cpu_sample(shape)
    cpu_step(shape, cpu_sample((1, 1, 1, 256, D, causal)))
    cpu_s = cpu_step(shape, sample)
    cpu_val = (UNITS_JVP + UNITS_HVP) * unit_flops(1, 1, S, D, causal) / cpu_s / 1e12

    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload, "B": B, "Hq": Hq, "Hkv": Hkv, "S": S, "D": D, "causal": causal,
                   "mode": "fused JVP-fwd (O, LSE, O_dot, stats) + HVP-bwd (dQ,dK,dV + directional derivatives, dO_dot given)",
                   "sharding": f"(batch, kv-head) partition of the one problem: {B * Hkv // world} of {B * Hkv} groups per GPU "
                               f"(per-GPU view B={Bs} Hq={Hq_s} Hkv={Hkv_s}), no communication",
                   "l2": "inputs+outputs of the problem > 1 GB per step (> 126 MB L2 on every rank at every N <= 8)",
                   "useful_units": UNITS_JVP + UNITS_HVP, "executed_units": sum(exec_units.values()), "warmup_steps_run": n_w},
        "executed_tflops": executed / (ms_per_step * 1e-3) / 1e12,
        "jvp_fwd": {"ms": kern_ms["jvp_fwd"], "tflops_executed_per_gpu": per_kernel["jvp_fwd"]["tflops_per_gpu"],
                    "frac_of_burst_peak": per_kernel["jvp_fwd"]["frac_of_burst_peak"]},
        "hvp_bwd": {"ms": hvp_ms, "tflops_useful_per_gpu": UNITS_HVP * Fr / (hvp_ms * 1e-3) / 1e12,
                    "tflops_executed_per_gpu": hvp_exec * Fr / (hvp_ms * 1e-3) / 1e12,
                    "frac_of_burst_peak_useful": UNITS_HVP * Fr / (hvp_ms * 1e-3) / 1e12 / pk["burst"],
                    "frac_of_burst_peak_executed": hvp_exec * Fr / (hvp_ms * 1e-3) / 1e12 / pk["burst"]},
        "kernels": per_kernel,
        "double_backward": {"note": "the reference's K1 + K2 step (LSE known, tangents only, dO_dot = 0), slowest rank's share",
                            "k1_ms": db_k1, "k2_ms": db_k2, "useful_units": 15, "executed_units": 20,
                            "tflops_useful_per_gpu": 15 * Fr / ((db_k1 + db_k2) * 1e-3) / 1e12,
                            "k1_tflops_per_gpu": 5 * Fr / (db_k1 * 1e-3) / 1e12, "k2_tflops_executed_per_gpu": 15 * Fr / (db_k2 * 1e-3) / 1e12},
        "roofline": {"bound": "tensor", "kernel": dom, "achieved": dom_tf, "peak": pk["burst"], "unit": "TFLOP/s",
                     "frac": round(dom_tf / pk["burst"], 4), "traffic": traffic, "peak_source": pk["src"] + " (burst bf16 GEMM)",
                     "peak_sustained": pk["sustained"], "frac_of_sustained": round(dom_tf / pk["sustained"], 4)},
        "cpu_baseline": {"value": cpu_val, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"1 (batch, q-head) slice at S={S}, float32, eager forward-over-reverse, {cpu_s:.1f} s"},
        "e2e": {"value": useful / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms, "ms_per_step_repeats": e2e_repeats,
                "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world,
                "note": "bytes are the whole job's (every rank copies its own share); host copies are PCIe-bound, not kernel-bound"},
        "gpu_launches": launches,
        "clocks": clocks,
    }
    if weak is not None:
        line["weak_replicas"] = weak
    if long_ctx is not None:
        line["long_context"] = long_ctx
    print(json.dumps(line), flush=True)


COLLECTIVE = {
    "none": "one rank: nothing to exchange",
    "copy": "device-to-device copies (copy engines, side stream) of every head group's float32 key blocks into the owner rank's "
            "symmetric-memory slots over NVLink, overlapped with the next group's kernels, then a stream barrier and a local sum of the "
            "received slots (fb_sum_slots)",
    "peer": "fused into the dK/dV kernels: float32 key tiles stored into the owner rank's symmetric-memory slots over NVLink as they "
            "complete, then a stream barrier and a local sum of the received slots (fb_hvp_bwd_scatter + fb_sum_slots)",
    "nccl": "NCCL reduce-scatter (sum, float32) of partial dK, dV, dK_dot, dV_dot along the key axis on a side stream",
    "gather": "no partial sums: every rank's 16-bit q, dO, q_dot, dO_dot rows go to every peer (copy engines over NVLink, under the "
              "query-side kernels), the four row statistics by an all-gather at the phase boundary, and every rank computes the "
              "complete dK, dV, dK_dot, dV_dot of the keys of its own chunks (key segments)",
}


def long_context_check(x, res, rank, world, scale):
    """Compares this rank's results for ONE head with the float64 oracle, evaluated on this GPU: its
    query chunks (O, O_dot, dQ, dQ_dot) and the key rows it ends up with (dK, dV, dK_dot, dV_dot). Returns the
    largest error relative to the largest reference value, per output."""
    from oracle import attention_oracle as orc

    assert x["q"].shape[2] == x["k"].shape[2], "one-head check: the long-context workload has heads_q == heads_kv"
    h = x["q"].shape[2] - 1  # the last head
    pick = lambda t: t[:, :, h:h + 1]
    ref = orc.attention_hvp_dense(pick(x["q"]), pick(x["k"]), pick(x["v"]), scale, True, pick(x["q_dot"]), pick(x["k_dot"]), pick(x["v_dot"]),
                                  pick(x["dout"]), pick(x["dout_dot"]), row_block=256)
    errs = {}
    rel = lambda got, want: ((got.double() - want).abs().max() / want.abs().max().clamp_min(1e-30)).item()
    for (a, b) in res["chunks"]:
        for n in ("out", "out_dot", "dq", "dq_dot"):
            errs[n] = max(errs.get(n, 0.0), rel(res["q_side"][(a, b)][n][:, :, h:h + 1], getattr(ref, n)[:, a:b]))
    for n in ("dk", "dv", "dk_dot", "dv_dot"):  # the key rows this rank ends up with
        errs[n] = rel(res[n][:, h:h + 1], torch.cat([getattr(ref, n)[0, a:b] for a, b in res["kv_rows"]]))
    return errs


def long_context_run(shape, rank, world, dev, steps, warmup, check, exchange=None):
    """The long-context workload on `world` GPUs: ms per step (max over ranks), rates, the bytes every rank
    puts through the reduce-scatter, the part of the exchange that is not hidden under kernels, and (check)
    the results' largest relative error against the float64 oracle on one head."""
    import torch.distributed as dist
    from flashback_cute import _lib, parallel

    B, Hq, Hkv, S, D, causal = shape
    x = make_inputs(shape, dev, seed=0)  # same full tensors on every rank; each reads its own query chunks
    scale = D ** -0.5
    # a zig-zag-sharded job holds the rank's own query rows (its chunks, one after the other); K, V whole
    chunks = parallel.zigzag_chunks(S, rank, world, parallel.default_chunks_per_rank(S, world))
    mine = {n: parallel.zigzag_local(x[n], chunks).contiguous() for n in ("q", "dout", "q_dot", "dout_dot")}
    run = lambda **kw: parallel.hvp_query_sharded(mine["q"], x["k"], x["v"], mine["dout"], mine["q_dot"], x["k_dot"], x["v_dot"], mine["dout_dot"],
                                                  scale, True, rank=rank, world=world, exchange=exchange, **kw)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    errs = None
    if check:
        res = run()
        torch.cuda.synchronize()
        errs = long_context_check(x, res, rank, world, scale)
        t = torch.tensor(list(errs.values()), device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        errs = {n: v for n, v in zip(errs, t.tolist())}
        del res
    for _ in range(warmup):
        run()
    barrier()
    _lib.check_device_status()
    n0 = _lib.launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    tails = []
    for _ in range(steps):
        tails.append(run()["tail_events"])
    e1.record()
    barrier()
    # exchange time no kernel hid: how long the compute stream waited for the communication stream at the
    # end of a step (events recorded by the driver around that wait)
    tail = sum(a.elapsed_time(b) for a, b in tails) / steps
    launches = _lib.launches() - n0
    t = torch.tensor([e0.elapsed_time(e1), tail], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t[0].item() / steps
    F = unit_flops(B, Hq, S, D, causal)
    used = "none" if world == 1 else (exchange or "gather")
    if used in ("copy", "peer") and parallel._peer_disabled is not None:
        used = "nccl"  # symmetric memory could not be set up in this process: the driver fell back
    out = {
        "workload": LONG, "n_gpus": world, "ms_per_step": ms, "steps": steps,
        "value": (UNITS_JVP + UNITS_HVP) * F / (ms * 1e-3) / 1e12, "unit": "TFLOP/s (useful, whole job)",
        "per_gpu_tflops_useful": (UNITS_JVP + UNITS_HVP) * F / (ms * 1e-3) / 1e12 / world,
        "executed_tflops": sum(EXEC_UNITS.values()) * F / (ms * 1e-3) / 1e12,
        "query_chunks_per_gpu": len(chunks),  # zig-zag chunks, run as one problem with query segments
        "exchange": used,
        "collective": COLLECTIVE[used] + (" [symmetric memory unavailable: rows gathered by an all-gather collective instead]"
                                          if used == "gather" and parallel._peer_disabled is not None else ""),
        "exchanged_bytes_per_rank_per_step": 0 if world == 1 else (
            (4 * (S // world) * Hq * D * 2 + 4 * Hq * (S // world) * 4) * (world - 1) if used == "gather"   # own 16-bit rows + statistics to every peer
            else 4 * S * Hkv * D * 4 * (world - 1) // world),                                                 # float32 partial sums of the other ranks' key blocks
        "exposed_comm_ms": t[1].item(),
        "gpu_launches": launches,
    }
    if errs is not None:
        out["max_rel_err_vs_float64_oracle_one_head"] = {n: round(v, 5) for n, v in errs.items()}
        out["check_ok"] = all(v < 3e-2 for v in errs.values())  # sanity bound; the 2x-eager gate is in tests/
    del x
    torch.cuda.empty_cache()
    return out


def run_long(args, shape, rank, world, local_rank):
    """Long-context workload: zig-zag query-block sharding; key-side results by `--exchange` (parallel.hvp_query_sharded)."""
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    r = long_context_run(shape, rank, world, dev, steps=args.steps, warmup=max(args.warmup, 3), check=not args.no_check, exchange=args.exchange)
    clocks = sampler.stop() if sampler else None
    if rank != 0:
        return
    B, Hq, Hkv, S, D, causal = shape
    pk = peaks()
    line = {
        "metric": METRIC, "value": r["value"], "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload, "B": B, "H": Hq, "S": S, "D": D, "causal": causal,
                   "sharding": "zig-zag query blocks per GPU; K,V and tangents replicated; key side: " + r["collective"],
                   "l2": "inputs 2.1 GB, larger than the 126 MB L2"},
        "executed_tflops": r["executed_tflops"],
        "roofline": {"bound": "tensor", "kernel": "whole step (kernels + reduce-scatter)", "achieved": r["executed_tflops"] / world, "peak": pk["burst"],
                     "unit": "TFLOP/s", "frac": round(r["executed_tflops"] / world / pk["burst"], 4), "traffic": None,
                     "peak_source": pk["src"] + " (burst bf16 GEMM)"},
        "long_context": r,
        "cpu_baseline": None, "e2e": None, "gpu_launches": r["gpu_launches"], "clocks": clocks,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# autograd pipelines through the public API (the table the reference's bench/bench_double_backward.py prints)
# ------------------------------------------------------------------------------------------------
def eager_attention_gpu(q, k, v, causal, scale):
    """Plain eager attention with an S x S score matrix, the memory-hungry method the table compares with."""
    s = torch.einsum("bqhd,bkhd->bhqk", q, k).float() * scale
    if causal:
        sq, sk = q.shape[1], k.shape[1]
        keep = torch.ones(sq, sk, dtype=torch.bool, device=q.device).tril(sk - sq)
        s = s.masked_fill(~keep, float("-inf"))
    return torch.einsum("bhqk,bkhd->bqhd", s.softmax(-1).to(q.dtype), v)


def pipeline_call(depth, fn, q, k, v):
    """depth 0: forward without a tape; 1: + first-order grads; 2: + grads of the grads (double backward)."""
    if depth == 0:
        with torch.no_grad():
            return fn(q, k, v)
    grads = torch.autograd.grad(fn(q, k, v).sum(), (q, k, v), create_graph=depth == 2)
    if depth == 2:
        torch.autograd.grad(sum(g.sum() for g in grads), (q, k, v))


def time_call(call, warmup, iters):
    """Median CUDA-event ms of `call` and the peak bytes it allocates; None when it runs out of memory."""
    try:
        for _ in range(warmup):
            call()
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
        for a, b in ev:
            a.record()
            call()
            b.record()
        torch.cuda.synchronize()
        return statistics.median(a.elapsed_time(b) for a, b in ev), torch.cuda.max_memory_allocated()
    except torch.OutOfMemoryError:
        torch.cuda.empty_cache()
        return None


def run_pipelines(args):
    from flashback_cute import flashback_attn_func

    names = ("fwd", "fwd+bwd", "fwd+bwd+bwdbwd")
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[args.dtype]
    rows = []
    for hdim in args.hdim:
        scale = hdim ** -0.5
        for method in ("flashback_b200", "naive"):
            fn = (lambda q, k, v: flashback_attn_func(q, k, v, softmax_scale=scale, causal=args.causal)) if method == "flashback_b200" \
                else (lambda q, k, v: eager_attention_gpu(q, k, v, args.causal, scale))
            for seqlen in args.seqlens:
                if method == "naive" and seqlen > args.naive_max_seqlen:
                    continue
                g = torch.Generator(device="cuda").manual_seed(0)
                q, k, v = (torch.randn(args.batch, seqlen, args.heads, hdim, device="cuda", dtype=dtype, generator=g).requires_grad_() for _ in range(3))
                for depth, name in enumerate(names):
                    r = time_call(lambda: pipeline_call(depth, fn, q, k, v), warmup=3, iters=10)
                    rec = {"method": method, "hdim": hdim, "seqlen": seqlen, "pipeline": name, "batch": args.batch, "heads": args.heads,
                           "dtype": args.dtype, "causal": args.causal, "ms": None if r is None else round(r[0], 4),
                           "peak_gb": None if r is None else round(r[1] / 2**30, 3)}
                    rows.append(rec)
                    print(json.dumps(rec), flush=True)
                del q, k, v
                torch.cuda.empty_cache()
    # the same records as a table
    print(f"# batch={args.batch} heads={args.heads} dtype={args.dtype} causal={args.causal} ({torch.cuda.get_device_name()})")
    print("# " + f"{'method':<15}{'hdim':>5}{'seqlen':>7}" + "".join(f"{n + ' ms':>19}{'GB':>7}" for n in names))
    key = lambda r: (r["method"], r["hdim"], r["seqlen"])
    for kk in dict.fromkeys(map(key, rows)):
        cells = ""
        for n in names:
            r = next(x for x in rows if key(x) == kk and x["pipeline"] == n)
            cells += f"{'OOM':>19}{'-':>7}" if r["ms"] is None else f"{r['ms']:>19.3f}{r['peak_gb']:>7.2f}"
        print("# " + f"{kk[0]:<15}{kk[1]:>5}{kk[2]:>7}" + cells)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--no-long", action="store_true", help="N > 1, default workload: leave out the long_context sub-run")
    ap.add_argument("--no-check", action="store_true", help="long-context workload: leave out the comparison with the oracle")
    ap.add_argument("--exchange", default=None, choices=["copy", "peer", "nccl", "gather"],
                    help="long-context workload: how the key-side results come about across the GPUs (see parallel.hvp_query_sharded)")
    ap.add_argument("--pipelines", action="store_true", help="print the autograd-pipelines table (1 GPU) instead of the bench line")
    ap.add_argument("--kernels-only", action="store_true", help="1 GPU: only the four kernel calls, per-kernel times (for ncu captures)")
    ap.add_argument("--rank-share", default=None, help="long-context workload, 1 GPU: R/N = time the kernels of rank R of an N-rank job (no communication)")
    ap.add_argument("--shape", default=None, help="with --kernels-only: B,Hq,Hkv,S,D,causal(0/1) instead of the workload's shape")
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--hdim", type=int, nargs="+", default=[64, 128])
    ap.add_argument("--seqlens", type=int, nargs="+", default=[512, 1024, 2048, 4096, 8192])
    ap.add_argument("--dtype", choices=["bf16", "fp16", "fp32"], default="bf16")
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--naive-max-seqlen", type=int, default=4096)
    args = ap.parse_args()
    if args.pipelines:
        run_pipelines(args)
        return
    shape = WORKLOADS[args.workload]
    if args.rank_share:
        run_rank_share(args, WORKLOADS[LONG])
        return
    if args.kernels_only:
        if args.shape:
            v = [int(t) for t in args.shape.split(",")]
            shape = (*v[:5], bool(v[5]))
        run_kernels_only(args, shape)
        return
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        run_reference(args, shape, rank)
        return
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        (run_long if args.workload == LONG else run_ours)(args, shape, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()

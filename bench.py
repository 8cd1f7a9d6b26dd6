"""Benchmark of the attention JVP-forward + HVP-backward hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One "step" = one JVP-forward pass (O, LSE, O_dot, row statistics) followed by one HVP-backward
pass (dQ, dK, dV and their directional derivatives from dO and dO_dot) over one batch of
synthetic inputs with the shapes and value distributions of the named workload
(default: causal GQA bf16, B=2, Hq=32, Hkv=8, S=8192, D=128).

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
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = [r for r in self.rows if len(r) == 6 and r[0].isdigit()]
        if not rows:
            return None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in rows for n, v in zip(names, r[2:]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(int(r[0]) for r in rows), "sm_max_mhz": int(rows[0][1]), "reasons": reasons, "samples": len(rows)}


def make_inputs(shape, device, seed, dtype=torch.bfloat16, pinned_host=False):
    """Q,K,V ~ N(0,1); tangents ~ N(0, 0.1^2); dO, dO_dot ~ N(0,1); drawn in this fixed order."""
    B, Hq, Hkv, S, D, _ = shape
    g = torch.Generator(device=device).manual_seed(seed)
    def rn(h, std=1.0):
        return (torch.randn(B, S, h, D, generator=g, device=device, dtype=torch.float32) * std).to(dtype)
    t = dict(q=rn(Hq), k=rn(Hkv), v=rn(Hkv), q_dot=rn(Hq, 0.1), k_dot=rn(Hkv, 0.1), v_dot=rn(Hkv, 0.1), dout=rn(Hq), dout_dot=rn(Hq))
    if pinned_host:
        t = {n: x.cpu().pin_memory() for n, x in t.items()}
    return t


# ------------------------------------------------------------------------------------------------
# reference arm / CPU baseline: eager forward-over-reverse on the host cores
# ------------------------------------------------------------------------------------------------
def cpu_step(shape, sample):
    """One (batch, q-head) slice of the workload through the eager CPU restatement."""
    from oracle import attention_oracle as orc

    _, _, _, _, D, causal = shape
    scale = D ** -0.5
    fn = lambda a, b, c: orc.eager_attention(a, b, c, causal, scale, False)

    def vjp_fn(a, b, c, d):
        o, pull = torch.func.vjp(fn, a, b, c)
        return (o, *pull(d))

    t0 = time.perf_counter()
    torch.func.jvp(vjp_fn, (sample["q"], sample["k"], sample["v"], sample["dout"]),
                   (sample["q_dot"], sample["k_dot"], sample["v_dot"], sample["dout_dot"]))
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
    t = make_inputs((1, 1, 1, S, D, causal), "cpu", seed, dtype=torch.float32)
    return t


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
        "impl": "reference", "metric": "JVP-fwd + HVP-bwd TFLOP/s (useful matmuls)", "value": val, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "B": B, "Hq": Hq, "Hkv": Hkv, "S": S, "D": D, "causal": causal},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def run_ours(args, shape, rank, world, local_rank):
    import torch.distributed as dist
    from flashback_cute import _lib, interface as I, flashback_attn_hvp

    B, Hq, Hkv, S, D, causal = shape
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    scale = D ** -0.5
    # Weak scaling: every rank owns its own (batch, head) shard of a world-times larger batch.
    x = make_inputs(shape, dev, seed=rank)
    g = I._Geom(x["q"], x["k"], None, None, None, None, scale, causal)
    out, out_dot = torch.empty_like(x["q"]), torch.empty_like(x["q"])
    lse, z1, dpsum, ddot = (I._stat(x["q"], None) for _ in range(4))
    dq, dqd = torch.empty_like(x["q"]), torch.empty_like(x["q"])
    dk, dv, dkd, dvd = (torch.empty_like(x["k"]) for _ in range(4))
    tang = (x["q_dot"], x["k_dot"], x["v_dot"], x["dout_dot"])
    N_ = None

    def k_jvp():
        _lib.jvp_fwd(g.prob, x["q"], x["k"], x["v"], x["q_dot"], x["k_dot"], x["v_dot"], out, out_dot, lse, z1,
                     x["dout"], x["dout_dot"], dpsum, ddot)

    def k_dq():
        _lib.hvp_bwd(g.prob, x["q"], x["k"], x["v"], x["dout"], *tang, lse, dpsum, z1, ddot, dq, N_, N_, dqd, N_, N_)

    def k_dkv_first():
        _lib.hvp_bwd(g.prob, x["q"], x["k"], x["v"], x["dout"], *tang, lse, dpsum, z1, ddot, N_, dk, dv, N_, N_, N_)

    def k_dkv_dot():
        _lib.hvp_bwd(g.prob, x["q"], x["k"], x["v"], x["dout"], *tang, lse, dpsum, z1, ddot, N_, N_, N_, N_, dkd, dvd)

    def k_dkv_all():
        _lib.hvp_bwd(g.prob, x["q"], x["k"], x["v"], x["dout"], *tang, lse, dpsum, z1, ddot, N_, dk, dv, N_, dkd, dvd)

    kernels = [("jvp_fwd", k_jvp), ("hvp_dq", k_dq), ("hvp_dkv_first", k_dkv_first), ("hvp_dkv_dot", k_dkv_dot)]
    exec_units = dict(EXEC_UNITS)
    if D == 64:  # head_dim 64: dK, dV and their tangents come out of one launch (6 S-like + 6 output GEMMs)
        kernels = [("jvp_fwd", k_jvp), ("hvp_dq", k_dq), ("hvp_dkv_all", k_dkv_all)]
        exec_units = {"jvp_fwd": 6, "hvp_dq": 9, "hvp_dkv_all": 12}

    def step(events=None):
        for i, (_, fn) in enumerate(kernels):
            if events is not None:
                events[i].record()
            fn()
        if events is not None:
            events[len(kernels)].record()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    _lib.check_device_status()
    launches0 = _lib.launches()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(len(kernels) + 1)] for _ in range(args.steps)]
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_start.record()
    for s in range(args.steps):
        step(evs[s])
    t_end.record()
    barrier()
    clocks = sampler.stop() if sampler else None
    launches = _lib.launches() - launches0
    _lib.check_device_status()
    total_ms = t_start.elapsed_time(t_end)
    kern_ms = {n: sum(e[i].elapsed_time(e[i + 1]) for e in evs) / args.steps for i, (n, _) in enumerate(kernels)}

    # The reference's own double backward (K1 + K2: O and LSE known, tangents only, dO_dot = 0), timed
    # separately for information: 5 + 10 matmul units needed, 5 + 15 executed.
    def k1():
        _lib.jvp_fwd(g.prob, x["q"], x["k"], x["v"], x["q_dot"], x["k_dot"], x["v_dot"], out, out_dot, lse, z1,
                     x["dout"], None, dpsum, ddot, lse_known=True)

    def k2():
        _lib.hvp_bwd(g.prob, x["q"], x["k"], x["v"], x["dout"], x["q_dot"], x["k_dot"], x["v_dot"], None, lse, dpsum, z1, ddot,
                     N_, N_, N_, dqd, dkd, dvd)

    _lib.jvp_fwd(g.prob, x["q"], x["k"], x["v"], None, None, None, out, None, lse, None)  # O, LSE for K1
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

    # End to end through the public API with HOST buffers: every step copies all eight inputs from
    # pinned host memory and all eight results back. The three legs of consecutive steps overlap on
    # three streams (copy-in of step i+1 and copy-out of step i-1 run under the kernels of step i),
    # with two device input sets; each step's copies are inside the timed region.
    host = make_inputs(shape, dev, seed=rank, pinned_host=True)
    dev_in = [{n: torch.empty(t.shape, dtype=t.dtype, device=dev) for n, t in host.items()} for _ in range(2)]
    host_out = None
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    s_comp = torch.cuda.current_stream(dev)
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_free = [torch.cuda.Event() for _ in range(2)]
    ev_out = None
    e2e_i = 0

    def e2e_step():
        nonlocal host_out, ev_out, e2e_i
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
    e2e_ms = sorted(e2e_repeats)[1]
    h2d = sum(t.numel() * t.element_size() for t in host.values())
    d2h = sum(t.numel() * t.element_size() for t in host_out)

    # max over ranks
    stats = torch.tensor([total_ms, e2e_ms, *kern_ms.values()], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms = stats[0].item(), stats[1].item()
    kern_ms = {n: stats[2 + i].item() for i, n in enumerate(kern_ms)}
    if rank != 0:
        return

    F = unit_flops(B, Hq, S, D, causal)
    ms_per_step = total_ms / args.steps
    useful = (UNITS_JVP + UNITS_HVP) * F * world
    executed = sum(exec_units.values()) * F * world
    value = useful / (ms_per_step * 1e-3) / 1e12
    pk = peaks()
    per_kernel = {}
    for n, ms in kern_ms.items():
        tf = exec_units[n] * F / (ms * 1e-3) / 1e12
        per_kernel[n] = {"ms": round(ms, 4), "executed_units": exec_units[n], "tflops": round(tf, 1),
                         "frac_of_burst_peak": round(tf / pk["burst"], 4), "frac_of_sustained_peak": round(tf / pk["sustained"], 4),
                         "frac_of_nominal_2250": round(tf / 2250.0, 4)}
    dom = max(kern_ms, key=kern_ms.get)
    dom_tf = per_kernel[dom]["tflops"]
    hvp_ms = sum(ms for n, ms in kern_ms.items() if n.startswith("hvp_"))
    hvp_exec = sum(u for n, u in exec_units.items() if n.startswith("hvp_"))
    traffic_file = ROOT / "profiles" / "dram_traffic.json"
    traffic = None
    if traffic_file.exists():
        traffic = json.loads(traffic_file.read_text()).get(args.workload, {}).get(dom)

    # CPU baseline: bounded sample on this box's host cores
    use_all_host_threads()
    sample = cpu_sample(shape)
    cpu_step(shape, cpu_sample((1, 1, 1, 256, D, causal)))
    cpu_s = cpu_step(shape, sample)
    cpu_val = (UNITS_JVP + UNITS_HVP) * unit_flops(1, 1, S, D, causal) / cpu_s / 1e12

    line = {
        "metric": "JVP-fwd + HVP-bwd TFLOP/s (useful matmuls)", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload, "B_per_gpu": B, "Hq": Hq, "Hkv": Hkv, "S": S, "D": D, "causal": causal,
                   "mode": "fused JVP-fwd (O, LSE, O_dot, stats) + HVP-bwd (dQ,dK,dV + directional derivatives, dO_dot given)",
                   "sharding": "(batch, kv-head) groups per GPU, no communication",
                   "l2": "inputs+outputs > 1 GB per step, larger than the 126 MB L2", "useful_units": UNITS_JVP + UNITS_HVP,
                   "executed_units": sum(exec_units.values())},
        "executed_tflops": executed / (ms_per_step * 1e-3) / 1e12,
        "jvp_fwd": {"ms": kern_ms["jvp_fwd"], "tflops_executed": per_kernel["jvp_fwd"]["tflops"],
                    "frac_of_burst_peak": per_kernel["jvp_fwd"]["frac_of_burst_peak"]},
        "hvp_bwd": {"ms": hvp_ms, "tflops_useful": UNITS_HVP * F / (hvp_ms * 1e-3) / 1e12,
                    "tflops_executed": hvp_exec * F / (hvp_ms * 1e-3) / 1e12,
                    "frac_of_burst_peak_executed": hvp_exec * F / (hvp_ms * 1e-3) / 1e12 / pk["burst"]},
        "kernels": per_kernel,
        "double_backward": {"note": "the reference's K1 + K2 step (LSE known, tangents only, dO_dot = 0), this rank only",
                            "k1_ms": db_k1, "k2_ms": db_k2, "useful_units": 15, "executed_units": 20,
                            "tflops_useful": 15 * F / ((db_k1 + db_k2) * 1e-3) / 1e12,
                            "k1_tflops": 5 * F / (db_k1 * 1e-3) / 1e12, "k2_tflops_executed": 15 * F / (db_k2 * 1e-3) / 1e12},
        "roofline": {"bound": "tensor", "kernel": dom, "achieved": dom_tf, "peak": pk["sustained"], "unit": "TFLOP/s",
                     "frac": round(dom_tf / pk["sustained"], 4), "traffic": traffic, "peak_source": pk["src"] + " (sustained bf16 GEMM)",
                     "peak_burst": pk["burst"]},
        "cpu_baseline": {"value": cpu_val, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"1 (batch, q-head) slice at S={S}, float32, eager forward-over-reverse, {cpu_s:.1f} s"},
        "e2e": {"value": useful / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms, "ms_per_step_repeats": e2e_repeats,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "clocks": clocks,
    }
    print(json.dumps(line), flush=True)


def run_long(args, shape, rank, world, local_rank):
    """Long-context workload: zig-zag query-block sharding + reduce-scatter of partial dK/dV."""
    import torch.distributed as dist
    from flashback_cute import _lib, parallel

    B, Hq, Hkv, S, D, causal = shape
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    x = make_inputs(shape, dev, seed=0)  # same full tensors on every rank; each reads its own query chunks
    scale = D ** -0.5

    def step():
        return parallel.hvp_query_sharded(x["q"], x["k"], x["v"], x["dout"], x["q_dot"], x["k_dot"], x["v_dot"], x["dout_dot"],
                                          scale, True, rank=rank, world=world)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    _lib.check_device_status()
    n0 = _lib.launches()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    clocks = sampler.stop() if sampler else None
    launches = _lib.launches() - n0
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank != 0:
        return
    ms = t.item() / args.steps
    F = unit_flops(B, Hq, S, D, causal)
    value = (UNITS_JVP + UNITS_HVP) * F / (ms * 1e-3) / 1e12
    executed = sum(EXEC_UNITS.values()) * F / (ms * 1e-3) / 1e12
    pk = peaks()
    line = {
        "metric": "JVP-fwd + HVP-bwd TFLOP/s (useful matmuls)", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload, "B": B, "H": Hq, "S": S, "D": D, "causal": causal,
                   "sharding": "zig-zag query blocks per GPU; K,V and tangents replicated; NCCL reduce-scatter (fp32) of partial dK,dV,dK_dot,dV_dot overlapped per head group",
                   "l2": "inputs 2.1 GB, larger than the 126 MB L2"},
        "executed_tflops": executed,
        "roofline": {"bound": "tensor", "kernel": "whole step (kernels + reduce-scatter)", "achieved": executed / world, "peak": pk["sustained"],
                     "unit": "TFLOP/s", "frac": round(executed / world / pk["sustained"], 4), "traffic": None, "peak_source": pk["src"] + " (sustained bf16 GEMM)"},
        "cpu_baseline": None, "e2e": None, "gpu_launches": launches, "clocks": clocks,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    args = ap.parse_args()
    shape = WORKLOADS[args.workload]
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

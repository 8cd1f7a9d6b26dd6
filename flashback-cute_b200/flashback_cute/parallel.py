"""Multi-GPU drivers for the JVP-forward / HVP-backward path: one process per GPU,
`torch.distributed` for the plumbing. (The reference is single-GPU; its kernel grids are already
(tile, head, batch), flashback_cute/jvp_fwd_sm90.py:242-264 and hvp_bwd_sm90.py:340-363, which is
what makes both partitions below natural.)

Two partitions:

* `group_slices` / `hvp_head_sharded` — every (batch, kv-head) group is independent (the G query
  heads of a kv head stay together so dK/dV never cross ranks): rank r takes a contiguous range
  of groups and runs the same kernels on strided views. No communication.

* `hvp_query_sharded` — long sequences with few heads: query rows are split into 2*world chunks
  and rank r takes chunks r and 2*world-1-r (zig-zag, so causal work is balanced). K, V and their
  tangents are replicated. Because the kernels' causal mask is bottom-right aligned, a query chunk
  [a, b) run against keys [0, b) is masked exactly as in the full problem. O, O_dot, dQ, dQ_dot
  are local to the chunk; every rank produces PARTIAL dK, dV, dK_dot, dV_dot over the keys it
  saw, which are summed in float32 and reduce-scattered along the key axis (NCCL reduce-scatter
  over NVLink; all-reduce + slice on backends without reduce-scatter, e.g. gloo in the CPU tests).
  Heads are processed in groups so the collective of one group overlaps the kernels of the next.
"""

from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from .interface import flashback_attn_hvp


def group_slices(batch: int, heads_kv: int, rank: int, world: int) -> Tuple[slice, slice]:
    """(batch slice, kv-head slice) of the (batch, kv-head) groups owned by `rank`.
    Requires world | batch*heads_kv and that a rank's range is whole batches or lies inside one."""
    total = batch * heads_kv
    if total % world:
        raise ValueError(f"{world} ranks do not divide {batch}x{heads_kv} (batch, kv-head) groups")
    n = total // world
    g0 = rank * n
    if n % heads_kv == 0:
        return slice(g0 // heads_kv, (g0 + n) // heads_kv), slice(0, heads_kv)
    if heads_kv % n == 0:
        b = g0 // heads_kv
        h0 = g0 - b * heads_kv
        return slice(b, b + 1), slice(h0, h0 + n)
    raise ValueError("a rank's group range must be whole batches or lie inside one batch")


def shard_by_group(t: torch.Tensor, bs: slice, hs: slice, heads_kv: int) -> torch.Tensor:
    """View of a (B, S, H, D) tensor restricted to the groups (bs, hs); H may be heads_q = G*heads_kv."""
    g = t.shape[2] // heads_kv
    return t[bs, :, hs.start * g : hs.stop * g]


def hvp_head_sharded(q, k, v, dout, q_dot, k_dot, v_dot, dout_dot=None, softmax_scale=None, causal=False,
                     rank: Optional[int] = None, world: Optional[int] = None, first_order: bool = True):
    """Each rank computes its own (batch, kv-head) groups of the full problem; returns the local
    results (O, O_dot, dQ, dK, dV, dQ_dot, dK_dot, dV_dot) for its slice and the slices themselves."""
    rank = dist.get_rank() if rank is None else rank
    world = dist.get_world_size() if world is None else world
    hkv = k.shape[2]
    bs, hs = group_slices(q.shape[0], hkv, rank, world)
    pick = lambda t: None if t is None else shard_by_group(t, bs, hs, hkv)
    res = flashback_attn_hvp(pick(q), pick(k), pick(v), pick(dout), pick(q_dot), pick(k_dot), pick(v_dot), pick(dout_dot),
                             softmax_scale, causal, first_order=first_order)
    return res, (bs, hs)


def zigzag_chunks(seqlen: int, rank: int, world: int) -> List[Tuple[int, int]]:
    """Query-row ranges [a, b) of rank `rank`: chunks r and 2*world-1-r of 2*world equal chunks."""
    if seqlen % (2 * world):
        raise ValueError("sequence length must be a multiple of 2*world")
    c = seqlen // (2 * world)
    return [(rank * c, (rank + 1) * c), ((2 * world - 1 - rank) * c, (2 * world - rank) * c)]


def _reduce_scatter_sum(full: torch.Tensor, world: int, rank: int, group=None):
    """Sum `full` (leading dim = keys, a multiple of world) over ranks; return this rank's key block
    and the async work handle."""
    n = full.shape[0] // world
    if world == 1:
        return full, None
    if dist.get_backend(group) == "nccl":
        out = torch.empty((n, *full.shape[1:]), dtype=full.dtype, device=full.device)
        work = dist.reduce_scatter_tensor(out, full, op=dist.ReduceOp.SUM, group=group, async_op=True)
        return out, work
    work = dist.all_reduce(full, op=dist.ReduceOp.SUM, group=group, async_op=True)
    return full[rank * n : (rank + 1) * n], work


def hvp_query_sharded(q, k, v, dout, q_dot, k_dot, v_dot, dout_dot=None, softmax_scale=None, causal=True,
                      rank: Optional[int] = None, world: Optional[int] = None, heads_per_group: int = 16, group=None):
    """Long-context partition (batch must be 1). q-like inputs are the FULL tensors (every rank draws
    or receives the same data); each rank reads only its zig-zag query chunks.

    Returns a dict: per local chunk (a, b) the q-side results ("out", "out_dot", "dq", "dq_dot"),
    and under "dk", "dv", "dk_dot", "dv_dot" this rank's key block [rank*S/world, (rank+1)*S/world)
    of the fully summed gradients, in float32.
    """
    rank = dist.get_rank(group) if rank is None else rank
    world = dist.get_world_size(group) if world is None else world
    if q.shape[0] != 1:
        raise ValueError("query-block sharding is for batch 1; use the (batch, kv-head) partition otherwise")
    S, Hq, D = q.shape[1], q.shape[2], q.shape[3]
    Sk, Hkv = k.shape[1], k.shape[2]
    if S != Sk or not causal:
        raise ValueError("query-block sharding expects causal self-attention (Sq == Sk)")
    G = Hq // Hkv
    chunks = zigzag_chunks(S, rank, world)
    hg = max(1, min(heads_per_group, Hkv))
    while Hkv % hg:
        hg -= 1
    q_side = {c: {n: torch.empty((1, c[1] - c[0], Hq, D), dtype=q.dtype, device=q.device) for n in ("out", "out_dot", "dq", "dq_dot")} for c in chunks}
    kv_out = {n: torch.empty((S // world, Hkv, D), dtype=torch.float32, device=q.device) for n in ("dk", "dv", "dk_dot", "dv_dot")}
    pending = []
    comm_stream = torch.cuda.Stream(device=q.device) if q.is_cuda else None

    def exchange(names, partial, hk):
        """Reduce-scatter partial[n] for n in names on the communication stream, after everything
        enqueued so far on the compute stream."""
        if comm_stream is not None:
            comm_stream.wait_stream(torch.cuda.current_stream(q.device))
            ctx = torch.cuda.stream(comm_stream)
        else:
            ctx = _NullCtx()
        with ctx:
            for n in names:
                shard, work = _reduce_scatter_sum(partial[n], world, rank, group)
                pending.append((n, hk, shard, work, partial[n]))

    for h0 in range(0, Hkv, hg):
        hk = slice(h0, h0 + hg)
        hq = slice(h0 * G, (h0 + hg) * G)
        # partial sums over this rank's queries, float32: the first chunk is cast into the buffer, the
        # other one is added on top. The chunk that sees the most keys goes last, so that the exchange
        # of dK, dV (complete after its first-order kernels) runs under its long tangent kernels; the
        # exchange of dK_dot, dV_dot runs under the next head group's kernels.
        partial = {n: torch.empty((S, hg, D), dtype=torch.float32, device=q.device) for n in kv_out}
        order = sorted(chunks, key=lambda c: c[1])

        def fold(n, t, b, first):
            if first:
                partial[n][:b].copy_(t[0])
                partial[n][b:].zero_()
            else:
                partial[n][:b].add_(t[0])

        for ci, (a, b) in enumerate(order):
            first, last = ci == 0, ci == len(order) - 1
            qs = lambda t: None if t is None else t[:, a:b, hq]
            ks = lambda t: t[:, :b, hk]

            def kv_ready(dk, dv):
                fold("dk", dk, b, first)
                fold("dv", dv, b, first)
                if last:
                    exchange(("dk", "dv"), partial, hk)

            o, od, dq, dk, dv, dqd, dkd, dvd = flashback_attn_hvp(
                qs(q), ks(k), ks(v), qs(dout), qs(q_dot), ks(k_dot), ks(v_dot), qs(dout_dot), softmax_scale, True,
                on_first_order_kv=kv_ready)
            for n, t in (("out", o), ("out_dot", od), ("dq", dq), ("dq_dot", dqd)):
                q_side[(a, b)][n][:, :, hq] = t
            fold("dk_dot", dkd, b, first)
            fold("dv_dot", dvd, b, first)
        exchange(("dk_dot", "dv_dot"), partial, hk)
    for n, hk, shard, work, keep in pending:
        if work is not None:
            work.wait()
    if comm_stream is not None:
        torch.cuda.current_stream(q.device).wait_stream(comm_stream)
    for n, hk, shard, work, keep in pending:
        kv_out[n][:, hk] = shard
    return {"chunks": chunks, "q_side": q_side, **kv_out}


class _NullCtx:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False

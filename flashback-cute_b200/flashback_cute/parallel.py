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


def zigzag_chunks(seqlen: int, rank: int, world: int, per_rank: int = 2) -> List[Tuple[int, int]]:
    """Query-row ranges [a, b) of rank `rank`, ascending. per_rank = 2: chunks r and 2*world-1-r of
    2*world equal chunks (zig-zag: every rank gets the same causal work). per_rank = 4: the same zig-zag
    over each half of 4*world chunks (r, 2*world-1-r, 2*world+r, 4*world-1-r): the same balance between the
    ranks, and inside a rank four classes of query tiles instead of a heavy and a light one, which is what
    lets a launch's heaviest-first order fill the last wave of CTAs."""
    if per_rank not in (2, 4) or seqlen % (per_rank * world):
        raise ValueError("chunks per rank must be 2 or 4 and the sequence length a multiple of chunks per rank x world")
    c = seqlen // (per_rank * world)
    idx = []
    for z in range(per_rank // 2):
        idx += [2 * world * z + rank, 2 * world * (z + 1) - 1 - rank]
    return [(i * c, (i + 1) * c) for i in idx]


def default_chunks_per_rank(seqlen: int, world: int, on_gpu: bool = True) -> int:
    """Four chunks per rank where they are whole 128-row owner tiles of the kernels (any size on CPU ranks), else two."""
    return 4 if seqlen % (4 * world * (128 if on_gpu else 1)) == 0 else 2


def zigzag_local(t: Optional[torch.Tensor], chunks) -> Optional[torch.Tensor]:
    """Rows of a rank's chunks of a (1, S, H, D) tensor, one after the other: the layout the kernels take
    as ONE problem with query segments (a view when the chunks are adjacent, else a copy)."""
    if t is None:
        return None
    if all(b == a for (_, b), (a, _) in zip(chunks[:-1], chunks[1:])):
        return t[:, chunks[0][0]:chunks[-1][1]]
    return torch.cat([t[:, a:b] for a, b in chunks], 1)


def zigzag_segments(chunks) -> List[Tuple[int, int]]:
    """fb_problem.seg_rows / seg_shift for a rank's chunks held one after the other against keys
    [0, end of the last chunk): per break (local row where the next chunk starts, positions by which the
    rows before it sit earlier than bottom-right alignment puts them). Adjacent chunks need no break."""
    total = sum(b - a for a, b in chunks)
    off = chunks[-1][1] - total
    segs, lo = [], 0
    for (a, b), (a_next, _) in zip(chunks[:-1], chunks[1:]):
        hi = lo + (b - a)
        if a_next != b:
            segs.append((hi, lo + off - a))
        lo = hi
    # rows of one segment must share a shift: adjacent chunks do (their rows continue each other)
    return segs


def zigzag_key_segments(chunks, seqlen: int) -> List[Tuple[int, int]]:
    """fb_problem.seg_rows / seg_shift with FB_FLAG_SEG_KEYS for a rank's KEY chunks held one after the
    other against all `seqlen` query rows: per break (local row where a run of adjacent chunks ends,
    positions by which its rows sit earlier than bottom-right alignment puts them)."""
    total = sum(b - a for a, b in chunks)
    segs, lo = [], 0
    for t, (a, b) in enumerate(chunks):
        hi = lo + (b - a)
        if t + 1 == len(chunks) or chunks[t + 1][0] != b:
            segs.append((hi, (seqlen - total) + lo - a))
        lo = hi
    if segs and segs[-1][1] == 0:
        segs.pop()  # the last run is where bottom-right alignment puts it
    return segs


_perm_cache = {}


def zigzag_permutation(seqlen: int, world: int, per_rank: int, device) -> torch.Tensor:
    """perm[g] = position of global row g in the concatenation of all ranks' local rows (rank-major)."""
    key = (seqlen, world, per_rank, str(device))
    if key not in _perm_cache:
        perm = torch.empty(seqlen, dtype=torch.int64)
        n_loc = seqlen // world
        for r in range(world):
            lo = 0
            for a, b in zigzag_chunks(seqlen, r, world, per_rank):
                perm[a:b] = r * n_loc + lo + torch.arange(b - a)
                lo += b - a
        _perm_cache[key] = perm.to(device)
    return _perm_cache[key]


def default_heads_per_group(heads_kv: int, world: int) -> int:
    """Heads per exchange group of `hvp_query_sharded`: all of them. Smaller groups would let the
    reduce-scatter of one group run under the kernels of the next, but measured on 8 B200s (S=65536,
    16 heads) that loses more than it hides: the kernels here keep one CTA per SM for the whole launch,
    so NCCL's CTAs wait for SMs, then hold them, and both sides slow down - 29.8 ms per step with one
    group (4.1 ms of exchange after the last kernel), 31.9 with two or four groups (3.2 / 1.8 ms exposed),
    32.5 with eight, 35.4 with sixteen. With one group only the dK, dV exchange overlaps (the tangent
    kernels of the same group)."""
    return heads_kv


def _reduce_scatter_sum(full: torch.Tensor, out: Optional[torch.Tensor], world: int, rank: int, group=None):
    """Sum `full` (leading dim = keys, a multiple of world) over ranks; return this rank's key block
    and the async work handle. `out` (NCCL only) receives the block."""
    n = full.shape[0] // world
    if world == 1:
        return full, None
    if dist.get_backend(group) == "nccl":
        # NCCL runs the collective on its own stream; waiting on the handle makes the CURRENT stream (the
        # driver's communication stream) wait for it, without blocking the host, so that events recorded
        # on that stream afterwards mean "exchange complete".
        dist.reduce_scatter_tensor(out, full, op=dist.ReduceOp.SUM, group=group, async_op=True).wait()
        return out, None
    work = dist.all_reduce(full, op=dist.ReduceOp.SUM, group=group, async_op=True)
    return full[rank * n : (rank + 1) * n], work


_KV_NAMES = ("dk", "dv", "dk_dot", "dv_dot")
_peer_cache = {}       # (device, world, rows, heads, D) -> (slots tensor, peer addresses, handle, flag)
_peer_disabled = None  # reason why the peer-store exchange is not available in this process, once known


def _peer_slots(device, world, rows, heads, D, group):
    """Symmetric buffer [source rank][4 outputs][rows][heads][D] float32 on every rank (rows = this rank's
    key block) together with its address on every peer. A collective call; cached per shape."""
    global _peer_disabled
    key = (str(device), world, rows, heads, D)
    if key not in _peer_cache:
        import torch.distributed._symmetric_memory as symm_mem

        _peer_cache.clear()
        t = symm_mem.empty((world, 4, rows, heads, D), dtype=torch.float32, device=device)
        hdl = symm_mem.rendezvous(t, group if group is not None else dist.group.WORLD)
        flag = torch.zeros(1, dtype=torch.float32, device=device)
        _peer_cache[key] = (t, [int(p) for p in hdl.buffer_ptrs], hdl, flag)
    return _peer_cache[key]


def _stream_barrier(flag, group):
    """Barrier across the ranks in stream order (a one-element all-reduce): every rank's work enqueued before
    it has completed when work enqueued after it starts, on every rank. The host does not block."""
    dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=group)
_partial_cache = {}  # (device, S, heads, D) -> two sets of float32 partial-sum buffers, reused call after call


def _partial_sets(device, S, hg, D):
    key = (str(device), S, hg, D)
    if key not in _partial_cache:
        _partial_cache.clear()  # one shape at a time: these are the largest buffers of the driver
        _partial_cache[key] = [{n: torch.empty((S, hg, D), dtype=torch.float32, device=device) for n in _KV_NAMES} for _ in range(2)]
    return _partial_cache[key]


# The stream that carries the row copies of "gather" beside the kernels is HIGH priority: at normal priority the
# copies only completed at the next kernel boundary (2 GPUs, a rank's 536 MB to its peer and to itself: 1.4 ms
# on an idle GPU, 4.5 ms beside the forward kernel at high priority, the whole forward at normal priority).
_COPY_PRIORITY = -1
_gather_cache = {}  # (device, world, S, heads, D, dtype) -> (symmetric tensor [4][S][heads][D], every rank's copy as a flat tensor, flag)


def _gather_buffers(device, world, S, heads, D, dtype, group):
    """Symmetric buffer for the gathered q-like tensors (q, dout, q_dot, dout_dot in global row order) on
    every rank, with every rank's buffer as a flat tensor. A collective call; cached per shape."""
    key = (str(device), world, S, heads, D, dtype)
    if key not in _gather_cache:
        import torch.distributed._symmetric_memory as symm_mem

        _gather_cache.clear()
        t = symm_mem.empty((4, S, heads, D), dtype=dtype, device=device)
        hdl = symm_mem.rendezvous(t, group if group is not None else dist.group.WORLD)
        remote = [hdl.get_buffer(o, (t.numel(),), dtype, 0) for o in range(world)]
        flag = torch.zeros(1, dtype=torch.float32, device=device)
        _gather_cache[key] = (t, remote, flag)
    return _gather_cache[key]


_hp_groups = {}  # process group -> a twin whose NCCL kernels run on a high-priority stream


def _high_priority_group(group):
    """A process group over the same ranks whose collectives run on a HIGH-priority stream. The kernels here
    keep every SM busy with one long CTA each; a collective enqueued beside them at normal priority gets no
    SM until the compute kernel's last wave, at high priority it gets the first SM a CTA leaves. A collective
    call (every rank creates the group at the same point); cached. Only for the default group: creating a
    group needs every process of the job, which the members of a caller's subgroup cannot promise, so a
    subgroup is used as it is."""
    if group is not None and group is not dist.group.WORLD:
        return group
    key = dist.distributed_c10d._get_default_group()  # (a process that re-initialises torch.distributed gets a new twin)
    if key not in _hp_groups:
        _hp_groups.clear()
        opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
        _hp_groups[key] = dist.new_group(ranks=list(range(dist.get_world_size())), backend="nccl", pg_options=opts)
    return _hp_groups[key]


class _QueryGather:
    """exchange="gather": instead of summing partial dK/dV over the ranks, every rank gets ALL query-side
    rows (q, dout, q_dot, dout_dot and, after the query-side kernels, the four row statistics) and runs
    the dK/dV kernels for the KEYS of its own chunks against all queries (key segments): each rank then
    holds the complete dK, dV, dK_dot, dV_dot of its own tokens, in the I/O dtype, and nothing is summed
    across GPUs. What travels: the 16-bit q-like rows (every rank sends its S / world rows to every peer:
    half the bytes of the float32 partial sums) while the query-side kernels run - copy engines, no SM -
    and 16 bytes of statistics per query row and head, all-gathered under the dQ kernels."""

    def __init__(self, _lib, x, st_all, chunks, rank, world, S, Hq, D, per_rank, group, use_symm):
        self._lib, self.x, self.st_all, self.chunks = _lib, x, st_all, chunks
        self.rank, self.world, self.S, self.Hq, self.D, self.per_rank, self.group = rank, world, S, Hq, D, per_rank, group
        self.dev = x["q"].device
        self.on_gpu = x["q"].is_cuda
        self.names = ("q", "do", "qd", "dod")
        self.symm = None
        if world > 1 and use_symm and self.on_gpu and _peer_disabled is None:
            try:
                self.symm = _gather_buffers(self.dev, world, S, Hq, D, x["q"].dtype, group)
            except Exception as e:  # no symmetric memory in this process (every rank fails alike): use the collective
                globals()["_peer_disabled"] = f"{type(e).__name__}: {e}"
        self.full = None
        self.copy_stream = None

    def start(self):
        """Before the query-side kernels: send this rank's q-like rows on their way."""
        if self.world == 1:
            self.full = [self.x[n] for n in self.names]
            return
        n_loc, rows = self.S // self.world, self.Hq * self.D
        if self.symm is not None:
            buf, remote, flag = self.symm
            compute = torch.cuda.current_stream(self.dev)
            _stream_barrier(flag, self.group)  # every rank has finished the kernels that read the previous call's rows
            self.copy_stream = torch.cuda.Stream(device=self.dev, priority=_COPY_PRIORITY)
            self.copy_stream.wait_stream(compute)
            with torch.cuda.stream(self.copy_stream):
                for ti, n in enumerate(self.names):
                    src = self.x[n].contiguous().view(n_loc, rows)
                    # every rank starts with a different owner, so that at any time an owner receives from one source
                    for owner in ((self.rank + i) % self.world for i in range(1, self.world + 1)):
                        lo = 0
                        for a, b in self.chunks:
                            dst = remote[owner][(ti * self.S + a) * rows: (ti * self.S + b) * rows]
                            dst.copy_(src[lo:lo + b - a].reshape(-1), non_blocking=True)
                            lo += b - a
            self.full = [buf[ti][None] for ti in range(4)]
        else:  # collective fallback (CPU ranks; GPUs without symmetric memory): all-gather, then global row order
            mine = torch.stack([self.x[n].contiguous().view(n_loc, rows) for n in self.names])
            parts = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(parts, mine, group=self.group)
            perm = zigzag_permutation(self.S, self.world, self.per_rank, self.dev)
            allrows = torch.stack(parts, 1).reshape(4, self.S, rows).index_select(1, perm)
            self.full = [allrows[ti].view(1, self.S, self.Hq, self.D) for ti in range(4)]

    def exchange_stats(self):
        """After the JVP-forward kernel (which writes all four statistics): all-gather them, on a side stream
        of high priority, so that the wait for the slowest rank's forward and the collective's latency pass
        under this rank's dQ kernel."""
        self.stats, self.comm_stream = None, None
        if self.world == 1:
            self.stats = self.st_all
            return
        compute = None
        if self.on_gpu:
            compute = torch.cuda.current_stream(self.dev)
            self.comm_stream = torch.cuda.Stream(device=self.dev, priority=-1)
            self.comm_stream.wait_stream(compute)
            if self.copy_stream is not None:
                # this rank's copies have landed before its statistics leave: a rank that has received everybody's
                # statistics has therefore also received everybody's rows
                self.comm_stream.wait_stream(self.copy_stream)
        with (torch.cuda.stream(self.comm_stream) if self.comm_stream is not None else _NullCtx()):
            perm = zigzag_permutation(self.S, self.world, self.per_rank, self.dev)
            if dist.get_backend(self.group) == "nccl":
                parts = torch.empty((self.world,) + tuple(self.st_all.shape), dtype=torch.float32, device=self.dev)
                dist.all_gather_into_tensor(parts, self.st_all, group=_high_priority_group(self.group))
                parts = parts.permute(1, 2, 0, 3)
            else:
                parts = [torch.empty_like(self.st_all) for _ in range(self.world)]
                dist.all_gather(parts, self.st_all, group=self.group)
                parts = torch.stack(parts, 2)
            self.stats = parts.reshape(4, self.Hq, self.S).index_select(2, perm)
        if compute is not None:
            self.stats.record_stream(compute)  # allocated on the side stream, read by the dK/dV kernels on the compute stream

    def finish(self, k_like, scale):
        """After the dQ kernels: the dK/dV kernels of the own keys against all query rows."""
        _lib, N = self._lib, None
        tail_events = None
        if self.on_gpu:
            compute = torch.cuda.current_stream(self.dev)
            tail_events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            tail_events[0].record(compute)
            if self.comm_stream is not None:
                compute.wait_stream(self.comm_stream)
            tail_events[1].record(compute)
        q, do, qd, dod = self.full
        k, v, kd, vd = k_like
        flags = _lib.FB_FLAG_SEG_KEYS | _lib.DEFAULT_FLAGS
        prob = _lib.problem(q, k, None, None, None, None, scale, True, flags=flags, segments=zigzag_key_segments(self.chunks, self.S))
        out = {n: torch.empty_like(k) for n in _KV_NAMES}
        lse, z1, dpsum, ddot = self.stats
        args = (q, k, v, do, qd, kd, vd, dod, lse, dpsum, z1, ddot)
        _lib.hvp_bwd(prob, *args, N, out["dk"], out["dv"], N, N, N)
        _lib.hvp_bwd(prob, *args, N, N, N, N, out["dk_dot"], out["dv_dot"])
        return {"tail_events": tail_events, "kv_rows": list(self.chunks), **{n: t[0] for n, t in out.items()}}


def hvp_query_sharded(q, k, v, dout, q_dot, k_dot, v_dot, dout_dot=None, softmax_scale=None, causal=True,
                      rank: Optional[int] = None, world: Optional[int] = None, heads_per_group: Optional[int] = None, group=None,
                      exchange: Optional[str] = None, chunks_per_rank: Optional[int] = None, _emulated_peers=None):
    """Long-context partition (batch must be 1). K, V and their tangents are the full tensors on every
    rank. The q-like inputs (q, dout, q_dot, dout_dot) are either the full tensors too (every rank draws
    or receives the same data and reads only its zig-zag chunks) or already local: S / world rows, the
    rank's chunks one after the other (`zigzag_local`), which is how a zig-zag-sharded job holds them.

    A rank's chunks (`zigzag_chunks`; `chunks_per_rank` 2 or 4, default 4 where the chunk size allows)
    are ONE problem for the kernels: S / world query rows against keys [0, end of the last chunk), causal
    with query segments (fb_problem.seg_rows / seg_shift, `zigzag_segments`). Every kernel therefore runs
    once per rank (not once per chunk), the query tiles of all chunks balance each other inside one
    launch, and a key tile adds up all chunks' contributions in its accumulators before it is written.

    Two phases per call:
      1. query side, all heads at once: the JVP-forward and dQ / dQ_dot kernels;
      2. key side, head group by head group: the dK/dV kernels write float32 partial sums (no 16-bit round
         trip); the exchange of a group's dK, dV runs under its tangent kernels, that of its dK_dot,
         dV_dot under the next group's kernels. Two sets of partial buffers alternate between groups and
         are kept between calls.

    How the partial sums reach the ranks that own the key blocks (`exchange`):
      "copy": every rank owns a
             symmetric buffer with one slot per source rank; after a head group's kernels the group's key
             blocks are copied into the owners' slots by the copy engines (plain device-to-device copies on
             a side stream: they take no SM from the kernels of the next group), and after a stream
             barrier every rank adds up the slots it received with fb_sum_slots (fixed order:
             deterministic). Heads go in groups of a quarter so that only the last group's copies are exposed.
      "peer": the same slots, written from inside the kernels: every finished key tile goes straight into
             the owner's slot (fb_hvp_bwd_scatter), no partial buffers at all. Measured slower on 8 GPUs
             (the stores of a whole wave of CTAs hit NVLink at once while their SMs wait), kept as an option.
      "nccl": reduce-scatter on a side stream (the fallback, and what CPU ranks use).
      "gather" (default on GPUs with several ranks): no partial sums at all (`_QueryGather`): every rank receives all ranks' q-like rows (16-bit,
             sent by the copy engines while the query-side kernels run) and row statistics and computes
             the complete dK, dV, dK_dot, dV_dot of the keys of its OWN chunks (key segments). The results
             come in the I/O dtype for the rows "kv_rows" = the rank's chunks, not for a contiguous block.
    (`_emulated_peers = (slots of this rank, every rank's slots as addresses ["peer"] or as flat tensors
    ["copy"])` is for tests that run the ranks one after the other on one GPU: these paths without a
    process group; the result then carries "finish", to be called once every emulated rank has delivered,
    which adds up the slots.)

    Returns a dict: per chunk (a, b) the q-side results ("out", "out_dot", "dq", "dq_dot"; views of one
    local tensor per name, also under "local"), under "dk", "dv", "dk_dot", "dv_dot" this rank's key
    block [rank*S/world, (rank+1)*S/world) of the fully summed gradients, in float32 (with "gather": the
    keys of the rank's own chunks, see above; "kv_rows" lists the key ranges either way), and under
    "tail_events" two CUDA events that bracket the compute stream's final wait for the communication
    stream (their distance = exchange time that no kernel hid; None on CPU).
    """
    from . import _lib, interface as I

    rank = dist.get_rank(group) if rank is None else rank
    world = dist.get_world_size(group) if world is None else world
    if q.shape[0] != 1:
        raise ValueError("query-block sharding is for batch 1; use the (batch, kv-head) partition otherwise")
    Hq, D = q.shape[2], q.shape[3]
    S, Hkv = k.shape[1], k.shape[2]
    if not causal or q.shape[1] not in (S, S // world):
        raise ValueError("query-block sharding expects causal self-attention: q-like tensors with all S rows or the rank's S / world")
    if softmax_scale is None:
        softmax_scale = D ** -0.5
    G = Hq // Hkv
    if chunks_per_rank is None:
        chunks_per_rank = default_chunks_per_rank(S, world, q.is_cuda)
    chunks = zigzag_chunks(S, rank, world, chunks_per_rank)
    b1 = chunks[-1][1]      # keys this rank's queries can see
    n_loc = S // world      # its query rows
    segments = zigzag_segments(chunks)
    if segments and q.is_cuda and (S // (chunks_per_rank * world)) % 128:
        raise ValueError("a zig-zag chunk (S / (chunks per rank x world) rows) must be a multiple of 128 rows")
    keys_seen = lambda r: zigzag_chunks(S, r, world, chunks_per_rank)[-1][1]
    hg = default_heads_per_group(Hkv, world) if heads_per_group is None else max(1, min(heads_per_group, Hkv))
    while Hkv % hg:
        hg -= 1
    dev = q.device
    on_gpu = q.is_cuda
    N = None

    # ---- phase 1: query side, all heads, both chunks in one launch per kernel ----
    ql = (lambda t: t) if q.shape[1] != S or world == 1 else (lambda t: zigzag_local(t, chunks))  # world 1: the chunks are all rows
    qs = lambda t: None if t is None else I._rows(ql(t))
    ks = lambda t: I._rows(t[:, :b1])
    x = dict(q=qs(q), k=ks(k), v=ks(v), do=qs(dout), qd=qs(q_dot), kd=ks(k_dot), vd=ks(v_dot), dod=qs(dout_dot))
    st_all = torch.empty((4, Hq, n_loc), dtype=torch.float32, device=dev)
    st = list(st_all)  # lse, z1, dpsum, ddot: (Hq, rows)
    local = {n: torch.empty((1, n_loc, Hq, D), dtype=q.dtype, device=dev) for n in ("out", "out_dot", "dq", "dq_dot")}
    if exchange is None and _emulated_peers is None and on_gpu and world > 1:
        exchange = "gather"  # the fastest of the four on 2 and 4 B200s
    gather = None
    if exchange == "gather":
        gather = _QueryGather(_lib, x, st_all, chunks, rank, world, S, Hq, D, chunks_per_rank, group, use_symm=_emulated_peers is None)
        gather.start()
    prob = _lib.problem(x["q"], x["k"], None, None, None, None, softmax_scale, True, segments=segments)
    _lib.jvp_fwd(prob, x["q"], x["k"], x["v"], x["qd"], x["kd"], x["vd"], local["out"], local["out_dot"], st[0], st[1],
                 x["do"], x["dod"], st[2], st[3])
    if gather is not None:
        gather.exchange_stats()
    _lib.hvp_bwd(prob, x["q"], x["k"], x["v"], x["do"], x["qd"], x["kd"], x["vd"], x["dod"], st[0], st[2], st[1], st[3],
                 local["dq"], N, N, local["dq_dot"], N, N)
    q_side, lo = {}, 0
    for a, b in chunks:
        q_side[(a, b)] = {n: t[:, lo:lo + b - a] for n, t in local.items()}
        lo += b - a
    common = dict(chunks=chunks, q_side=q_side, local=local, kv_rows=[(rank * n_loc, (rank + 1) * n_loc)])
    if gather is not None:
        own = lambda t: I._rows(zigzag_local(t, chunks)).contiguous()
        return {**common, **gather.finish((own(k), own(v), own(k_dot), own(v_dot)), softmax_scale)}

    def dkv(hk, hq, flags, tangents, outs, scatter=None):
        """First-order (dK, dV) or tangent (dK_dot, dV_dot) kernel of head group (hk, hq): `outs` = the two
        float32 destinations (rows [0, b1)), or with `scatter` the two local marker tensors."""
        hq_ = lambda t: None if t is None else t[:, :, hq]
        hk_ = lambda t: t[:, :, hk]
        xq, xk = hq_(x["q"]), hk_(x["k"])
        pk = _lib.problem(xq, xk, None, None, None, None, softmax_scale, True, flags=flags, segments=segments)
        lse, z1, dpsum, ddot = (t[hq] for t in st)
        args = (xq, xk, hk_(x["v"]), hq_(x["do"]), hq_(x["qd"]), hk_(x["kd"]), hk_(x["vd"]), hq_(x["dod"]), lse, dpsum, z1, ddot)
        if scatter is not None:
            _lib.hvp_bwd_scatter(pk, scatter, *args, *((N, N) + outs if tangents else outs + (N, N)))
        else:
            _lib.hvp_bwd(pk, *args, *((N, N, N, N) + outs if tangents else (N,) + outs + (N, N, N)))

    barrier = None
    remote = None
    if _emulated_peers is not None:
        slots, peers = _emulated_peers
        if torch.is_tensor(peers[0]):
            exchange, remote = "copy", peers
        else:
            exchange, peer_ptrs = "peer", peers
    elif exchange is None:
        exchange = "copy" if (on_gpu and world > 1 and _peer_disabled is None) else "nccl"
    if exchange in ("peer", "copy") and _emulated_peers is None:
        try:
            slots, peer_ptrs, handle, flag = _peer_slots(dev, world, S // world, Hkv, D, group)
            barrier = lambda: _stream_barrier(flag, group)
        except Exception as e:  # no symmetric memory in this process (every rank fails alike): use the collective
            globals()["_peer_disabled"] = f"{type(e).__name__}: {e}"
            exchange = "nccl"
    if exchange == "copy":
        if heads_per_group is None:
            hg = max(1, Hkv // 4)
            while Hkv % hg:
                hg -= 1
        if remote is None:  # every rank's slot buffer as a flat tensor (this rank's own included)
            remote = [handle.get_buffer(o, (slots.numel(),), torch.float32, 0) for o in range(world)]
        res, finish = _key_side_copy(_lib, dkv, slots, remote, barrier, rank, world, S, keys_seen, Hkv, hg, G, D, _partial_sets(dev, S, hg, D))
    elif exchange == "peer":
        res, finish = _key_side_peer(_lib, dkv, slots, peer_ptrs, barrier, rank, world, S, keys_seen, Hkv, Hq, D)
    if exchange in ("copy", "peer"):
        res.update(common)
        if _emulated_peers is not None:
            res["finish"] = finish
            return res
        res.update(finish())
        return res

    # ---- phase 2, "nccl": key side, head group by head group, reduce-scatter overlapped ----
    sets = _partial_sets(dev, S, hg, D)
    kv_out = {n: torch.empty((S // world, Hkv, D), dtype=torch.float32, device=dev) for n in _KV_NAMES}
    compute = torch.cuda.current_stream(dev) if on_gpu else None
    comm_stream = torch.cuda.Stream(device=dev) if on_gpu else None
    set_free = [None, None]  # event: the exchanges that read this set of partial buffers have completed
    pending = []             # (name, head slice, shard, work)

    def reduce_scatter(names, partial, hk, last_of_set, si):
        """Reduce-scatter partial[n] for n in names on the communication stream, after everything
        enqueued so far on the compute stream."""
        shards = {n: (torch.empty((S // world, hg, D), dtype=torch.float32, device=dev) if world > 1 and on_gpu else None) for n in names}
        if comm_stream is not None:
            comm_stream.wait_stream(compute)
        with (torch.cuda.stream(comm_stream) if comm_stream is not None else _NullCtx()):
            for n in names:
                if world == 1:
                    kv_out[n][:, hk] = partial[n]  # nothing to exchange: the partial sums are the result
                    continue
                shard, work = _reduce_scatter_sum(partial[n], shards[n], world, rank, group)
                pending.append((n, hk, shard, work))
            if comm_stream is not None and last_of_set:
                set_free[si] = torch.cuda.Event()
                set_free[si].record(comm_stream)

    for gi, h0 in enumerate(range(0, Hkv, hg)):
        hk = slice(h0, h0 + hg)
        hq = slice(h0 * G, (h0 + hg) * G)
        si = gi % 2
        partial = sets[si]
        if on_gpu and set_free[si] is not None:
            compute.wait_event(set_free[si])  # the exchange of the group that used this set two groups ago
        elif not on_gpu:
            _drain(pending, kv_out)           # CPU ranks: collectives complete before their buffers are reused
        view = lambda n: partial[n][None, :b1]
        for n in _KV_NAMES:
            partial[n][b1:].zero_()           # keys past this rank's last query: it has nothing to add there
        dkv(hk, hq, _lib.FB_FLAG_KV_OUT_F32, False, (view("dk"), view("dv")))
        reduce_scatter(("dk", "dv"), partial, hk, False, si)
        dkv(hk, hq, _lib.FB_FLAG_KV_OUT_F32, True, (view("dk_dot"), view("dv_dot")))
        reduce_scatter(("dk_dot", "dv_dot"), partial, hk, True, si)

    tail_events = None
    if on_gpu:
        tail_events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        tail_events[0].record(compute)
    for n, hk, shard, work in pending:
        if work is not None:
            work.wait()
    if on_gpu:
        compute.wait_stream(comm_stream)
        tail_events[1].record(compute)
    _drain(pending, kv_out, wait=False)
    return {**common, "tail_events": tail_events, **kv_out}


def _key_side_copy(_lib, dkv, slots, remote, barrier, rank, world, S, keys_seen, Hkv, hg, G, D, sets):
    """Phase 2 of `hvp_query_sharded`, exchange by device-to-device copies into the owners' slots.
    Slot layout on every rank: [source rank][output][head group][key row of the block][head in group][D].
    Returns (dict with "tail_events", finish): finish() waits for every rank's copies (barrier) and adds
    up the slots this rank received; it returns the four key-block results."""
    n_k = S // world
    ngroups = Hkv // hg
    blk = n_k * hg * D                      # one (output, head group) block of a slot, in floats
    slot_elems = 4 * ngroups * blk          # = 4 * n_k * Hkv * D: one source rank's slot
    dev = slots.device
    compute = torch.cuda.current_stream(dev)
    copy_stream = torch.cuda.Stream(device=dev)  # (high priority measured no better here: 54.5 against 53.2-53.9 ms on 4 GPUs)
    b1 = keys_seen(rank)
    # what each source rank covers of each owner's block: source s saw keys [0, keys_seen(s))
    rows_from = lambda s, owner: max(0, min(n_k, keys_seen(s) - owner * n_k))
    if barrier is not None:
        barrier()  # every rank has added up the slots of the previous call before anybody copies into them again

    def send(names, partial, gi):
        """Copies this rank's partial key blocks of head group gi into every owner's slot for this rank."""
        copy_stream.wait_stream(compute)
        with torch.cuda.stream(copy_stream):
            for n in names:
                o_idx = _KV_NAMES.index(n)
                # every rank starts with a different owner, so that at any time an owner receives from one source
                for owner in ((rank + i) % world for i in range(1, world + 1)):
                    rows = rows_from(rank, owner)
                    if rows == 0:
                        continue
                    off = rank * slot_elems + (o_idx * ngroups + gi) * blk
                    src = partial[n][owner * n_k: owner * n_k + rows].reshape(-1)
                    remote[owner][off: off + rows * hg * D].copy_(src, non_blocking=True)

    set_free = [None, None]
    for gi, h0 in enumerate(range(0, Hkv, hg)):
        hk, hq = slice(h0, h0 + hg), slice(h0 * G, (h0 + hg) * G)
        si = gi % 2
        partial = sets[si]
        if set_free[si] is not None:
            compute.wait_event(set_free[si])  # the copies out of this set two groups ago
        view = lambda n: partial[n][None, :b1]
        for tangents, names in ((False, ("dk", "dv")), (True, ("dk_dot", "dv_dot"))):
            dkv(hk, hq, _lib.FB_FLAG_KV_OUT_F32, tangents, tuple(view(n) for n in names))
            send(names, partial, gi)
        set_free[si] = torch.cuda.Event()
        set_free[si].record(copy_stream)

    tail_events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
    tail_events[0].record(compute)
    compute.wait_stream(copy_stream)

    def finish():
        if barrier is not None:
            barrier()  # every rank's copies have landed
        kv = torch.empty((4, ngroups, n_k, hg, D), dtype=torch.float32, device=dev)
        valid = [rows_from(s, rank) * hg * D for s in range(world)]  # per (output, head group) block of a slot
        _lib.sum_slots(slots.view(world, slot_elems), kv.view(-1), valid, period=blk)
        out = {n: (kv[o, 0] if ngroups == 1 else kv[o].permute(1, 0, 2, 3).reshape(n_k, Hkv, D)) for o, n in enumerate(_KV_NAMES)}
        tail_events[1].record(torch.cuda.current_stream(dev))
        return out

    return {"tail_events": tail_events}, finish


_marker_cache = {}  # (device, heads, D) -> small float32 tensor that only says "this output is wanted"


def _key_side_peer(_lib, dkv, slots, peer_ptrs, barrier, rank, world, S, keys_seen, Hkv, Hq, D):
    """Phase 2 of `hvp_query_sharded` with the exchange fused into the kernels (all heads in one launch):
    every finished key tile is stored straight into its owner's slot, nothing is kept locally.
    Returns (dict with "tail_events", finish): finish() waits for every rank's stores (barrier) and adds
    up the slots this rank received; it returns the four key-block results."""
    n_k = S // world
    out_elems = n_k * Hkv * D          # one output's block in a slot
    slot_elems = 4 * out_elems         # one source rank's slot
    dev = slots.device
    if barrier is not None:
        barrier()  # every rank has added up the slots of the previous call before anybody writes into them again

    def dst(o):  # my slot, output o, on every peer
        return [p + 4 * (rank * slot_elems + o * out_elems) for p in peer_ptrs]

    key = (str(dev), Hkv, D)
    if key not in _marker_cache:
        _marker_cache[key] = torch.zeros((1, 128, Hkv, D), dtype=torch.float32, device=dev)
    marker = _marker_cache[key]  # without accumulation the local tensors are not touched: their presence selects the outputs
    sc = _lib.kv_scatter(world, n_k, Hkv * D, D, dk=dst(0), dv=dst(1), dk_dot=dst(2), dv_dot=dst(3))
    for tangents in (False, True):
        dkv(slice(0, Hkv), slice(0, Hq), _lib.FB_FLAG_KV_OUT_F32, tangents, (marker, marker), scatter=sc)
    compute = torch.cuda.current_stream(dev)
    tail_events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
    tail_events[0].record(compute)

    def finish():
        if barrier is not None:
            barrier()  # every rank's stores have landed
        # source rank s saw keys [0, keys_seen(s)): rows of my block beyond that were not written
        valid = [max(0, min(n_k, keys_seen(s) - rank * n_k)) * Hkv * D for s in range(world)]
        kv = torch.empty((4, n_k, Hkv, D), dtype=torch.float32, device=dev)
        for o in range(4):
            _lib.sum_slots(slots[:, o], kv[o], valid)
        tail_events[1].record(torch.cuda.current_stream(dev))
        return {n: kv[o] for o, n in enumerate(_KV_NAMES)}

    return {"tail_events": tail_events}, finish


def _drain(pending, kv_out, wait=True):
    """Copies finished key blocks into the result tensors (waiting for their collectives first)."""
    for n, hk, shard, work in pending:
        if wait and work is not None:
            work.wait()
        kv_out[n][:, hk] = shard
    pending.clear()


class _NullCtx:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False

"""world_size-2 tests of the multi-GPU drivers on CPU ranks (gloo). Device calls are replaced by
tests/fake_backend.py; what is tested is the partitioning, the zig-zag causal chunking and the
reduce-scatter of partial dK/dV."""

import os
import socket
import sys
import traceback
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _inputs(B, S, Hq, Hkv, D):
    g = torch.Generator().manual_seed(0)
    r = lambda h: torch.randn(B, S, h, D, generator=g, dtype=torch.float64)
    return r(Hq), r(Hkv), r(Hkv), r(Hq), r(Hq), r(Hkv), r(Hkv), r(Hq)  # q k v dout qd kd vd doutd


def _worker(rank, world, port, q_out):
    try:
        for p in (str(ROOT), str(ROOT / "flashback-cute_b200")):
            if p not in sys.path:
                sys.path.insert(0, p)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from flashback_cute import parallel
        from oracle import attention_oracle as orc
        from tests import fake_backend

        names = ("out", "out_dot", "dq", "dk", "dv", "dq_dot", "dk_dot", "dv_dot")
        with fake_backend.installed():
            # (batch, kv-head) partition, GQA, no communication
            B, S, Hq, Hkv, D = 2, 24, 4, 2, 8
            q, k, v, do, qd, kd, vd, dod = _inputs(B, S, Hq, Hkv, D)
            ref = orc.attention_hvp_dense(q, k, v, 0.3, True, qd, kd, vd, do, dod)
            res, (bs, hs) = parallel.hvp_head_sharded(q, k, v, do, qd, kd, vd, dod, 0.3, True)
            for n, got in zip(names, res):
                want = parallel.shard_by_group(getattr(ref, n), bs, hs, Hkv)
                assert torch.allclose(got, want, atol=1e-10), n
            # heads split inside one batch
            B2 = 1
            q, k, v, do, qd, kd, vd, dod = _inputs(B2, S, Hq, Hkv, D)
            ref = orc.attention_hvp_dense(q, k, v, 0.3, False, qd, kd, vd, do, dod)
            res, (bs, hs) = parallel.hvp_head_sharded(q, k, v, do, qd, kd, vd, dod, 0.3, False)
            assert (hs.stop - hs.start) == 1
            for n, got in zip(names, res):
                assert torch.allclose(got, parallel.shard_by_group(getattr(ref, n), bs, hs, Hkv), atol=1e-10), n

            # long-context partition: zig-zag query chunks + reduce-scatter of partial dK/dV
            S = 32
            q, k, v, do, qd, kd, vd, dod = _inputs(1, S, Hq, Hkv, D)
            ref = orc.attention_hvp_dense(q, k, v, 0.3, True, qd, kd, vd, do, dod)
            for per_rank in (2, 4):
                r = parallel.hvp_query_sharded(q, k, v, do, qd, kd, vd, dod, 0.3, True, heads_per_group=1, chunks_per_rank=per_rank)
                assert r["chunks"] == parallel.zigzag_chunks(S, rank, world, per_rank) and len(r["chunks"]) == per_rank
                for (a, b), d in r["q_side"].items():
                    for n in ("out", "out_dot", "dq", "dq_dot"):
                        assert torch.allclose(d[n], getattr(ref, n)[:, a:b], atol=1e-10), (n, a, b)
                n_k = S // world
                for n in ("dk", "dv", "dk_dot", "dv_dot"):
                    want = getattr(ref, n)[0, rank * n_k:(rank + 1) * n_k]
                    assert torch.allclose(r[n].double(), want, atol=1e-5), n  # partial sums travel in float32
            # no partial sums: every rank gathers all query-side rows and owns the keys of its chunks
            for per_rank in (2, 4):
                r = parallel.hvp_query_sharded(q, k, v, do, qd, kd, vd, dod, 0.3, True, chunks_per_rank=per_rank, exchange="gather")
                assert r["kv_rows"] == parallel.zigzag_chunks(S, rank, world, per_rank)
                for (a, b), d in r["q_side"].items():
                    for n in ("out", "out_dot", "dq", "dq_dot"):
                        assert torch.allclose(d[n], getattr(ref, n)[:, a:b], atol=1e-10), (n, a, b)
                for n in ("dk", "dv", "dk_dot", "dv_dot"):
                    want = torch.cat([getattr(ref, n)[0, a:b] for a, b in r["kv_rows"]])
                    assert torch.allclose(r[n], want, atol=1e-5), n  # the row statistics travel in float32
            r = parallel.hvp_query_sharded(q, k, v, do, qd, kd, vd, dod, 0.3, True, heads_per_group=1, chunks_per_rank=4)
            # the rank's own rows only (how a zig-zag-sharded job holds its q-like tensors): same results
            mine = [parallel.zigzag_local(t, r["chunks"]).contiguous() for t in (q, do, qd, dod)]
            r2 = parallel.hvp_query_sharded(mine[0], k, v, mine[1], mine[2], kd, vd, mine[3], 0.3, True, heads_per_group=1, chunks_per_rank=4)
            for n in ("out", "out_dot", "dq", "dq_dot"):
                assert torch.equal(r2["local"][n], r["local"][n]), n
        dist.barrier()
        dist.destroy_process_group()
        q_out.put((rank, "ok"))
    except Exception:
        q_out.put((rank, traceback.format_exc()))


def test_two_rank_partitions_match_single_process():
    world = 2
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q_out)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q_out.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}:\n{msg}"


def test_group_slices_cover_all_groups_once():
    from flashback_cute import parallel

    for B, Hkv, world in [(2, 8, 1), (2, 8, 2), (2, 8, 4), (2, 8, 8), (2, 8, 16), (4, 16, 8), (8, 32, 8), (1, 16, 8)]:
        seen = set()
        for r in range(world):
            bs, hs = parallel.group_slices(B, Hkv, r, world)
            for b in range(bs.start, bs.stop):
                for h in range(hs.start, hs.stop):
                    assert (b, h) not in seen
                    seen.add((b, h))
        assert len(seen) == B * Hkv
    with pytest.raises(ValueError):
        parallel.group_slices(2, 3, 0, 4)


def test_zigzag_chunks_balance_causal_work():
    from flashback_cute import parallel

    S, world = 1024, 8
    work = []
    for r in range(world):
        ch = parallel.zigzag_chunks(S, r, world)
        assert len(ch) == 2
        work.append(sum((b * (b + 1) - a * (a + 1)) // 2 for a, b in ch))  # visible (query, key) pairs
    assert max(work) - min(work) <= S  # balanced to within one row's worth of keys per chunk pair
    rows = sorted(x for r in range(world) for a, b in parallel.zigzag_chunks(S, r, world) for x in range(a, b))
    assert rows == list(range(S))
    # four chunks per rank: the same balance, every row once, ascending chunks
    work4 = []
    for r in range(world):
        ch = parallel.zigzag_chunks(S, r, world, 4)
        assert len(ch) == 4 and ch == sorted(ch)
        work4.append(sum((b * (b + 1) - a * (a + 1)) // 2 for a, b in ch))
    assert max(work4) - min(work4) <= 2 * S
    rows = sorted(x for r in range(world) for a, b in parallel.zigzag_chunks(S, r, world, 4) for x in range(a, b))
    assert rows == list(range(S))


def test_zigzag_segments_place_every_local_row_at_its_global_position():
    """zigzag_segments' (break, shift) pairs, read the way the kernels read fb_problem.seg_rows / seg_shift
    (position of local row i = i + seqlen_k - seqlen_q - shift of its segment), give back the chunks."""
    from flashback_cute import parallel

    for S, world, per_rank in ((1024, 4, 2), (2048, 4, 4), (4096, 8, 4), (512, 1, 4), (512, 2, 2)):
        for r in range(world):
            ch = parallel.zigzag_chunks(S, r, world, per_rank)
            segs = parallel.zigzag_segments(ch)
            assert len(segs) <= 3 and [b for b, _ in segs] == sorted(b for b, _ in segs)
            assert all(s1 >= s2 >= 0 for (_, s1), (_, s2) in zip(segs, segs[1:] + [(0, 0)]))
            n_loc, sk = S // world, ch[-1][1]
            pos = []
            for i in range(n_loc):
                shift = next((sh for brk, sh in segs if i < brk), 0)
                pos.append(i + sk - n_loc - shift)
            assert pos == [x for a, b in ch for x in range(a, b)], (S, world, per_rank, r)


def test_zigzag_key_segments_place_every_local_key_at_its_global_position():
    """zigzag_key_segments' (break, shift) pairs, read the way the kernels read them with FB_FLAG_SEG_KEYS
    (position of local key j against `seqlen` query rows = j + seqlen_q - seqlen_k - shift of its segment),
    give back the chunks; and zigzag_permutation finds every global row in the rank-major concatenation."""
    import torch

    from flashback_cute import parallel

    for S, world, per_rank in ((1024, 4, 2), (2048, 4, 4), (4096, 8, 4), (512, 1, 4), (512, 2, 2)):
        n_loc = S // world
        order = []
        for r in range(world):
            ch = parallel.zigzag_chunks(S, r, world, per_rank)
            order += [x for a, b in ch for x in range(a, b)]
            segs = parallel.zigzag_key_segments(ch, S)
            assert len(segs) <= 4 and [b for b, _ in segs] == sorted(b for b, _ in segs)
            assert all(s1 >= s2 >= 0 for (_, s1), (_, s2) in zip(segs, segs[1:] + [(0, 0)]))
            pos = []
            for j in range(n_loc):
                shift = next((sh for brk, sh in segs if j < brk), 0)
                pos.append(j + S - n_loc - shift)
            assert pos == [x for a, b in ch for x in range(a, b)], (S, world, per_rank, r)
        perm = parallel.zigzag_permutation(S, world, per_rank, "cpu")
        assert torch.equal(torch.tensor(order)[perm], torch.arange(S))


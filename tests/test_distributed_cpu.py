"""Host-side logic of the multi-GPU paths, run as two gloo ranks on CPU: partition plans,
output gather, candidate exchange + deterministic global top-k, partial exchange."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from thriftattention_b200 import distributed as tad


def test_head_shard_plan():
    shards = tad.plan_head_shards(32, 8, 4)
    assert [(s.kv_begin, s.kv_end, s.q_begin, s.q_end) for s in shards] == [(0, 2, 0, 8), (2, 4, 8, 16), (4, 6, 16, 24), (6, 8, 24, 32)]
    with pytest.raises(ValueError):
        tad.plan_head_shards(32, 8, 3)
    q, k, v = torch.arange(32).view(1, 32, 1, 1), torch.arange(8).view(1, 8, 1, 1), torch.arange(8).view(1, 8, 1, 1)
    ql, kl, _ = tad.shard_heads(q, k, v, shards[2])
    assert ql.flatten().tolist() == list(range(16, 24)) and kl.flatten().tolist() == [4, 5]


def test_page_shard_plan_covers_every_page_once():
    for n, w in ((2048, 8), (2047, 4), (5, 8), (64, 1), (100, 3), (700, 5), (64, 4)):
        shards = tad.plan_page_shards(n, w)
        assert shards[0].page_begin == 0 and shards[-1].page_end == n
        assert all(a.page_end == b.page_begin for a, b in zip(shards, shards[1:]))
        assert sum(s.num_pages for s in shards) == n
        assert all(s.page_begin % 32 == 0 for s in shards if s.num_pages)       # the tie-break needs aligned starts
    assert [s.num_pages for s in tad.plan_page_shards(2048, 8)] == [256] * 8
    assert [(s.page_begin, s.page_end) for s in tad.plan_page_shards(100, 3)] == [(0, 32), (32, 64), (64, 100)]
    assert [s.num_pages for s in tad.plan_page_shards(64, 4)] == [32, 0, 32, 0]   # fewer than 32 pages per rank: empty shards


def test_local_cut_then_merge_resolves_exact_ties_like_the_global_rule():
    """Every score equal: each shard keeps its top c by the tie-break on LOCAL ids (what the selection kernel does),
    the merge ranks the union by the tie-break on global ids.  With shard starts at multiples of 32 that is the
    global rule's own answer; an unaligned start (the even split of 100 pages over 3 ranks starts a shard at 33)
    loses a page the global rule keeps."""
    n, k = 100, 7
    want = tad.merge_topk_candidates(torch.zeros(1, n), torch.arange(n, dtype=torch.int32).view(1, n), k)

    def via_shards(bounds):
        parts = []
        for lo, hi in bounds:
            m = hi - lo
            local = tad.merge_topk_candidates(torch.zeros(1, m), torch.arange(m, dtype=torch.int32).view(1, m), min(k, m))
            parts.append(local + lo)
        pages = torch.cat(parts, 1)
        return tad.merge_topk_candidates(torch.zeros(1, pages.shape[1]), pages, k)

    aligned = [(s.page_begin, s.page_end) for s in tad.plan_page_shards(n, 3)]
    assert torch.equal(via_shards(aligned), want)
    assert not torch.equal(via_shards([(0, 33), (33, 66), (66, 100)]), want)


def test_merge_topk_candidates_matches_global_topk_and_kernel_tie_order():
    g = torch.Generator().manual_seed(0)
    scores = torch.randn(6, 256, generator=g)
    pages = torch.arange(256, dtype=torch.int32).repeat(6, 1)
    # per-shard top-k then merge == global top-k
    k = 9
    parts_s, parts_p = [], []
    for sh in tad.plan_page_shards(256, 4):
        t = torch.topk(scores[:, sh.page_begin:sh.page_end], k, dim=1)
        parts_s.append(t.values)
        parts_p.append((t.indices + sh.page_begin).to(torch.int32))
    merged = tad.merge_topk_candidates(torch.cat(parts_s, 1), torch.cat(parts_p, 1), k)
    assert torch.equal(merged.long(), torch.topk(scores, k, dim=1).indices)
    # exact ties: smallest bit-reversed (page mod 32) first, then the smaller page
    s = torch.zeros(1, 64)
    p = torch.arange(64, dtype=torch.int32).view(1, 64)
    assert tad.merge_topk_candidates(s, p, 6).tolist() == [[0, 32, 16, 48, 8, 40]]
    # padding entries never win
    p2 = p.clone(); p2[0, :60] = -1
    assert sorted(tad.merge_topk_candidates(s, p2, 6).tolist()[0]) == [-1, -1, 60, 61, 62, 63]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # output gather: rank r holds heads [2r, 2r+2)
        local = torch.full((1, 2, 3, 4), float(rank)) + torch.arange(2).view(1, 2, 1, 1) * 0.5
        full = tad.gather_heads(local)
        ok1 = full.shape == (1, 4, 3, 4) and full[0, :, 0, 0].tolist() == [0.0, 0.5, 1.0, 1.5]
        # candidate exchange + global selection is identical on both ranks and equals the global top-k
        g = torch.Generator().manual_seed(7)
        scores = torch.randn(3, 40, generator=g)
        sh = tad.plan_page_shards(40, world)[rank]
        t = torch.topk(scores[:, sh.page_begin:sh.page_end], 5, dim=1)
        s_all, p_all = tad.exchange_candidates(t.values.contiguous(), (t.indices + sh.page_begin).to(torch.int32).contiguous())
        sel = tad.merge_topk_candidates(s_all, p_all, 5)
        ok2 = torch.equal(sel.long(), torch.topk(scores, 5, dim=1).indices)
        # partial exchange keeps shard order
        po = torch.full((2, 1, 4, 8), float(rank))
        pml = torch.full((2, 1, 4, 2), float(rank))
        ao, aml = tad.exchange_partials(po, pml)
        ok3 = ao.shape == (world, 2, 1, 4, 8) and ao[:, 0, 0, 0, 0].tolist() == [0.0, 1.0] and aml.shape == (world, 2, 1, 4, 2)
        q.put((rank, bool(ok1), bool(ok2), bool(ok3)))
    except Exception as exc:  # report instead of leaving the parent waiting
        q.put((rank, repr(exc), False, False))
    finally:
        dist.destroy_process_group()


def test_two_rank_exchange_over_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=90) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True, True, True), (1, True, True, True)]


def _silent_peer_worker(rank, world, port, q):
    """Rank 1 joins the group and then never takes part in the exchange; rank 0 must get an error, not a hang."""
    import datetime
    import time

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    try:
        if rank == 1:
            time.sleep(8)                      # alive, but silent, for longer than the group's timeout
            q.put((rank, "silent"))
            return
        po = torch.zeros(2, 1, 4, 8)
        pml = torch.zeros(2, 1, 4, 2)
        t0 = time.time()
        try:
            tad.exchange_partials(po, pml)
            q.put((rank, "returned"))
        except Exception as exc:               # the collective gives up after the group's timeout
            q.put((rank, f"error after {time.time() - t0:.0f}s: {type(exc).__name__}"))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:                      # the group is broken on the rank that timed out
            pass


def test_a_rank_that_never_sends_its_partials_is_an_error_on_its_peer_not_a_hang():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_silent_peer_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        results = dict(q.get(timeout=60) for _ in procs)
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    assert results[1] == "silent"
    assert results[0].startswith("error after"), results[0]

#!/usr/bin/env python
"""Headline benchmark: long-context selective mixed-precision prefill attention, and the paged decode step.

Workload of the headline metric ("prefill attn TFLOP/s @128k top-10% NVFP4; decode us/step & HBM GB/s @128k"):
batch 1, 32 query heads / 8 KV heads, q_len = kv_len = 131072, head_dim 128, fp16, causal, Quest selection with
128-token blocks keeping top-10% (53 of 1024 blocks) in 16-bit and the rest in NVFP4; q, v ~ N(0,1), k ~ N(0,1)
with 4 fixed channels per KV head scaled x10 (seeded, synthetic).  One step = ``ta.attention(q, k, v, config=...)``:
block statistics + selection + quantisation of Q/K/V + the fused attention kernel over the whole problem.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload headline|mxfp4-bf16]

N > 1 (launched under torch.distributed.run): the 8 KV-head groups are split across the ranks (strong scaling, no
communication during compute; the outputs are all-gathered on a side stream, two q-row ranges per step, so that the
gather of the first range runs under the kernel of the second).  ``--workload mxfp4-bf16 --fraction F`` runs the
long-context bf16 / MXFP4 configuration with F of the blocks in bf16 instead (prefill only).
``--impl reference`` times the CPU oracle (the restatement of the reference's arithmetic) on the host cores on a
bounded sample of the same workload, and runs the small CPU configuration (8 heads x 2048 tokens) in full.

Rank 0 prints one JSON line.
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

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HQ, HKV, SEQ, D = 32, 8, 131072, 128
BLOCK = 128
METRIC = "prefill_attention_tflops_128k_top10pct_nvfp4"
FP4_TO_BF16_PEAK_RATIO = 4.0  # dense FP4 : dense bf16 tensor peak on B200 (9 : 2.25 PFLOP/s nominal)
# DRAM bytes of one prefill_kernel launch over all 32 q heads of the timed workload: dram__bytes_read.sum (4.23 GB) +
# dram__bytes_write.sum (1.31 GB) of a one-pass ncu capture of this very command (summarised under profiles/).  A rank
# of an N-GPU run, a q-head chunk or a KV-head group launch processes a share of the heads and moves that share of
# the bytes (every head's work is the same), so the figure is scaled by the FLOPs of the launch.
BENCH_DRAM_BYTES, BENCH_FLOPS = 5.54e9, 1.4093e14


def algorithmic_flops(hq: int, seq: int, d: int, block: int) -> float:
    """4 * D * Hq * sum_i (i + 1) * block^2 over q blocks (block-granular causal)."""
    nb = seq // block
    return 4.0 * d * hq * (nb * (nb + 1) // 2) * block * block


def fp16_flop_share(seq: int, block: int, k: int) -> float:
    nb = seq // block
    return sum(min(i + 1, k) for i in range(nb)) / (nb * (nb + 1) / 2)


def call_stats(times_ms) -> dict:
    """mean / median / p90 / min of per-call CUDA-event times (the reference harness's columns,
    benchmarks/run_kernel_benchmarks.py:282-303)."""
    t = sorted(times_ms)
    pos = (len(t) - 1) * 0.9
    lo = int(pos)
    p90 = t[lo] + (t[min(lo + 1, len(t) - 1)] - t[lo]) * (pos - lo)
    return {"mean": statistics.fmean(t), "median": statistics.median(t), "p90": p90, "min": t[0], "n": len(t)}


def measured_peaks() -> dict:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f)
    except (OSError, ValueError):
        return {}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                smax = float(parts[1])
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        busy = [x for x in sm if smax is None or x > 0.3 * smax] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm)}


def make_inputs(hq: int, hkv: int, seq: int, device, dtype, seed: int = 0, kv_head_offset: int = 0, total_hkv: int = HKV):
    """Seeded synthetic q, k, v; K gets 4 fixed outlier channels per KV head (x10)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    channels = torch.stack([torch.randperm(D, generator=g)[:4] for _ in range(total_hkv)])  # [total_hkv, 4]
    gd = torch.Generator(device=device).manual_seed(seed + 1 + kv_head_offset)
    q = torch.randn(1, hq, seq, D, device=device, dtype=dtype, generator=gd)
    k = torch.randn(1, hkv, seq, D, device=device, dtype=dtype, generator=gd)
    v = torch.randn(1, hkv, seq, D, device=device, dtype=dtype, generator=gd)
    for h in range(hkv):
        k[0, h, :, channels[kv_head_offset + h].to(device)] *= 10
    return q, k, v


def run_small_cpu_config(cores: int) -> dict:
    """The CPU-runnable configuration in full: batch 1, 8 query = 8 KV heads, 2048 tokens, head_dim 128, q, k, v ~
    N(0,1) from seed 0, causal, 64-token blocks, top-10 % (2 of 32 blocks) + the first block (sink) + the newest block
    (local) in 16 bits, the rest NVFP4 - oracle output against fp32 softmax attention, with the oracle's wall time."""
    import oracle

    torch.manual_seed(0)
    q32, k32, v32 = (torch.randn(1, 8, 2048, D) for _ in range(3))
    q, k, v = q32.half(), k32.half(), v32.half()
    top_k = oracle.resolve_top_k(2048 // 64, causal=True, fraction=0.10)
    t0 = time.perf_counter()
    qm, = oracle.block_stats(q, 64, ("mean",))
    km, = oracle.block_stats(k, 64, ("mean",))
    sel = oracle.select_prefill(qm, km, None, k=top_k, causal=True, sink=1, local=1)
    out = oracle.prefill_attention(q, k, v, sel, fmt="nvfp4", block=64, causal=True)
    dt = time.perf_counter() - t0
    exact = torch.nn.functional.scaled_dot_product_attention(q32, k32, v32, is_causal=True)
    err = (out.float() - exact).abs()
    cos = torch.nn.functional.cosine_similarity(out.float().flatten(), exact.flatten(), dim=0).item()
    return {"workload": "1x8q/8kv x2048 x128, causal, block-mean top-10% (2 of 32 64-token blocks) + sink 1 + local 1 in "
                        "f16, rest NVFP4; CPU oracle vs fp32 softmax attention",
            "top_k": top_k, "wall_s": dt, "cores": cores, "max_abs_err": err.max().item(), "mean_abs_err": err.mean().item(),
            "cosine": cos}


def run_reference(args) -> dict:
    """CPU arm: the oracle (a port of the reference's arithmetic) on a bounded sample of the headline workload."""
    import oracle

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return {}
    cores = os.cpu_count() or 1
    os.environ.setdefault("OMP_NUM_THREADS", str(cores))
    torch.set_num_threads(cores)
    rows = 4096  # the last 4096 query rows of one q head against all 131072 keys of its KV head
    q, k, v = make_inputs(1, 1, SEQ, "cpu", torch.float16)
    top_k = oracle.resolve_top_k(SEQ // BLOCK, causal=True, fraction=0.10)

    def step():
        qm, = oracle.block_stats(q, BLOCK, ("mean",))
        kmin, kmax = oracle.block_stats(k, BLOCK, ("min", "max"))
        sel = oracle.select_prefill(qm, kmin, kmax, k=top_k, causal=True)
        return oracle.prefill_attention(q, k, v, sel, fmt="nvfp4", block=BLOCK, causal=True, rows=(SEQ - rows, SEQ))

    nb, r0 = SEQ // BLOCK, (SEQ - rows) // BLOCK
    pairs = sum(i + 1 for i in range(r0, nb))
    sample_flops = 4.0 * D * pairs * BLOCK * BLOCK
    for _ in range(max(0, min(args.warmup, 1))):
        step()
    steps = max(1, min(args.steps, 3))
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    value = sample_flops / dt / 1e12
    sample = (f"last {rows} query rows of 1 of {HQ} q heads vs all {SEQ} keys of its KV head (statistics, selection, "
              f"quantisation of that head and mixed attention), {sample_flops:.3e} of {algorithmic_flops(HQ, SEQ, D, BLOCK):.3e} FLOP")
    result = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": min(args.warmup, 1), "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "fp4+f16 (emulated in fp32 on CPU)", "data": "synthetic",
        "config": {"workload": "prefill 1x32q/8kv x131072 x128 fp16 causal, Quest top-10% of 128-token blocks, NVFP4",
                   "sample": sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    if getattr(args, "with_small_cpu_config", True):
        result["cpu_config"] = run_small_cpu_config(cores)
    return result


# --------------------------------------------------------------------------------------------- decode leg
DEC_BATCH, DEC_SEQ, DEC_GROUP = 32, 131072, HQ // HKV
DEC_SINK, DEC_LOCAL, DEC_FRACTION = 4, 16, 0.10
DEC_CHECK_ROWS = ((0, 0), (DEC_BATCH - 1, HKV - 1))       # (sequence, KV head) pairs compared with the oracle
CHECK_MAX_ABS, CHECK_MEAN_ABS = 2e-3, 2e-4               # the fp16 attention tolerance of the parity tests


def check_decode_rows(out, q, k_hi, v_hi, table, *, world: int, rank: int, pages: int, top_k: int, splits_local: int) -> str:
    """Rank 0 compares DEC_CHECK_ROWS of the step's result with the CPU oracle run on the same cached K/V (the
    16-bit shadow in logical page order, gathered from all ranks; the oracle quantises it exactly as the cache was
    filled).  A shard's chains are the single-GPU chains of the same page ranges, so the oracle runs with
    world x splits_local chains.  Raises on a mismatch."""
    import torch.distributed as dist

    import oracle

    worst = 0.0
    for b, h in DEC_CHECK_ROWS:
        idx = table[b].long()
        mine = [k_hi[idx, h].contiguous(), v_hi[idx, h].contiguous()]            # [n_local, 64, D] each
        if world > 1:
            parts = []
            for t in mine:
                bufs = [torch.empty_like(t) for _ in range(world)]
                dist.all_gather(bufs, t)
                parts.append(torch.cat(bufs, 0))
        else:
            parts = mine
        if rank != 0:
            continue
        k_row = parts[0].reshape(1, 1, pages * 64, D).cpu()
        v_row = parts[1].reshape(1, 1, pages * 64, D).cpu()
        q_row = q[b, h].reshape(1, 1, DEC_GROUP, D).cpu()
        lo, hi = oracle.block_stats(k_row, 64, ("min", "max"))
        sel = oracle.select_decode(q_row, lo, hi, k=top_k, num_kv_blocks=pages, sink=DEC_SINK, local=DEC_LOCAL)
        ref = oracle.decode_attention(q_row, k_row, v_row, sel, fmt="nvfp4", splits=world * splits_local)
        err = (out[b, h].float().cpu() - ref[0, 0].float()).abs()
        if not (err.max().item() <= CHECK_MAX_ABS and err.mean().item() <= CHECK_MEAN_ABS):
            raise RuntimeError(f"decode check failed for (sequence {b}, KV head {h}): max-abs {err.max().item():.3e}, "
                               f"mean-abs {err.mean().item():.3e} against the CPU oracle")
        worst = max(worst, err.max().item())
    return f"ok ({len(DEC_CHECK_ROWS)} (sequence, KV head) rows vs CPU oracle, max-abs {worst:.1e} <= {CHECK_MAX_ABS:g})"


def run_decode_leg(device, world: int, rank: int, steps: int, warmup: int, hbm_gbs: float) -> dict:
    """Second half of the headline metric: one paged decode step for 32 sequences of 131072 cached tokens
    (64-token pages through a seeded random page table, NVFP4 codes quantised from the fp16 shadow that holds the
    selected pages, Quest top-10 % + 4 sink + 16 recent pages).  A step = quantise q + page selection + split-KV
    attention + merge.  With N GPUs every sequence's pages are split N ways (KV-sequence sharding):
    kernel-scored candidates and partial results are exchanged with two all-gathers per step.  Returns
    microseconds per step, whole-job algorithmic GB/s and the outcome of the oracle check."""
    import torch.distributed as dist

    from thriftattention_b200 import _C
    from thriftattention_b200 import distributed as tad

    pages = DEC_SEQ // 64
    shard = tad.plan_page_shards(pages, world)[rank]
    n_local = shard.num_pages
    top_k = max(1, round(DEC_FRACTION * pages))
    pool = DEC_BATCH * n_local
    g = torch.Generator(device=device)
    g.manual_seed(1234 + rank)
    # the cache: fp16 shadow pools, their NVFP4 quantisation in the pool layouts, per-page key minima / maxima
    k_hi = torch.empty(pool, HKV, 64, D, dtype=torch.float16, device=device).normal_(generator=g)
    v_hi = torch.empty(pool, HKV, 64, D, dtype=torch.float16, device=device).normal_(generator=g)
    k4, ks = _C.nvfp4_quantize(k_hi)                                   # [pool, HKV, 64, D/2], [.., D/16]
    v4p, vsp = _C.nvfp4_quantize_transposed(v_hi)                      # padded to 128 tokens per page
    v4, vs = v4p[..., :32].contiguous(), vsp[..., :4].contiguous()     # [pool, HKV, D, 32], [pool, HKV, D, 4]
    del v4p, vsp
    _, pmin, pmax = _C.block_stats(k_hi, 64, minmax=True)              # [pool, HKV, 1, D]
    table = torch.randperm(pool, generator=g, device=device).to(torch.int32).reshape(DEC_BATCH, n_local)
    k_min = pmin[table.long(), :, 0].permute(0, 2, 1, 3).contiguous()  # [B, HKV, n_local, D] in logical page order
    k_max = pmax[table.long(), :, 0].permute(0, 2, 1, 3).contiguous()
    del pmin, pmax
    gq = torch.Generator(device=device)
    gq.manual_seed(99)                                                             # the query is replicated
    q = torch.empty(DEC_BATCH, HKV, DEC_GROUP, D, dtype=torch.float16, device=device).normal_(generator=gq)
    splits_local = max(1, min(_C.decode_pick_splits(DEC_BATCH * HKV, n_local), n_local))
    # The two exchanges of a sharded step (page candidates, one partial per head: < 1 MB each) go through the process
    # group's all-gather, or with TA100_BENCH_EXCHANGE=peer through the library's own peer-memory kernel.
    exchange, exchange_kind = None, "none (one GPU)"
    if world > 1:
        exchange_kind = "nccl all_gather"
        if os.environ.get("TA100_BENCH_EXCHANGE", "nccl") == "peer":
            try:
                exchange = tad.PeerExchange(1 << 20, device=device)
                exchange_kind = "peer stores over NVLink (ta100_peer_all_gather)"
            except Exception as exc:                              # noqa: BLE001 - any refusal means the collective
                if rank == 0:
                    print(f"peer exchange not available ({type(exc).__name__}: {exc}); using NCCL", file=sys.stderr)
        ready = torch.tensor([1 if exchange is not None else 0], device=device)
        dist.all_reduce(ready, op=dist.ReduceOp.MIN)              # all ranks or none
        if ready.item() == 0:
            exchange, exchange_kind = None, "nccl all_gather"

    def step():
        q4, qs = _C.nvfp4_quantize(q)
        if world == 1:
            sel = _C.select_decode_blocks(q, k_min, k_max, top_k, pages, False, sink=DEC_SINK, local=DEC_LOCAL)
            return _C.decode_attention(q, k_hi, v_hi, sel, q4, k4, v4, qs, ks, vs, is_mx=False, is_bf16=False,
                                       kv_len=n_local * 64, page_table=table, allow_padded_selection=True)
        sel = tad.select_pages_sharded(q, k_min, k_max, shard=shard, total_pages=pages, top_k=top_k, sink=DEC_SINK,
                                       local=DEC_LOCAL, exchange=exchange)
        return tad.decode_partials_exchange_merge(
            lambda **kw: _C.decode_attention(q, k_hi, v_hi, sel, q4, k4, v4, qs, ks, vs, is_mx=False, is_bf16=False,
                                             kv_len=n_local * 64, page_table=table, allow_padded_selection=True, **kw),
            heads=DEC_BATCH * HKV, group_size=DEC_GROUP, head_dim=D, shard=shard, total_pages=pages, num_splits=0,
            is_mx=False, is_bf16=False, device=device, exchange=exchange)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def time_pieces(reps: int = 10) -> dict:
        """The sharded step launched piece by piece (eagerly, so launch gaps are inside the figures) with CUDA events
        between the pieces: median microseconds per piece on this rank."""
        n_sink = min(DEC_SINK, pages)
        local_lo = max(pages - DEC_LOCAL, n_sink)
        my_sink = max(0, min(n_sink, shard.page_end) - shard.page_begin)
        my_local = max(0, shard.page_end - max(local_lo, shard.page_begin))
        k_glob = min(top_k, max(pages - n_sink - (pages - local_lo), 0))
        cand = min(k_glob, max(n_local - my_sink - my_local, 0))
        biggest = max(sh.num_pages for sh in tad.plan_page_shards(pages, world))
        width = min(n_sink, biggest) + min(pages - local_lo, biggest) + min(k_glob, biggest)
        rows = heads = DEC_BATCH * HKV
        n_o, n_ml = heads * DEC_GROUP * D, heads * DEC_GROUP * 2
        names = ["quantise_q", "select", "gather1", "merge_candidates", "attend", "reduce", "gather2", "merge"]
        samples = {n: [] for n in names}
        for _ in range(reps + 2):
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(len(names) + 1)]
            if world > 1:
                dist.barrier()
            ev[0].record()
            q4, qs = _C.nvfp4_quantize(q)
            ev[1].record()
            buf = torch.empty(2, rows, width, dtype=torch.int32, device=device)
            _C.select_decode_blocks(q, k_min, k_max, cand, n_local, False, sink=my_sink, local=my_local, out=buf[0],
                                    return_scores=True, scores_out=buf[1].view(torch.float32), row_width=width)
            ev[2].record()
            gathered = tad._all_gather_stack(buf, None, exchange)
            ev[3].record()
            sel = _C.merge_page_candidates(gathered.contiguous(), rank=rank, total_pages=pages, top_k=top_k, sink=DEC_SINK,
                                           local=DEC_LOCAL)
            ev[4].record()
            _, part_o, part_ml = _C.decode_attention(q, k_hi, v_hi, sel, q4, k4, v4, qs, ks, vs, is_mx=False, is_bf16=False,
                                                     kv_len=n_local * 64, page_table=table, allow_padded_selection=True,
                                                     return_partials=True)
            ev[5].record()
            flat = torch.empty(n_o + n_ml, dtype=torch.float32, device=device)
            _C.reduce_decode_partials(part_o, part_ml, out=(flat[:n_o].view(heads, 1, DEC_GROUP, D),
                                                            flat[n_o:].view(heads, 1, DEC_GROUP, 2)))
            ev[6].record()
            allp = tad._all_gather_stack(flat, None, exchange)
            ev[7].record()
            _C.merge_decode_partials(allp[:, :n_o].view(world, heads, 1, DEC_GROUP, D),
                                     allp[:, n_o:].view(world, heads, 1, DEC_GROUP, 2), is_mx=False, is_bf16=False)
            ev[8].record()
            torch.cuda.synchronize()
            for j, n in enumerate(names):
                samples[n].append(ev[j].elapsed_time(ev[j + 1]) * 1e3)
        return {n: round(sorted(v[2:])[len(v[2:]) // 2], 1) for n, v in samples.items()}

    for _ in range(max(warmup, 3)):
        step()
    barrier()
    _C.decode_status()
    # A decode step is a fixed sequence of kernels and (N > 1) two all-gathers with no host decision in between,
    # so it is captured once and replayed: what is timed is the device work, not the Python that queues it.
    # Falls back to queueing the step eagerly where the capture is refused.
    run, mode = step, "eager"
    if os.environ.get("TA100_BENCH_DECODE_GRAPH", "1") != "0":
        try:
            side = torch.cuda.Stream(device=device)
            side.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(side):
                step()
            torch.cuda.current_stream(device).wait_stream(side)
            barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            barrier()
            graph.replay()
            barrier()
            run, mode = graph.replay, "cuda graph"
        except Exception as exc:                                  # noqa: BLE001 - any refusal means eager
            if rank == 0:
                print(f"decode step not captured ({type(exc).__name__}: {exc}); timing eager launches", file=sys.stderr)
            torch.cuda.synchronize()
            run, mode = step, "eager"
    if world > 1:
        # every rank must time the same way, or the replays and the eager collectives would interleave
        flag = torch.tensor([1 if mode == "cuda graph" else 0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if flag.item() == 0:
            run, mode = step, "eager"
    for _ in range(3):
        run()
    barrier()
    n_steps = max(steps, 5) * 4
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(n_steps + 1)]
    marks[0].record()
    for i in range(n_steps):
        run()
        marks[i + 1].record()
    barrier()
    _C.decode_status()
    if exchange is not None:
        exchange.check()
    per_step = [marks[i].elapsed_time(marks[i + 1]) for i in range(n_steps)]
    ms = torch.tensor([marks[0].elapsed_time(marks[-1]) / n_steps], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    # correctness of what was timed: an eager step with the same inputs, rows compared with the CPU oracle
    out = step().reshape(DEC_BATCH, HKV, DEC_GROUP, D)
    barrier()
    check = check_decode_rows(out, q, k_hi, v_hi, table, world=world, rank=rank, pages=pages, top_k=top_k,
                              splits_local=splits_local)
    pieces = time_pieces() if world > 1 else None
    barrier()
    n16 = top_k + DEC_SINK + DEC_LOCAL
    step_bytes = DEC_BATCH * HKV * ((pages - n16) * 9216 + n16 * 32768 + pages * 512)
    gbs = step_bytes / (ms.item() * 1e-3) / 1e9
    stats = call_stats(per_step)
    return {"us_per_step": ms.item() * 1e3, "value": gbs, "unit": "GB/s", "bytes_per_step": step_bytes,
            "frac_of_hbm_peak": gbs / (hbm_gbs * world), "hbm_peak_gbs_per_gpu": hbm_gbs,
            "us_per_step_rank0": {k: (v * 1e3 if k != "n" else v) for k, v in stats.items()},
            "check": check, "exchange": exchange_kind, "pieces_us_rank0_eager": pieces,
            "workload": f"paged decode {DEC_BATCH} seq x {DEC_SEQ} tokens, {HQ}q/{HKV}kv x {D}, NVFP4 + fp16 shadow, Quest "
                        f"{top_k} + {DEC_SINK} sink + {DEC_LOCAL} recent of {pages} pages in 16 bits; step = quantise q + "
                        f"select + attend + merge; KV sequence split over {world} GPU(s)",
            "launches_per_step": 4 if world == 1 else 6, "queued_as": mode}


def run_ours(args) -> dict:
    import torch.distributed as dist

    import thriftattention_b200 as ta
    from thriftattention_b200 import _C
    from thriftattention_b200.selection import resolve_top_k

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    if HKV % world != 0:
        raise SystemExit("the number of GPUs must divide the 8 KV heads")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    headline = args.workload == "headline"
    fmt, dtype, fraction = ("nvfp4", torch.float16, 0.10) if headline else ("mxfp4", torch.bfloat16, args.fraction)
    hkv_local, hq_local = HKV // world, HQ // world
    q, k, v = make_inputs(hq_local, hkv_local, SEQ, device, dtype, kv_head_offset=rank * hkv_local)
    top_k = resolve_top_k(SEQ // BLOCK, causal=True, fraction=fraction)
    cfg = ta.AttentionConfig(method="thrift", causal=True, selection="quest", fraction=fraction, block_size=BLOCK,
                             quant_format=fmt)
    # A rank's heads go through the public API in two calls so that (N > 1) the all-gather of the first half's output
    # runs under the second half's kernel.  Halves are whole KV-head groups, or halves of the single group's q heads.
    group = HQ // HKV
    if hkv_local >= 2:
        halves = [(0, hkv_local // 2), (hkv_local // 2, hkv_local)]
        chunks = [(slice(a * group, b * group), slice(a, b)) for a, b in halves]
    else:
        chunks = [(slice(0, group // 2), slice(0, 1)), (slice(group // 2, group), slice(0, 1))]
    if world == 1:
        chunks = [(slice(0, hq_local), slice(0, hkv_local))]
    gathered = [torch.empty(world, 1, c[0].stop - c[0].start, SEQ, D, device=device, dtype=dtype) for c in chunks] \
        if world > 1 else None
    kernel_events: list = []

    def step():
        outs, works = [], []
        for i, (qs_, kvs) in enumerate(chunks):
            out = ta.attention(q[:, qs_], k[:, kvs], v[:, kvs], config=cfg)
            outs.append(out)
            if world > 1:
                works.append(dist.all_gather_into_tensor(gathered[i], out.unsqueeze(0), async_op=True))
        for w in works:
            w.wait()
        return outs

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    _C.set_prefill_event_sink(kernel_events)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    barrier()
    marks[0].record()
    for i in range(args.steps):
        step()
        marks[i + 1].record()
    barrier()
    _C.set_prefill_event_sink(None)
    clocks = sampler.stop() if rank == 0 else {}
    step_times = [marks[i].elapsed_time(marks[i + 1]) for i in range(args.steps)]
    ms = torch.tensor([marks[0].elapsed_time(marks[-1])], device=device, dtype=torch.float64)
    # the kernel time of a step = the sum over the step's launches (one per half), averaged over the steps
    kernel_ms = sum(a.elapsed_time(b) for a, b in kernel_events) / args.steps
    attn_ms = torch.tensor([kernel_ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(attn_ms, op=dist.ReduceOp.MAX)
    ms_per_step = ms.item() / args.steps
    total_flops = algorithmic_flops(HQ, SEQ, D, BLOCK)
    value = total_flops / (ms_per_step * 1e-3) / 1e12

    # ---- end to end through the public API with host buffers (pinned), H2D + D2H inside the timed region ----
    hq_h = q.cpu().pin_memory(), k.cpu().pin_memory(), v.cpu().pin_memory()
    out_host = torch.empty(1, hq_local, SEQ, D, dtype=dtype).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in hq_h)
    d2h = out_host.numel() * out_host.element_size()

    def e2e_step():
        # host in, host out: chunks of query heads, their copies overlapped with the neighbouring chunks' kernels
        ta.attention_host(*hq_h, config=cfg, device=device, out=out_host, q_heads_per_chunk=2 if hkv_local == 1 else 0)

    e2e_steps = max(1, min(args.steps, 3))
    e2e_step()
    barrier()
    s2, t2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record()
    for _ in range(e2e_steps):
        e2e_step()
    t2.record()
    barrier()
    e2e_ms = torch.tensor([s2.elapsed_time(t2) / e2e_steps], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_value = total_flops / (e2e_ms.item() * 1e-3) / 1e12

    # ---- decode half of the metric (all ranks take part; prefill tensors are released first) ----
    del q, k, v, hq_h, out_host, gathered
    torch.cuda.empty_cache()
    peaks = measured_peaks()
    hbm_gbs = float(peaks.get("hbm_gbs", 6650.0))
    decode = run_decode_leg(device, world, rank, args.steps, args.warmup, hbm_gbs) if headline else None

    result = {}
    if rank == 0:
        if "bf16_tflops_sustained" in peaks:
            bf16_peak, peak_src = float(peaks["bf16_tflops_sustained"]), "measured (bf16_tflops_sustained)"
        else:
            bf16_peak, peak_src = 1400.0, "fallback (1.4 PFLOP/s sustained)"
        share16 = fp16_flop_share(SEQ, BLOCK, top_k)
        # blended tensor bound: t_min = F_fp4 / P_fp4 + F_fp16 / P_fp16, expressed as an effective peak
        blended_peak = 1.0 / ((1.0 - share16) / (FP4_TO_BF16_PEAK_RATIO * bf16_peak) + share16 / bf16_peak)
        per_rank_flops = total_flops / world
        achieved = per_rank_flops / (attn_ms.item() * 1e-3) / 1e12
        launches_per_kernel = len(chunks)
        traffic = BENCH_DRAM_BYTES * (per_rank_flops / launches_per_kernel) / BENCH_FLOPS
        metric = METRIC if headline else f"prefill_attention_tflops_128k_top{fraction * 100:g}pct_mxfp4_bf16"
        result = {
            "metric": metric, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp4(e2m1, block-scaled)+f16, fp32 accumulate", "data": "synthetic",
            "config": {"workload": f"prefill 1x32q/8kv x131072 x128 {'fp16' if headline else 'bf16'} causal, Quest "
                                   f"top-{fraction:.0%} ({top_k} of 1024 128-token blocks) in 16 bits, rest "
                                   f"{fmt.upper()}; step = ta.attention(): stats+select+quantise+attend",
                       "partition": f"kv-head groups over {world} GPU(s)",
                       "l2": "inputs (1.5 GiB/GPU at N=1) exceed the 126 MB L2; no explicit flush"},
            "clocks": clocks,
            "ms_per_step_rank0": call_stats(step_times),
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d * world,
                    "d2h_bytes_per_step": d2h * world, "ms_per_step": e2e_ms.item()},
            "gpu_launches": 10 * len(chunks) * args.steps,
            "roofline": {"bound": "tensor", "kernel": "prefill_kernel (fused FP4 + f16 tcgen05 attention)",
                         "achieved": achieved, "peak": blended_peak, "unit": "TFLOP/s", "frac": achieved / blended_peak,
                         "traffic": traffic, "traffic_note": "bytes per launch: one-pass ncu capture of this workload (all 32 q heads), scaled by the share of the heads a launch processes",
                         "kernel_ms": attn_ms.item(), "launches_per_step": launches_per_kernel,
                         "peak_source": f"{peak_src} x blended FP4/f16 mix (FP4 peak taken as {FP4_TO_BF16_PEAK_RATIO:g}x bf16; "
                                        f"16-bit FLOP share {share16:.3f})"},
        }
        if decode is not None:
            result["decode"] = decode
            # the decode half of the metric, also as top-level keys
            result["decode_us_per_step"] = decode["us_per_step"]
            result["decode_gbs"] = decode["value"]
            result["decode_frac_of_hbm_peak"] = decode["frac_of_hbm_peak"]
            result["decode_check"] = decode["check"]
        if world == 1 and headline:
            result["cpu_baseline"] = run_reference(argparse.Namespace(gpus=args.gpus, steps=1, warmup=0,
                                                                      with_small_cpu_config=False))["cpu_baseline"]
    if world > 1:
        dist.destroy_process_group()
    return result


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="headline", choices=["headline", "mxfp4-bf16"],
                    help="headline = fp16 / NVFP4 top-10 %% prefill + the decode step; mxfp4-bf16 = the bf16 / MXFP4 prefill")
    ap.add_argument("--fraction", type=float, default=0.10, help="share of 128-token blocks kept in bf16 (mxfp4-bf16 workload)")
    ap.add_argument("--hf", action="store_true",
                    help="instead of the headline: generation through the Transformers hook on a random-init decoder of the "
                         "Llama-3-8B shape (65,536-token prompt, 256 decode steps; eager loop and one CUDA graph per token) - "
                         "what benchmarks/run_hook_generation.py --graph prints")
    args = ap.parse_args()
    if args.hf:
        import importlib.util

        spec = importlib.util.spec_from_file_location(
            "run_hook_generation", os.path.join(os.path.dirname(os.path.abspath(__file__)), "benchmarks", "run_hook_generation.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.run_hf(65536, 256, 32, graphed=True)
        return
    result = run_reference(args) if args.impl == "reference" else run_ours(args)
    if result:
        print(json.dumps(result), flush=True)


if __name__ == "__main__":
    main()

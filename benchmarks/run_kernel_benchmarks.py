#!/usr/bin/env python3
"""Kernel timing CLI over ``thriftattention_b200.attention``.

Same job and flags as the reference's ``benchmarks/run_kernel_benchmarks.py`` (its spec table at
:201-279 and ``measure_cuda_events`` at :282-303): for every sequence length build seeded q, k, v,
then time — with 10 warm-up calls and 50 repeats by default, one CUDA-event pair per call — an exact
16-bit attention, pure-FP4 attention and ThriftAttention at each (selection, coverage), and print
mean / median / p90 / min / max per row.  Added here: a TFLOP/s column (block-granular causal FLOPs),
``--block-size``, sink / local forcing, and three modes used by the committed profiler summaries:

  --profile-case prefill|decode   three launches of one hot kernel on a case of a few hundred MB
                                  (what an ``ncu --set full`` capture is taken on), then exit
  --helpers                       GB/s of the HBM-bound helper kernels (quantisers, block statistics)

Examples
  python benchmarks/run_kernel_benchmarks.py 8192,32768 --heads 32 --kv-heads 8 --selections quest --coverages 5%,10%
  python benchmarks/run_kernel_benchmarks.py 131072 --q-len 1 --batch-size 32 --heads 32 --kv-heads 8 --selections quest
"""
from __future__ import annotations

import argparse
import json
import math
import statistics
import sys
from dataclasses import dataclass
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

import thriftattention_b200 as ta  # noqa: E402


@dataclass
class Row:
    seq_len: int
    name: str
    coverage: float | None
    top_k: int | None
    status: str
    times_ms: list | None = None
    flops: float | None = None
    note: str = ""


def _fractions(text: str) -> list[float]:
    out = []
    for part in text.split(","):
        part = part.strip()
        if part:
            val = float(part[:-1]) / 100.0 if part.endswith("%") else float(part)
            if not 0.0 <= val <= 1.0:
                raise argparse.ArgumentTypeError("coverage values must be in [0, 1], or percentages")
            out.append(val)
    if not out:
        raise argparse.ArgumentTypeError("at least one coverage value is required")
    return out


def _int_list(values: list[str]) -> list[int]:
    out = [int(p) for v in values for p in v.split(",") if p.strip()]
    if not out:
        raise argparse.ArgumentTypeError("at least one sequence length is required")
    return out


def _selections(text: str) -> list[str]:
    out = [p.strip() for p in text.split(",") if p.strip()]
    bad = [p for p in out if p not in ("block_mean", "quest", "local")]
    if bad or not out:
        raise argparse.ArgumentTypeError("selection methods must be one of block_mean, local, quest")
    return out


def percentile(values: list[float], q: float) -> float:
    ordered = sorted(values)
    pos = (len(ordered) - 1) * q
    lo, hi = math.floor(pos), math.ceil(pos)
    return ordered[lo] + (ordered[hi] - ordered[lo]) * (pos - lo)


def time_calls(fn, warmup: int, repeat: int) -> list[float]:
    """Per-call CUDA-event times in ms after ``warmup`` untimed calls (reference harness :282-303)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(repeat):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    return times


def attention_flops(batch: int, heads: int, q_len: int, kv_len: int, d: int, causal: bool, block: int = 128) -> float:
    if q_len == 1 or not causal:
        return 4.0 * d * batch * heads * q_len * kv_len
    nb = kv_len // block
    return 4.0 * d * batch * heads * (nb * (nb + 1) // 2) * block * block


def make_qkv(args, seq_len: int):
    gen = torch.Generator(device=args.device)
    q_len = seq_len if args.q_len is None else args.q_len
    gen.manual_seed(args.seed + seq_len + q_len)
    kw = dict(device=args.device, dtype=args.torch_dtype, generator=gen)
    q = torch.randn(args.batch_size, args.heads, q_len, args.head_dim, **kw)
    k = torch.randn(args.batch_size, args.kv_heads, seq_len, args.head_dim, **kw)
    v = torch.randn(args.batch_size, args.kv_heads, seq_len, args.head_dim, **kw)
    if args.key_outliers:
        k[..., torch.randperm(args.head_dim, device=args.device, generator=gen)[:4]] *= 10.0
    return q, k, v


def build_specs(args, q, k, v, seq_len: int):
    q_len = q.shape[2]
    impl = "single_query" if q_len == 1 else "tiled"
    causal = args.causal and q_len != 1
    specs = []
    if not args.skip_fp16:
        if args.fp16_backend == "flash-attn":
            try:
                from flash_attn import flash_attn_func

                qb, kb, vb = (t.transpose(1, 2).contiguous() for t in (q, k, v))
                specs.append((f"{args.dtype}_flash_attn", None, None,
                              lambda: flash_attn_func(qb, kb, vb, dropout_p=0.0, causal=causal)))
            except Exception as exc:  # noqa: BLE001 - an optional comparator
                specs.append((f"{args.dtype}_flash_attn", None, None, f"flash-attn is not importable: {exc}"))
        else:
            specs.append((f"{args.dtype}_torch_sdpa", None, None,
                          lambda: torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=causal,
                                                                                   enable_gqa=args.heads != args.kv_heads)))
    if not args.skip_fp4:
        cfg = ta.AttentionConfig(method="fp4", causal=args.causal, implementation=impl, quant_format=args.quant_format)
        specs.append((f"ta_{args.quant_format}_fp4_attention", None, None, lambda cfg=cfg: ta.attention(q, k, v, config=cfg)))
    if not args.skip_thrift:
        block = 64 if q_len == 1 else args.block_size
        for selection in args.selections:
            for cov in args.coverages:
                cfg = ta.AttentionConfig(method="thrift", causal=args.causal, selection=selection, fraction=cov,
                                         implementation=impl, quant_format=args.quant_format, block_size=block,
                                         sink_blocks=args.sink_blocks, local_blocks=args.local_blocks)
                top_k = ta.resolve_top_k(seq_len // block, causal=causal, fraction=cov)
                specs.append((f"thrift_{args.quant_format}_{selection}_{cov * 100:g}pct", cov, top_k,
                              lambda cfg=cfg: ta.attention(q, k, v, config=cfg)))
    return specs


def print_table(rows: list[Row]) -> None:
    head = ["seq", "benchmark", "coverage", "top_k", "status", "mean_ms", "median_ms", "p90_ms", "min_ms", "max_ms",
            "TFLOP/s", "note"]
    table = []
    for r in rows:
        t = r.times_ms
        cells = [str(r.seq_len), r.name, "-" if r.coverage is None else f"{r.coverage * 100:.2f}%",
                 "-" if r.top_k is None else str(r.top_k), r.status]
        if t:
            med = statistics.median(t)
            cells += [f"{statistics.fmean(t):.3f}", f"{med:.3f}", f"{percentile(t, 0.9):.3f}", f"{min(t):.3f}",
                      f"{max(t):.3f}", f"{r.flops / med / 1e9:.1f}" if r.flops else "-"]
        else:
            cells += ["-"] * 6
        table.append(cells + [r.note])
    widths = [max(len(h), *(len(c[i]) for c in table)) if table else len(h) for i, h in enumerate(head)]
    print()
    print("  ".join(h.ljust(w) for h, w in zip(head, widths)))
    print("  ".join("-" * w for w in widths))
    for cells in table:
        print("  ".join(c.ljust(w) for c, w in zip(cells, widths)))


# ----------------------------------------------------------------------------- profiler cases / helper kernels
def profile_case(kind: str) -> None:
    """Three back-to-back launches of one hot kernel on inputs larger than L2 but small enough for a full-set
    profiler capture; prints the algorithmic work of one launch."""
    from thriftattention_b200 import _C

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    d, hkv = 128, 4 if kind == "prefill" else 8
    if kind == "prefill":
        hq, seq, block = 16, 8192, 128
        q = torch.randn(1, hq, seq, d, device=dev).half()
        k = torch.randn(1, hkv, seq, d, device=dev).half()
        v = torch.randn(1, hkv, seq, d, device=dev).half()
        k[..., torch.randperm(d, device=dev)[:4]] *= 10.0
        top_k = ta.resolve_top_k(seq // block, causal=True, fraction=0.10)
        q_mean, _, _ = _C.block_stats(q, block, mean=True)
        _, k_min, k_max = _C.block_stats(k, block, minmax=True)
        sel = _C.select_prefill_blocks(q_mean, k_min, k_max, top_k, True, False)
        q4, qs = _C.nvfp4_quantize(q)
        k4, ks = _C.nvfp4_quantize_permuted(k)
        v4, vs = _C.nvfp4_quantize_transposed(v)
        for _ in range(3):
            _C.prefill_attention(q, k, v, sel, q4, k4, v4, qs, ks, vs, causal=True, is_mx=False, is_bf16=False,
                                 block_size=block, k_permuted=True, check_status=True)
        torch.cuda.synchronize()
        print(json.dumps({"case": "prefill 1x16q/4kv x8192 x128 fp16 NVFP4 Quest top-10% of 128-token blocks",
                          "flops_per_launch": attention_flops(1, hq, seq, seq, d, True, block)}))
        return
    batch, seq, group = 8, 32768, 4
    pages = seq // 64
    pool = batch * pages
    u8 = dict(dtype=torch.uint8, device=dev)
    k4 = torch.randint(0, 256, (pool, hkv, 64, d // 2), **u8)
    v4 = torch.randint(0, 256, (pool, hkv, d, 32), **u8)
    ks = torch.randint(40, 60, (pool, hkv, 64, d // 16), **u8)
    vs = torch.randint(40, 60, (pool, hkv, d, 4), **u8)
    k_hi = torch.empty(pool, hkv, 64, d, dtype=torch.float16, device=dev).normal_()
    v_hi = torch.empty(pool, hkv, 64, d, dtype=torch.float16, device=dev).normal_()
    k_min = torch.randn(batch, hkv, pages, d, device=dev).half()
    k_max = k_min + 1
    table = torch.randperm(pool, device=dev).to(torch.int32).reshape(batch, pages)
    q = torch.randn(batch, hkv, group, d, device=dev).half()
    top_k = max(1, round(0.10 * pages))
    for _ in range(3):
        q4, qs = _C.nvfp4_quantize(q)
        sel = _C.select_decode_blocks(q, k_min, k_max, top_k, pages, False, sink=4, local=16)
        _C.decode_attention(q, k_hi, v_hi, sel, q4, k4, v4, qs, ks, vs, is_mx=False, is_bf16=False, kv_len=seq,
                            page_table=table, allow_padded_selection=True)
    torch.cuda.synchronize()
    _C.decode_status()
    n16 = top_k + 20
    print(json.dumps({"case": "paged decode 8 seq x 32768 tokens, 32q/8kv x128, NVFP4 + fp16 shadow, 71 of 512 pages in 16 bits",
                      "attention_bytes_per_launch": batch * hkv * ((pages - n16) * 9216 + n16 * 32768),
                      "selection_bytes_per_launch": batch * hkv * pages * 512}))


def helper_bandwidth(args) -> None:
    """GB/s of algorithmic bytes (16-bit input + codes + scale bytes; statistics: input only) of the helper kernels."""
    from thriftattention_b200 import _C

    dev = torch.device(args.device)
    peaks = ROOT / "MEASURED_PEAKS.json"
    hbm = float(json.load(open(peaks))["hbm_gbs"]) if peaks.exists() else 6650.0
    for fmt, dtype in (("nvfp4", torch.float16), ("mxfp4", torch.bfloat16)):
        bf16 = dtype == torch.bfloat16
        x = torch.randn(1, args.kv_heads, args.seq_lens[0], args.head_dim, device=dev).to(dtype)
        elems, group = x.numel(), 32 if fmt == "mxfp4" else 16
        qbytes = elems * (2 + 0.5 + 1.0 / group)
        for name, fn, nbytes in (
                (f"{fmt}_quantize", lambda: getattr(_C, f"{fmt}_quantize")(x, bf16), qbytes),
                (f"{fmt}_quantize_permuted", lambda: getattr(_C, f"{fmt}_quantize_permuted")(x, bf16), qbytes),
                (f"{fmt}_quantize_transposed", lambda: getattr(_C, f"{fmt}_quantize_transposed")(x, bf16), qbytes),
                ("block_stats min/max", lambda: _C.block_stats(x, args.block_size, minmax=True), elems * 2.0)):
            t = statistics.median(time_calls(fn, 3, 10))
            print(json.dumps({"case": f"{name} of {list(x.shape)} {str(dtype).split('.')[-1]}", "us": t * 1e3,
                              "gbs": nbytes / t / 1e6, "frac_of_hbm_peak": nbytes / t / 1e6 / hbm}), flush=True)


def parse_args():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0], formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    ap.add_argument("seq_lens", nargs="*", default=["8192"], help="sequence lengths, as spaces or comma-separated values")
    ap.add_argument("--coverages", type=_fractions, default=_fractions("1%,5%,10%"))
    ap.add_argument("--selections", type=_selections, default=_selections("block_mean"))
    ap.add_argument("--batch-size", type=int, default=1)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=16)
    ap.add_argument("--q-len", type=int, default=None, help="query length; defaults to each sequence length, 1 = decode")
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--block-size", type=int, default=64, help="selection block size of the tiled path (64 or 128)")
    ap.add_argument("--sink-blocks", type=int, default=0)
    ap.add_argument("--local-blocks", type=int, default=0)
    ap.add_argument("--dtype", choices=("fp16", "bf16"), default="fp16")
    ap.add_argument("--quant-format", choices=("nvfp4", "mxfp4"), default="nvfp4")
    ap.add_argument("--key-outliers", action="store_true", help="scale 4 random K channels x10 (long-context key statistics)")
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--repeat", type=int, default=50)
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--non-causal", dest="causal", action="store_false")
    ap.add_argument("--fp16-backend", choices=("flash-attn", "torch"), default="torch")
    ap.add_argument("--skip-fp16", action="store_true")
    ap.add_argument("--skip-thrift", action="store_true")
    ap.add_argument("--skip-fp4", action="store_true")
    ap.add_argument("--keep-going", action="store_true", help="report benchmark errors instead of stopping")
    ap.add_argument("--profile-case", choices=("prefill", "decode"), default=None)
    ap.add_argument("--helpers", action="store_true")
    args = ap.parse_args()
    args.seq_lens = _int_list(args.seq_lens)
    args.torch_dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    return args


def main() -> None:
    args = parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("CUDA is required for these benchmarks")
    if args.profile_case:
        profile_case(args.profile_case)
        return
    if args.helpers:
        helper_bandwidth(args)
        return
    if args.head_dim not in (64, 128):
        raise SystemExit("--head-dim must be 64 or 128")
    if args.heads % args.kv_heads:
        raise SystemExit("--heads must be divisible by --kv-heads")
    rows: list[Row] = []
    for seq_len in args.seq_lens:
        q_len = seq_len if args.q_len is None else args.q_len
        if seq_len % 64 or (q_len != 1 and q_len % 64):
            raise SystemExit("sequence and query lengths must be 1 or divisible by 64")
        q, k, v = make_qkv(args, seq_len)
        flops = attention_flops(args.batch_size, args.heads, q_len, seq_len, args.head_dim, args.causal)
        print(f"Running q={q_len}, kv={seq_len}, batch={args.batch_size}, heads={args.heads}, kv_heads={args.kv_heads}, "
              f"dim={args.head_dim}, dtype={args.dtype}, quant_format={args.quant_format}")
        for name, cov, top_k, fn in build_specs(args, q, k, v, seq_len):
            if isinstance(fn, str):
                rows.append(Row(seq_len, name, cov, top_k, "skip", note=fn))
            else:
                try:
                    rows.append(Row(seq_len, name, cov, top_k, "ok", time_calls(fn, args.warmup, args.repeat), flops))
                except Exception as exc:  # noqa: BLE001
                    if not args.keep_going:
                        raise
                    rows.append(Row(seq_len, name, cov, top_k, "error", note=repr(exc)))
            print(f"  {rows[-1].status.upper()} {name}")
        del q, k, v
        torch.cuda.empty_cache()
    print_table(rows)


if __name__ == "__main__":
    main()

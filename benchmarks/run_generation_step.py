#!/usr/bin/env python3
"""Cache + attention work of ONE generated token over all layers: launches queued from Python with the sequence
length as a launch parameter, against one CUDA graph replayed per token with the length in device memory.

  python benchmarks/run_generation_step.py [--context 65536] [--layers 32] [--tokens 128] [--paged]

Shape of Llama-3-8B (batch 1, 32 query / 8 KV heads x 128, fp16), NVFP4 with the top 10 % of the 64-token blocks in
16 bits, random K/V.  Per layer and token: the fused cache append of the new K/V row and the decode step (quantise q,
block selection, split-KV attention, merge).  The eager arm is what the Transformers hook does per layer
(``update`` + ``cached_decode_attention``); the graph arm captures ``device_length_decode_step`` of every layer plus
one ``advance_length`` once and replays it.  Both arms are timed with CUDA events around ``--tokens`` consecutive
tokens, after a warm-up; the last token's outputs are compared.  Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--context", type=int, default=65536)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--tokens", type=int, default=128)
    ap.add_argument("--fraction", type=float, default=0.10)
    ap.add_argument("--paged", action="store_true")
    args = ap.parse_args()

    import thriftattention_b200 as ta
    from thriftattention_b200 import _C
    from thriftattention_b200.integrations import transformers_cache as tc

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    b, hq, hkv, d, dtype = 1, 32, 8, 128, torch.float16
    total = args.tokens * 2 + 8                               # warm-up + timed tokens of either arm
    max_len = (args.context + total + 63) // 64 * 64
    cfg = ta.AttentionConfig(selection="block_mean", fraction=args.fraction, quant_format="nvfp4")
    caches = [ta.ThriftAttentionCache(config=cfg, max_cache_len=max_len, paged=args.paged) for _ in range(2)]
    for layer in range(args.layers):
        k = torch.randn(b, hkv, args.context, d, device=dev, dtype=dtype)
        v = torch.randn(b, hkv, args.context, d, device=dev, dtype=dtype)
        for c in caches:
            c.update(k, v, layer, {"thrift_return_new_states": True})
        del k, v
    eager, graphed = caches
    for layer in range(args.layers):
        graphed.layer(layer).reserve(max_len)
    chains = max(1, min(_C.decode_pick_splits(b * hkv, max_len // 64), max_len // 64))

    q_in = torch.randn(args.layers, b, hq, 1, d, device=dev, dtype=dtype)
    k_in = torch.randn(args.layers, b, hkv, 1, d, device=dev, dtype=dtype)
    v_in = torch.randn(args.layers, b, hkv, 1, d, device=dev, dtype=dtype)
    out_graph = torch.zeros(args.layers, b, hq, 1, d, device=dev, dtype=dtype)
    length = torch.tensor([args.context], dtype=torch.int32, device=dev)

    def eager_token():
        outs = []
        for layer in range(args.layers):
            eager.update(k_in[layer], v_in[layer], layer, {"thrift_return_new_states": True})
            outs.append(tc.cached_decode_attention(q_in[layer], eager, layer, cfg))
        return outs

    def graph_token_body():
        for layer in range(args.layers):
            tc.device_length_decode_step(q_in[layer], k_in[layer], v_in[layer], graphed, layer, cfg, length, max_len=max_len,
                                         splits=chains, out=out_graph[layer])
        _C.advance_length(length, 1, max_len)

    def timed(fn, n):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(n):
            fn()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) * 1e3 / n

    # graph arm: one eager token (kernel attributes, scratch), capture, replay
    graph_token_body()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        graph_token_body()
    graph.replay()
    for _ in range(6):
        graph.replay()
    graph_us = timed(graph.replay, args.tokens)
    graph_len = int(length.item())

    for _ in range(8):
        eager_token()
    eager_us = timed(eager_token, args.tokens)

    # same length in both caches: compare one more token (the chain count of the eager arm is the library's own choice
    # for the current length, so the merge order may differ: compare numerically)
    while eager.layer(0).seq_len < graph_len:
        eager_token()
    while int(length.item()) < eager.layer(0).seq_len:
        graph.replay()
    outs = eager_token()
    graph.replay()
    torch.cuda.synchronize()
    diff = max(float((outs[i].float() - out_graph[i].float()).abs().max()) for i in range(args.layers))
    _C.decode_status(dev)
    print(json.dumps({
        "workload": f"llama3-8b shape, batch 1, context {args.context}, {args.layers} layers, nvfp4 + top {args.fraction:.0%} fp16",
        "paged": bool(args.paged), "tokens_timed": args.tokens, "chains_per_kv_head_graph": chains,
        "eager_us_per_token": round(eager_us, 1), "graph_us_per_token": round(graph_us, 1),
        "speedup": round(eager_us / graph_us, 2), "max_abs_diff_last_token": diff,
        "final_length": int(length.item()),
    }))


if __name__ == "__main__":
    main()

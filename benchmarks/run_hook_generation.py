#!/usr/bin/env python3
"""End-to-end generation through the Transformers attention hook on a random-init decoder of the Llama-3-8B shape.

  python benchmarks/run_hook_generation.py [--prompt 65536] [--new-tokens 256] [--layers 32] [--paged] [--graph]

Prefill of ``--prompt`` uniform-random token ids, then ``--new-tokens`` greedy decode steps over a
``ThriftAttentionCache`` (NVFP4, block-mean top-10 % of 64-token blocks), and the same weights with Transformers' own
exact attention (``sdpa``, ``DynamicCache``) for scale.  Prints one JSON line.  The warm-up pass of each arm doubles as a logits
comparison: the hooked model is fed the tokens the exact-attention model chose, and the last-position logits of the
prefill and of every decode step are compared (cosine similarity, largest difference, agreement of the arg-max).  Logits
parity of this path against the CPU oracle is covered at reduced sizes by tests/test_gpu_hf_model.py.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch  # noqa: E402

FRACTION = 0.10


def run_hf(prompt_len: int, new_tokens: int, layers: int, fraction: float = FRACTION, paged: bool = False,
           graphed: bool = False) -> None:
    """End to end through the Transformers hook on a random-init decoder of the Llama-3-8B shape (d_model 4096,
    32 q / 8 kv heads x 128, SwiGLU 14336, RoPE theta 5e5, vocab 128256, fp16): prefill of `prompt_len` uniform
    random token ids, then `new_tokens` greedy decode steps over a ThriftAttentionCache, NVFP4 with the top 10 %
    of the key blocks in fp16.  One JSON line: prefill and decode token rates and the same model's exact-attention
    (sdpa) rates for scale."""
    import contextlib

    import transformers

    from thriftattention_b200.integrations import (TransformersAttentionConfig, prepare_transformers_generation_cache,
                                                   register_transformers_attention)

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    name = register_transformers_attention(TransformersAttentionConfig(name="thrift_bench_hf", fraction=fraction))
    cfg = transformers.LlamaConfig(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=layers,
                                   num_attention_heads=32, num_key_value_heads=8, head_dim=128, rope_theta=500000.0,
                                   max_position_embeddings=max(131072, prompt_len + new_tokens), tie_word_embeddings=False)
    cfg._attn_implementation = name
    torch.manual_seed(0)
    with torch.device(device):
        model = transformers.LlamaForCausalLM(cfg).half().eval()
    ids = torch.randint(0, 128256, (1, prompt_len), generator=torch.Generator().manual_seed(1)).to(device)

    def generate(use_hook: bool, forced=None, keep=None):
        """One prefill + decode pass.  `forced`: token ids to feed instead of the arg-max; `keep`: list that receives the
        last-position logits (fp32, on the host) and the chosen tokens of every step."""
        with torch.no_grad():
            if use_hook:
                model.config._attn_implementation = name
                prep = prepare_transformers_generation_cache(model, ids, max_new_tokens=new_tokens, paged=paged)
                ctx, cache, inputs, pos0 = prep.activate(), prep.past_key_values, prep.input_ids, prep.cache_position
            else:
                model.config._attn_implementation = "sdpa"
                prep, ctx = None, contextlib.nullcontext()
                cache, inputs = transformers.DynamicCache(config=model.config), ids
                pos0 = torch.arange(prompt_len, device=device)
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            with ctx:
                ev[0].record()
                out = model(input_ids=inputs, past_key_values=cache, cache_position=pos0, use_cache=True, logits_to_keep=1)
                if prep is not None:
                    prep.trim_padding()
                def pick(step):
                    if keep is not None:
                        keep.append((out.logits[0, -1].float().cpu(), int(out.logits[0, -1].argmax())))
                    if forced is not None:
                        return torch.tensor([[forced[step]]], device=device)
                    return out.logits[:, -1].argmax(-1, keepdim=True)

                tok = pick(0)
                ev[1].record()
                for step in range(new_tokens):
                    out = model(input_ids=tok, past_key_values=cache,
                                cache_position=torch.tensor([prompt_len + step], device=device), use_cache=True)
                    tok = pick(step + 1)
                ev[2].record()
            torch.cuda.synchronize()
            assert torch.isfinite(out.logits).all()
            return ev[0].elapsed_time(ev[1]), ev[1].elapsed_time(ev[2])

    def generate_graphed():
        """Prefill as above, then the decode loop as ONE CUDA graph replayed per token: the cache keeps its length on
        the GPU (enable_device_length), the graph holds a whole single-token forward pass plus the arg-max fed back."""
        with torch.no_grad():
            model.config._attn_implementation = name
            prep = prepare_transformers_generation_cache(model, ids, max_new_tokens=new_tokens + 8, paged=paged)
            cache = prep.past_key_values
            with prep.activate():
                out = model(input_ids=prep.input_ids, past_key_values=cache, cache_position=prep.cache_position, use_cache=True,
                            logits_to_keep=1)
                prep.trim_padding()
                tok = out.logits[:, -1].argmax(-1, keepdim=True).clone()
                cache.enable_device_length()

                def step():
                    pos = cache.device_positions()
                    o = model(input_ids=tok, past_key_values=cache, cache_position=pos, position_ids=pos.view(1, 1), use_cache=True)
                    tok.copy_(o.logits[:, -1].argmax(-1, keepdim=True))
                    cache.advance_device_length()

                step()
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    step()
                for _ in range(3):
                    graph.replay()
                ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
                ev[0].record()
                for _ in range(new_tokens):
                    graph.replay()
                ev[1].record()
                torch.cuda.synchronize()
                assert cache.disable_device_length() == prompt_len + new_tokens + 4
            return ev[0].elapsed_time(ev[1])

    exact, ours = [], []
    try:
        generate(False, keep=exact)                          # warm-up; its logits and tokens are the comparison's reference
        pre_x, dec_x = generate(False)
    except torch.OutOfMemoryError:
        pre_x = dec_x = float("nan")
        exact = []
    torch.cuda.empty_cache()
    generate(True, forced=[t for _, t in exact] if exact else None, keep=ours)   # warm-up (library handles, workspaces)
    pre, dec = generate(True)
    torch.cuda.empty_cache()
    dec_graph = generate_graphed() if graphed else None
    logits = None
    if exact:
        cos = [float(torch.nn.functional.cosine_similarity(a, b, dim=0)) for (a, _), (b, _) in zip(exact, ours)]
        logits = {"steps_compared": len(cos), "cosine_min": min(cos), "cosine_mean": sum(cos) / len(cos),
                  "max_abs_diff": max(float((a - b).abs().max()) for (a, _), (b, _) in zip(exact, ours)),
                  "exact_logit_abs_max": max(float(a.abs().max()) for a, _ in exact),
                  "argmax_agreement": sum(int(x[1] == y[1]) for x, y in zip(exact, ours)) / len(cos)}
    print(json.dumps({
        "case": f"Transformers hook, Llama-3-8B-shaped decoder ({layers} layers, random init, fp16): prefill {prompt_len} "
                f"tokens + {new_tokens} greedy decode steps, NVFP4 + block-mean top-{fraction:.0%}" + (", paged cache" if paged else ""),
        "prefill_ms": pre, "prefill_tokens_per_s": prompt_len / pre * 1e3,
        "decode_ms_per_token": dec / new_tokens, "decode_tokens_per_s": new_tokens / dec * 1e3,
        "graph_decode_ms_per_token": None if dec_graph is None else dec_graph / new_tokens,
        "sdpa_prefill_ms": pre_x, "sdpa_decode_ms_per_token": dec_x / new_tokens,
        "logits_vs_exact_attention": logits,
        "peak_memory_gib": torch.cuda.max_memory_allocated(device) / 2 ** 30}), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--prompt", type=int, default=65536)
    ap.add_argument("--new-tokens", type=int, default=256)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--fraction", type=float, default=FRACTION, help="share of the key blocks kept in 16 bit (1.0: all of them)")
    ap.add_argument("--paged", action="store_true", help="keep the cache in page pools behind a page table")
    ap.add_argument("--graph", action="store_true",
                    help="also time the decode loop as one CUDA graph per token (cache length kept on the GPU)")
    args = ap.parse_args()
    run_hf(args.prompt, args.new_tokens, args.layers, args.fraction, args.paged, args.graph)


if __name__ == "__main__":
    main()

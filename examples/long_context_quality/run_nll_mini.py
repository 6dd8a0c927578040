#!/usr/bin/env python3
"""Mini forward / next-token NLL run of a causal LM under the registered attention hooks.

Same job and flags as the reference's ``examples/long_context_quality/run_nll_mini.py`` (:58-123 set-up,
:131-190 the loop): tokenise a local text file (``--text-file``) into ``--num-docs`` documents of the
longest ``--lengths`` entry, run the model body once per (method, fraction, length) with the attention
implementation switched between the model's exact 16-bit attention (``fp16``: PyTorch SDPA here), pure FP4
(``fp4``) and ThriftAttention (``thrift``), compute the mean next-token negative log-likelihood in
``--ce-chunk`` slices and print / write a table with the delta against the 16-bit run.

Nothing is downloaded: ``--model`` is a local directory with weights and tokenizer, or — to exercise the
pipeline without any weights — ``--random-init llama-8b|tiny`` builds a randomly initialised decoder and a
byte-level tokenizer (NLL is then near log(vocab) for every method; what is compared is the DELTA between
attention implementations on identical weights and text).  The dataset streaming mode of the reference needs
network access and is not offered.
"""
from __future__ import annotations

import argparse
import json
import math
import sys
import time
from datetime import datetime, timezone
from pathlib import Path
from statistics import fmean

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

SHAPES = {
    # name: (layers, d_model, ffn, q heads, kv heads, head_dim)
    "llama-8b": (32, 4096, 14336, 32, 8, 128),
    "tiny": (2, 512, 1024, 8, 2, 64),
}


class ByteTokenizer:
    """UTF-8 bytes as token ids (vocabulary 256): enough to feed real text to a randomly initialised model."""

    eos_token_id = None
    bos_token_id = None

    def __call__(self, text, add_special_tokens=False):
        return {"input_ids": list(text.encode("utf-8"))}


def load_text_file_docs(tokenizer, path: Path, *, length: int, num_docs: int) -> list[list[int]]:
    ids = tokenizer(path.read_text(encoding="utf-8"), add_special_tokens=False)["input_ids"]
    need = length * num_docs
    if len(ids) < need:
        raise SystemExit(f"{path} only tokenized to {len(ids)} tokens, but this run needs {need} tokens "
                         f"({num_docs} docs x {length}).")
    return [ids[i * length:(i + 1) * length] for i in range(num_docs)]


def build_model(args, max_len: int):
    import torch
    import transformers

    dtype = torch.float16 if args.device.startswith("cuda") else torch.float32
    if args.random_init:
        layers, d_model, ffn, hq, hkv, hd = SHAPES[args.random_init]
        layers = args.layers or layers
        tok = ByteTokenizer()
        cfg = transformers.LlamaConfig(vocab_size=256, hidden_size=d_model, intermediate_size=ffn, num_hidden_layers=layers,
                                       num_attention_heads=hq, num_key_value_heads=hkv, head_dim=hd, rope_theta=500000.0,
                                       max_position_embeddings=max(max_len, 8192), tie_word_embeddings=False)
        cfg._attn_implementation = "sdpa"
        torch.manual_seed(args.seed)
        with torch.device(args.device):
            model = transformers.LlamaForCausalLM(cfg).to(dtype).eval()
        return tok, model, dtype
    tok = transformers.AutoTokenizer.from_pretrained(args.model, use_fast=True, local_files_only=True)
    cfg = transformers.AutoConfig.from_pretrained(args.model, local_files_only=True)
    if max_len > getattr(cfg, "max_position_embeddings", max_len):
        original = cfg.max_position_embeddings
        cfg.max_position_embeddings = max_len
        cfg.rope_scaling = {"rope_type": "yarn", "factor": max_len / original,
                            "original_max_position_embeddings": original}
    model = transformers.AutoModelForCausalLM.from_pretrained(args.model, config=cfg, torch_dtype=dtype,
                                                              attn_implementation="sdpa", local_files_only=True)
    return tok, model.to(args.device).eval(), dtype


def mean_nll(model, body, doc, length: int, ce_chunk: int, device: str) -> tuple[float, float]:
    import torch
    import torch.nn.functional as F

    ids = torch.tensor([doc[:length]], dtype=torch.long, device=device)
    targets = torch.tensor(doc[1:length], dtype=torch.long, device=device)
    if device.startswith("cuda"):
        torch.cuda.synchronize(device)
    t0 = time.perf_counter()
    with torch.inference_mode():
        hidden = body(input_ids=ids, use_cache=False, return_dict=True).last_hidden_state[:, :-1, :]
        total = 0.0
        head = model.get_output_embeddings()
        for a in range(0, targets.numel(), ce_chunk):
            b = min(a + ce_chunk, targets.numel())
            total += float(F.cross_entropy(head(hidden[:, a:b, :]).squeeze(0).float(), targets[a:b], reduction="sum"))
    if device.startswith("cuda"):
        torch.cuda.synchronize(device)
    return total / targets.numel(), time.perf_counter() - t0


def main() -> None:
    ap = argparse.ArgumentParser(description="Mini forward/NLL benchmark for the registered attention implementations.")
    ap.add_argument("--model", default=None, help="local directory with a causal LM and its tokenizer")
    ap.add_argument("--random-init", choices=sorted(SHAPES), default=None, help="random weights + byte tokenizer instead")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count of --random-init")
    ap.add_argument("--lengths", default="8192")
    ap.add_argument("--methods", default="fp16,fp4,thrift")
    ap.add_argument("--fractions", default="0.05")
    ap.add_argument("--selection", default="block_mean", choices=("block_mean", "quest", "local"))
    ap.add_argument("--quant-format", default="nvfp4", choices=("nvfp4", "mxfp4"))
    ap.add_argument("--num-docs", type=int, default=1)
    ap.add_argument("--text-file", type=Path, required=True)
    ap.add_argument("--ce-chunk", type=int, default=1024)
    ap.add_argument("--output", type=Path, default=None)
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--device", default="cuda")
    args = ap.parse_args()
    if (args.model is None) == (args.random_init is None):
        raise SystemExit("give exactly one of --model (a local directory) or --random-init")

    import torch

    from thriftattention_b200.integrations import TransformersAttentionConfig, register_transformers_attention

    lengths = [int(x) for x in args.lengths.replace(" ", ",").split(",") if x.strip()]
    methods = [x.strip().lower() for x in args.methods.split(",") if x.strip()]
    fractions = [float(x) for x in args.fractions.replace(" ", ",").split(",") if x.strip()]
    bad = [m for m in methods if m not in ("fp16", "fp4", "thrift")]
    if bad:
        raise SystemExit(f"unknown methods {bad}; choose from fp16, fp4, thrift")
    if any(n % 64 for n in lengths):
        raise SystemExit("lengths must be multiples of 64 tokens (the attention kernels' tile)")
    torch.manual_seed(args.seed)

    tokenizer, model, _ = build_model(args, max(lengths))
    docs = load_text_file_docs(tokenizer, args.text_file, length=max(lengths), num_docs=args.num_docs)
    body = getattr(model, getattr(model, "base_model_prefix", ""), None) or getattr(model, "model", None)

    rows = []
    for method in methods:
        for fraction in (fractions if method == "thrift" else [None]):
            label = f"thrift_{fraction * 100:g}pct".replace(".", "p") if method == "thrift" else method
            if method == "fp16":
                model.set_attn_implementation("sdpa")
                print(f"\n{label}: exact 16-bit attention (PyTorch SDPA)")
            else:
                name = "thrift_fp4" if method == "fp4" else f"thrift_attention_{label}"
                impl = register_transformers_attention(TransformersAttentionConfig(
                    name=name, method=method, fraction=0.0 if fraction is None else fraction, selection=args.selection,
                    quant_format=args.quant_format))
                model.set_attn_implementation(impl)
                print(f"\n{label}: registered {impl}")
            for length in lengths:
                vals, secs = zip(*(mean_nll(model, body, doc, length, args.ce_chunk, args.device) for doc in docs))
                nll, sec = fmean(vals), fmean(secs)
                rows.append({"method": method, "label": label, "fraction": fraction, "length": length, "status": "ok",
                             "mean_nll": nll, "ppl": math.exp(nll) if nll < 50 else float("inf"), "forward_s": sec,
                             "forward_tok_s": length / sec})
                print(f"  length={length:<6} nll={nll:.4f} forward_s={sec:.3f}")

    base = {r["length"]: r["mean_nll"] for r in rows if r["label"] == "fp16"}
    for r in rows:
        if r["length"] in base:
            r["delta_vs_fp16"] = r["mean_nll"] - base[r["length"]]
    cols = [("length", "tokens"), ("label", "method"), ("mean_nll", "mean_nll"), ("delta_vs_fp16", "delta"),
            ("forward_s", "forward_s"), ("forward_tok_s", "tok/s"), ("status", "status")]
    lines = ["| " + " | ".join(h for _, h in cols) + " |", "| " + " | ".join("---" for _ in cols) + " |"]
    for r in rows:
        cells = []
        for key, _ in cols:
            val = r.get(key, "")
            cells.append("-" if val is None else (f"{val:.4g}" if isinstance(val, float) else str(val)))
        lines.append("| " + " | ".join(cells) + " |")
    table = "\n".join(lines)
    print("\nAverage scores\n" + table)
    if args.output:
        out_dir = args.output / f"{datetime.now(timezone.utc).strftime('%Y%m%d-%H%M%S')}-nll-mini"
        out_dir.mkdir(parents=True)
        (out_dir / "environment.json").write_text(json.dumps(vars(args), indent=2, sort_keys=True, default=str) + "\n")
        with (out_dir / "metrics.jsonl").open("w", encoding="utf-8") as fh:
            for r in rows:
                fh.write(json.dumps(r, sort_keys=True) + "\n")
        (out_dir / "summary.md").write_text("# NLL Mini\n\n" + table + "\n", encoding="utf-8")
        print(f"\nWrote {out_dir}")


if __name__ == "__main__":
    main()

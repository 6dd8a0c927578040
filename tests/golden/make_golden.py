"""Generates tests/golden/reference_selection.pt by running the reference's own Python
(its CPU-runnable selection code) on seeded inputs.

Run where the reference checkout is importable, e.g.
    PYTHONPATH=<reference>/src python tests/golden/make_golden.py
The reference demands CUDA tensors in ``check_qkv``; as its own tests do, that check is
patched out so its PyTorch paths run on CPU.  Nothing here is needed at test time: the
tests read only the committed .pt file.
"""
from __future__ import annotations

import os
import sys

import torch


def main() -> None:
    from thriftattention.selection import block_mean, quest, resolve_top_k  # the reference package

    block_mean.check_qkv = lambda *a, **k: None
    quest.check_qkv = lambda *a, **k: None
    out: dict = {"top_k": [], "stats": [], "quest_prefill": [], "quest_decode": [], "mean_decode": []}

    for n in (1, 2, 7, 32, 256, 512, 1024, 2048):
        for causal in (True, False):
            for fraction in (0.0, 0.01, 0.05, 0.10, 0.25, 0.5, 0.99, 1.0):
                out["top_k"].append((n, causal, None, fraction, resolve_top_k(n, causal=causal, fraction=fraction)))
            for top_k in (0, 1, 5, n, n + 3):
                out["top_k"].append((n, causal, top_k, None, resolve_top_k(n, causal=causal, top_k=top_k)))

    g = torch.Generator().manual_seed(1234)
    for dtype in (torch.float16, torch.bfloat16):
        is_bf16 = dtype == torch.bfloat16
        for block in (64, 128):
            x = (torch.randn(1, 1, 2 * block, 64, generator=g) * 1.5).to(dtype)
            mean = block_mean.block_means(x, block_size=block, is_bf16=is_bf16)
            lo, hi = quest.block_minmax(x, block_size=block, is_bf16=is_bf16)
            out["stats"].append({"x": x, "block": block, "mean": mean, "min": lo, "max": hi})
        # Quest prefill through the reference's PyTorch scoring path (CPU tensors never reach its extension)
        for (hq, hkv, nblk, top_k, causal) in ((4, 2, 6, 2, True), (2, 2, 9, 3, False), (4, 1, 5, 5, True)):
            q = torch.randn(1, hq, nblk * 8, 64, generator=g).to(dtype)
            k = torch.randn(1, hkv, nblk * 8, 64, generator=g).to(dtype)
            sel = quest.select_quest_block_pairs(q, k, causal=causal, top_k=top_k, block_size=8, is_bf16=is_bf16)
            out["quest_prefill"].append({"q": q, "k": k, "top_k": top_k, "causal": causal, "block": 8, "sel": sel})
        for (hq, hkv, nblk, top_k) in ((6, 2, 7, 3), (4, 4, 12, 4)):
            q = torch.randn(2, hq, 1, 64, generator=g).to(dtype)
            k = torch.randn(2, hkv, nblk * 8, 64, generator=g).to(dtype)
            sel_q = quest.select_quest_key_blocks(q, k, top_k=top_k, block_size=8, is_bf16=is_bf16)
            sel_m = block_mean.select_key_blocks(q, k, top_k=top_k, block_size=8, is_bf16=is_bf16)
            out["quest_decode"].append({"q": q, "k": k, "top_k": top_k, "block": 8, "sel": sel_q})
            out["mean_decode"].append({"q": q, "k": k, "top_k": top_k, "block": 8, "sel": sel_m})

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_selection.pt")
    torch.save(out, path)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()

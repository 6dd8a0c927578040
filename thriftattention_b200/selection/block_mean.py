"""Block-mean selection: score(q block, kv block) = mean(q rows) . mean(k rows)
(the reference's src/thriftattention/selection/block_mean.py:44-191).

The per-block means come from one fused CUDA pass (no fp32 copy of Q/K, no per-Q-head
expansion of the K statistics); scoring and the exact top-k run in the selection kernel.
"""
from __future__ import annotations

import torch

from thriftattention_b200._checks import check_qkv, require_block_aligned
from thriftattention_b200._extension import get_extension
from thriftattention_b200.selection.base import SelectionConfig
from thriftattention_b200.selection.counts import resolve_top_k

MAX_KV_BLOCKS = 2048


def block_means(x: torch.Tensor, *, block_size: int = 64, is_bf16: bool = False) -> torch.Tensor:
    """[B,H,S,D] -> [B,H,S/block,D]: fp32 mean over each block, cast back to x.dtype."""
    require_block_aligned("x", x.shape[2], block_size)
    mean, _, _ = get_extension().block_stats(x.contiguous(), block_size, mean=True)
    return mean


def _empty_pairs(q: torch.Tensor, block_size: int) -> torch.Tensor:
    return torch.empty(q.shape[0] * q.shape[1], q.shape[2] // block_size, 0, device=q.device, dtype=torch.int32)


def _check_block_count(num_kv_blocks: int) -> None:
    if num_kv_blocks > MAX_KV_BLOCKS:
        raise NotImplementedError(f"block selection supports at most {MAX_KV_BLOCKS} KV blocks, got {num_kv_blocks}")


def select_block_pairs(q, k, *, causal: bool = True, top_k: int | None = None, fraction: float | None = 0.05,
                       block_size: int = 64, is_bf16: bool = False, sink_blocks: int = 0,
                       local_blocks: int = 0) -> torch.Tensor:
    """Selected KV blocks per query block: int32 [B*Hq, Sq/block, k], rank ordered, -1 padded."""
    check_qkv(q, k, k)
    require_block_aligned("q", q.shape[2], block_size)
    require_block_aligned("k", k.shape[2], block_size)
    num_kv_blocks = k.shape[2] // block_size
    count = resolve_top_k(num_kv_blocks, causal=causal, top_k=top_k, fraction=fraction)
    count = max(0, min(count, num_kv_blocks - sink_blocks - local_blocks)) if (sink_blocks or local_blocks) else count
    if count + sink_blocks + local_blocks == 0:
        return _empty_pairs(q, block_size)
    _check_block_count(num_kv_blocks)
    ext = get_extension()
    q_mean, _, _ = ext.block_stats(q.contiguous(), block_size, mean=True)
    k_mean, _, _ = ext.block_stats(k.contiguous(), block_size, mean=True)
    if sink_blocks or local_blocks:
        return ext.select_prefill_blocks(q_mean, k_mean, None, count, causal, is_bf16, sink_blocks, local_blocks)
    return ext.block_mean_topk(q_mean, k_mean, count, causal, is_bf16)


def select_key_blocks(q, k, *, top_k: int | None = None, fraction: float | None = 0.05, block_size: int = 64,
                      is_bf16: bool = False, sink_blocks: int = 0, local_blocks: int = 0) -> torch.Tensor:
    """Decode: selected KV blocks per KV head (score = max over its query heads): int32 [B*Hkv, k]."""
    check_qkv(q, k, k)
    if q.shape[2] != 1:
        raise ValueError("single-query block selection expects q sequence length 1")
    require_block_aligned("k", k.shape[2], block_size)
    num_kv_blocks = k.shape[2] // block_size
    count = resolve_top_k(num_kv_blocks, causal=False, top_k=top_k, fraction=fraction)
    count = max(0, min(count, num_kv_blocks - sink_blocks - local_blocks)) if (sink_blocks or local_blocks) else count
    batch, q_heads, _, head_dim = q.shape
    kv_heads = k.shape[1]
    if count + sink_blocks + local_blocks == 0:
        return torch.empty(batch * kv_heads, 0, device=q.device, dtype=torch.int32)
    _check_block_count(num_kv_blocks)
    ext = get_extension()
    q_grouped = q.reshape(batch, kv_heads, q_heads // kv_heads, head_dim).contiguous()
    k_mean, _, _ = ext.block_stats(k.contiguous(), block_size, mean=True)
    if sink_blocks or local_blocks:
        return ext.select_decode_blocks(q_grouped, k_mean, None, count, num_kv_blocks, is_bf16, sink_blocks,
                                        local_blocks)
    return ext.single_query_key_mean_topk(q_grouped, k_mean, count, num_kv_blocks, is_bf16)


class BlockMeanSelectionPolicy:
    name = "block_mean"

    def select(self, q, k, *, config: SelectionConfig, causal: bool, is_bf16: bool) -> torch.Tensor:
        if config.name != self.name:
            raise ValueError(f"selection config {config.name!r} does not match block_mean policy")
        common = dict(top_k=config.top_k, fraction=config.fraction, block_size=config.block_size, is_bf16=is_bf16,
                      sink_blocks=config.sink_blocks, local_blocks=config.local_blocks)
        if q.shape[2] == 1:
            return select_key_blocks(q, k, **common)
        return select_block_pairs(q, k, causal=causal, **common)

"""Quest selection: score(q block, kv block) = sum_d q_d * (q_d >= 0 ? kmax_d : kmin_d)
with q the block-mean query (or, for decode, the max over the grouped query heads)
(the reference's src/thriftattention/selection/quest.py:11-187).
"""
from __future__ import annotations

import torch

from thriftattention_b200._checks import check_qkv, require_block_aligned
from thriftattention_b200._extension import get_extension
from thriftattention_b200.selection.base import SelectionConfig
from thriftattention_b200.selection.block_mean import _check_block_count, _empty_pairs
from thriftattention_b200.selection.counts import resolve_top_k


def block_minmax(x: torch.Tensor, *, block_size: int = 64, is_bf16: bool = False):
    """[B,H,S,D] -> (min, max), each [B,H,S/block,D], over the rows of each block."""
    require_block_aligned("x", x.shape[2], block_size)
    _, lo, hi = get_extension().block_stats(x.contiguous(), block_size, minmax=True)
    return lo, hi


def select_quest_block_pairs(q, k, *, causal: bool = True, top_k: int | None = None,
                             fraction: float | None = 0.05, block_size: int = 64, is_bf16: bool = False,
                             sink_blocks: int = 0, local_blocks: int = 0) -> torch.Tensor:
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
    _, k_min, k_max = ext.block_stats(k.contiguous(), block_size, minmax=True)
    if sink_blocks or local_blocks:
        return ext.select_prefill_blocks(q_mean, k_min, k_max, count, causal, is_bf16, sink_blocks, local_blocks)
    return ext.quest_block_topk(q_mean, k_min, k_max, count, causal, is_bf16)


def select_quest_key_blocks(q, k, *, top_k: int | None = None, fraction: float | None = 0.05,
                            block_size: int = 64, is_bf16: bool = False, sink_blocks: int = 0,
                            local_blocks: int = 0) -> torch.Tensor:
    check_qkv(q, k, k)
    if q.shape[2] != 1:
        raise ValueError("single-query QUEST selection expects q sequence length 1")
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
    _, k_min, k_max = ext.block_stats(k.contiguous(), block_size, minmax=True)
    if sink_blocks or local_blocks:
        return ext.select_decode_blocks(q_grouped, k_min, k_max, count, num_kv_blocks, is_bf16, sink_blocks,
                                        local_blocks)
    return ext.single_query_quest_topk(q_grouped, k_min, k_max, count, num_kv_blocks, is_bf16)


class QuestSelectionPolicy:
    name = "quest"

    def select(self, q, k, *, config: SelectionConfig, causal: bool, is_bf16: bool) -> torch.Tensor:
        if config.name != self.name:
            raise ValueError(f"selection config {config.name!r} does not match QUEST policy")
        common = dict(top_k=config.top_k, fraction=config.fraction, block_size=config.block_size, is_bf16=is_bf16,
                      sink_blocks=config.sink_blocks, local_blocks=config.local_blocks)
        if q.shape[2] == 1:
            return select_quest_key_blocks(q, k, **common)
        return select_quest_block_pairs(q, k, causal=causal, **common)

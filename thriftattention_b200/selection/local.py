"""Local-window selection: the k blocks ending at the diagonal (causal), a centred window
(non-causal) or the trailing k blocks (decode)
(the reference's src/thriftattention/selection/local.py:11-115)."""
from __future__ import annotations

import torch

from thriftattention_b200._checks import check_qkv, require_block_aligned
from thriftattention_b200._extension import get_extension
from thriftattention_b200.selection.base import SelectionConfig
from thriftattention_b200.selection.counts import resolve_top_k


def select_local_block_pairs(q, k, *, causal: bool = True, top_k: int | None = None,
                             fraction: float | None = 0.05, block_size: int = 64,
                             is_bf16: bool = False) -> torch.Tensor:
    check_qkv(q, k, k)
    require_block_aligned("q", q.shape[2], block_size)
    require_block_aligned("k", k.shape[2], block_size)
    num_kv_blocks = k.shape[2] // block_size
    count = resolve_top_k(num_kv_blocks, causal=causal, top_k=top_k, fraction=fraction)
    if count == 0:
        return torch.empty(q.shape[0] * q.shape[1], q.shape[2] // block_size, 0, device=q.device, dtype=torch.int32)
    return get_extension().local_block_topk(q, num_kv_blocks, count, causal, block_size)


def select_local_key_blocks(q, k, *, top_k: int | None = None, fraction: float | None = 0.05,
                            block_size: int = 64, is_bf16: bool = False) -> torch.Tensor:
    check_qkv(q, k, k)
    if q.shape[2] != 1:
        raise ValueError("single-query local selection expects q sequence length 1")
    require_block_aligned("k", k.shape[2], block_size)
    num_kv_blocks = k.shape[2] // block_size
    count = resolve_top_k(num_kv_blocks, causal=False, top_k=top_k, fraction=fraction)
    batch, q_heads, _, head_dim = q.shape
    kv_heads = k.shape[1]
    if count == 0:
        return torch.empty(batch * kv_heads, 0, device=q.device, dtype=torch.int32)
    q_grouped = q.reshape(batch, kv_heads, q_heads // kv_heads, head_dim).contiguous()
    return get_extension().single_query_local_topk(q_grouped, count, num_kv_blocks)


class LocalSelectionPolicy:
    name = "local"

    def select(self, q, k, *, config: SelectionConfig, causal: bool, is_bf16: bool) -> torch.Tensor:
        if config.name != self.name:
            raise ValueError(f"selection config {config.name!r} does not match local policy")
        common = dict(top_k=config.top_k, fraction=config.fraction, block_size=config.block_size, is_bf16=is_bf16)
        if q.shape[2] == 1:
            return select_local_key_blocks(q, k, **common)
        return select_local_block_pairs(q, k, causal=causal, **common)

"""Helpers for the q_len == 1 (decode) path: dispatch rule and GQA grouping
(the reference's src/thriftattention/backends/single_query.py)."""
from __future__ import annotations

import torch

MAX_GROUP = 16


def _use_single_query(q: torch.Tensor, implementation: str) -> bool:
    if implementation == "auto":
        return q.shape[2] == 1
    if implementation == "tiled":
        return False
    if implementation == "single_query":
        if q.shape[2] != 1:
            raise ValueError("implementation='single_query' requires q sequence length 1")
        return True
    raise ValueError("implementation must be 'auto', 'tiled', or 'single_query'")


def _group_single_query(q: torch.Tensor, kv_heads: int) -> torch.Tensor:
    """[B,Hq,1,D] -> [B,Hkv,G,D]: the G query heads sharing a KV head become the rows of one problem."""
    batch, q_heads, q_len, head_dim = q.shape
    if q_len != 1:
        raise ValueError("single-query attention expects q sequence length 1")
    group = q_heads // kv_heads
    if group > MAX_GROUP:
        raise NotImplementedError("single-query kernels support at most 16 Q heads per KV head")
    return q.reshape(batch, kv_heads, group, head_dim).contiguous()


def _ungroup_single_query(out: torch.Tensor, q_heads: int) -> torch.Tensor:
    return out.reshape(out.shape[0], q_heads, 1, out.shape[3]).contiguous()

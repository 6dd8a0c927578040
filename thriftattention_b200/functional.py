"""``attention(q, k, v, config=...)`` — the public entry point
(signature and orchestration of the reference's src/thriftattention/functional.py:12-56)."""
from __future__ import annotations

import torch

from thriftattention_b200.backends.registry import select_backend
from thriftattention_b200.config import AttentionConfig
from thriftattention_b200.quant.formats import get_quant_format
from thriftattention_b200.selection import get_selection_policy
from thriftattention_b200.selection.base import SelectionConfig


def attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    *,
    config: AttentionConfig | None = None,
) -> torch.Tensor:
    """q [B,Hq,Sq,D], k/v [B,Hkv,Skv,D] (fp16 or bf16, CUDA) -> [B,Hq,Sq,D]."""
    return _attention(q, k, v, config, seq_major_out=False)


def attention_seq_major(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *,
                        config: AttentionConfig | None = None) -> torch.Tensor:
    """``attention`` with the result laid out ``[B, Sq, Hq, D]`` by the kernel itself: what the Transformers
    hook returns (the reference transposes and copies, integrations/transformers.py:200)."""
    return _attention(q, k, v, config, seq_major_out=True)


def _attention(q, k, v, config, *, seq_major_out: bool) -> torch.Tensor:
    cfg = AttentionConfig() if config is None else config
    is_bf16 = q.dtype == torch.bfloat16
    quant_format = get_quant_format(cfg.quant_format)
    backend = select_backend(cfg, quant_format, head_dim=q.shape[-1], device=q.device)

    selection = None
    if cfg.method == "thrift":
        policy = get_selection_policy(cfg.selection)
        sel_cfg = SelectionConfig(
            name=cfg.selection,
            fraction=cfg.fraction,
            top_k=cfg.top_k,
            block_size=cfg.block_size,
            **_selection_extras(cfg),
        )
        selection = policy.select(q, k, config=sel_cfg, causal=cfg.causal, is_bf16=is_bf16)

    extra = {"seq_major_out": True} if seq_major_out else {}
    return backend.attention(q, k, v, selection=selection, quant_format=quant_format, config=cfg, is_bf16=is_bf16,
                             **extra)


def _selection_extras(cfg: AttentionConfig) -> dict:
    extras = {}
    if getattr(cfg, "sink_blocks", 0):
        extras["sink_blocks"] = cfg.sink_blocks
    if getattr(cfg, "local_blocks", 0):
        extras["local_blocks"] = cfg.local_blocks
    return extras

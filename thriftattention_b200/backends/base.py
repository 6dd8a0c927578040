"""Backend protocol (the reference's src/thriftattention/backends/base.py:11-25)."""
from __future__ import annotations

from typing import Protocol

import torch

from thriftattention_b200.config import AttentionConfig
from thriftattention_b200.quant.formats import QuantFormat


class AttentionBackend(Protocol):
    name: str

    def attention(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, selection: torch.Tensor | None,
                  quant_format: QuantFormat, config: AttentionConfig, is_bf16: bool) -> torch.Tensor: ...

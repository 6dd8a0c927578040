"""Selection configuration and policy protocol
(the reference's src/thriftattention/selection/base.py:11-31)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Protocol

import torch

from thriftattention_b200.config import SelectionMethod


@dataclass(frozen=True)
class SelectionConfig:
    name: SelectionMethod = "block_mean"
    fraction: float | None = 0.05
    top_k: int | None = None
    block_size: int = 64
    # extensions (0 reproduces the reference): always-kept leading / trailing blocks
    sink_blocks: int = 0
    local_blocks: int = 0


class SelectionPolicy(Protocol):
    name: str

    def select(self, q: torch.Tensor, k: torch.Tensor, *, config: SelectionConfig, causal: bool,
               is_bf16: bool) -> torch.Tensor: ...

"""Backend selection (the reference's src/thriftattention/backends/registry.py:12-33).  One
backend exists: sm100.  ``backend="auto"`` resolves to it; there is no fallback."""
from __future__ import annotations

import torch

from thriftattention_b200._checks import require_supported_head_dim
from thriftattention_b200.backends.base import AttentionBackend
from thriftattention_b200.backends.sm100 import SM100_BACKEND
from thriftattention_b200.config import AttentionConfig
from thriftattention_b200.quant.formats import QuantFormat


def select_backend(config: AttentionConfig, quant_format: QuantFormat, *, head_dim: int,
                   device: torch.device | None = None) -> AttentionBackend:
    require_supported_head_dim(head_dim)
    if config.method not in ("thrift", "fp4"):
        raise NotImplementedError(f"attention method {config.method!r} is not implemented")
    if quant_format.name not in ("nvfp4", "mxfp4"):
        raise NotImplementedError(f"quant format {quant_format.name!r} is not implemented")
    if config.backend in ("auto", "sm100"):
        return SM100_BACKEND
    raise NotImplementedError(f"backend {config.backend!r} is not implemented")

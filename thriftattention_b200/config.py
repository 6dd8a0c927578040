"""User-facing configuration (field names and defaults of the reference's
src/thriftattention/config.py:15-26, plus the sm100 extensions noted below)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Literal

AttentionMethod = Literal["thrift", "fp4"]
SelectionMethod = Literal["block_mean", "quest", "local"]
QuantFormatName = Literal["nvfp4", "mxfp4"]
AttentionBackendName = Literal["auto", "sm100"]
AttentionImplementation = Literal["auto", "tiled", "single_query"]
FallbackBackend = Literal["error"]


@dataclass(frozen=True)
class AttentionConfig:
    """How ``attention`` selects, quantises and multiplies.

    ``method``: "thrift" keeps the selected KV blocks in 16-bit and runs the rest in FP4;
    "fp4" quantises everything.  ``fraction``/``top_k`` size the selection (``top_k`` wins).
    ``block_size`` is the selection granularity in tokens: 64 (the reference) or 128.
    Extensions with no reference counterpart: ``sink_blocks`` / ``local_blocks`` always keep
    the first / last valid KV blocks in 16-bit in addition to the scored top-k (0 = off).
    """

    method: AttentionMethod = "thrift"
    causal: bool = True
    selection: SelectionMethod = "block_mean"
    fraction: float | None = 0.05
    top_k: int | None = None
    block_size: int = 64
    quant_format: QuantFormatName = "nvfp4"
    backend: AttentionBackendName = "auto"
    implementation: AttentionImplementation = "auto"
    fallback: FallbackBackend = "error"
    sink_blocks: int = 0
    local_blocks: int = 0

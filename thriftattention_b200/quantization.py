"""FP4 quantiser wrappers (names and checks of the reference's src/thriftattention/quantization.py)."""
from __future__ import annotations

import torch

from ._checks import require_cuda_half, require_supported_head_dim
from ._extension import get_extension


def _run(op: str, x: torch.Tensor, is_bf16: bool) -> tuple[torch.Tensor, torch.Tensor]:
    require_cuda_half("x", x)
    if x.dtype != (torch.bfloat16 if is_bf16 else torch.float16):
        raise ValueError(f"x dtype must match is_bf16={is_bf16}")
    require_supported_head_dim(x.shape[-1])
    packed, scale = getattr(get_extension(), op)(x.contiguous(), is_bf16)
    return packed, scale


def nvfp4_quantize(x: torch.Tensor, *, is_bf16: bool = False):
    """[B,H,S,D] -> (uint8 [B,H,S,D/2], float8_e4m3fn [B,H,S,D/16])."""
    return _run("nvfp4_quantize", x, is_bf16)


def nvfp4_quantize_permuted(x: torch.Tensor, *, is_bf16: bool = False):
    """As ``nvfp4_quantize`` with rows permuted inside every 32-row group (prefill K layout)."""
    return _run("nvfp4_quantize_permuted", x, is_bf16)


def nvfp4_quantize_transposed(x: torch.Tensor, *, is_bf16: bool = False):
    """[B,H,S,D] -> (uint8 [B,H,D,P/2], float8_e4m3fn [B,H,D,P/16]), P = S rounded up to 128 (V layout)."""
    return _run("nvfp4_quantize_transposed", x, is_bf16)


def nvfp4_quantize_transposed_permuted(x: torch.Tensor, *, is_bf16: bool = False):
    return _run("nvfp4_quantize_transposed_permuted", x, is_bf16)


def mxfp4_quantize(x: torch.Tensor, *, is_bf16: bool = False):
    """[B,H,S,D] -> (uint8 [B,H,S,D/2], float8_e8m0fnu [B,H,S,D/32])."""
    return _run("mxfp4_quantize", x, is_bf16)


def mxfp4_quantize_permuted(x: torch.Tensor, *, is_bf16: bool = False):
    return _run("mxfp4_quantize_permuted", x, is_bf16)


def mxfp4_quantize_transposed(x: torch.Tensor, *, is_bf16: bool = False):
    return _run("mxfp4_quantize_transposed", x, is_bf16)


def mxfp4_quantize_transposed_permuted(x: torch.Tensor, *, is_bf16: bool = False):
    return _run("mxfp4_quantize_transposed_permuted", x, is_bf16)

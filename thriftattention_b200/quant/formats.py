"""Quantisation formats and the layout policy for Q, K and V
(the reference's src/thriftattention/quant/formats.py:48-113):

  prefill: Q rows, K rows permuted, V transposed
  decode:  Q rows, K rows (plain),  V transposed
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Protocol

import torch

from thriftattention_b200 import quantization as _q
from thriftattention_b200.config import QuantFormatName

PackedQKV = tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]


class QuantFormat(Protocol):
    name: str

    def quantize(self, x: torch.Tensor, *, is_bf16: bool = False) -> tuple[torch.Tensor, torch.Tensor]: ...

    def quantize_qkv(self, q, k, v, *, is_bf16: bool = False) -> PackedQKV: ...

    def quantize_single_query_qkv(self, q, k, v, *, is_bf16: bool = False) -> PackedQKV: ...


@dataclass(frozen=True)
class _Fp4Format:
    name: QuantFormatName
    group_size: int

    def _op(self, suffix: str):
        return getattr(_q, f"{self.name}_quantize{suffix}")

    def quantize(self, x: torch.Tensor, *, is_bf16: bool = False):
        return self._op("")(x, is_bf16=is_bf16)

    def _pack(self, q, k, v, k_suffix: str, is_bf16: bool) -> PackedQKV:
        if q.is_cuda and all(t.dim() == 4 and t.is_contiguous() for t in (q, k, v)) and k.shape == v.shape:
            from thriftattention_b200 import _C          # one launch for the three tensors
            return _C.quantize_qkv(q, k, v, is_mx=self.name == "mxfp4", is_bf16=is_bf16, k_permuted=k_suffix == "_permuted")
        q_packed, q_scale = self._op("")(q, is_bf16=is_bf16)
        k_packed, k_scale = self._op(k_suffix)(k, is_bf16=is_bf16)
        v_packed_t, v_scale_t = self._op("_transposed")(v, is_bf16=is_bf16)
        return q_packed, k_packed, v_packed_t, q_scale, k_scale, v_scale_t

    def quantize_qkv(self, q, k, v, *, is_bf16: bool = False) -> PackedQKV:
        return self._pack(q, k, v, "_permuted", is_bf16)

    def quantize_single_query_qkv(self, q, k, v, *, is_bf16: bool = False) -> PackedQKV:
        return self._pack(q, k, v, "", is_bf16)


class Nvfp4QuantFormat(_Fp4Format):
    def __init__(self) -> None:
        super().__init__(name="nvfp4", group_size=16)


class Mxfp4QuantFormat(_Fp4Format):
    def __init__(self) -> None:
        super().__init__(name="mxfp4", group_size=32)


_FORMATS = {"nvfp4": Nvfp4QuantFormat(), "mxfp4": Mxfp4QuantFormat()}


def get_quant_format(name: QuantFormatName) -> QuantFormat:
    try:
        return _FORMATS[name]
    except KeyError:
        raise NotImplementedError(f"quant format {name!r} is not implemented") from None

"""The sm_100a backend: quantise with the format's layout policy, then one fused kernel for
prefill (tiled) or the split-KV kernel for decode (single query).  Same protocol and call
sequence as the reference's SM120 backend (src/thriftattention/backends/sm120.py:17-134); the
operator names called on the extension are the reference's."""
from __future__ import annotations

import torch

from thriftattention_b200._checks import check_qkv, require_block_aligned
from thriftattention_b200._extension import get_extension
from thriftattention_b200.backends.single_query import (
    _group_single_query,
    _ungroup_single_query,
    _use_single_query,
)
from thriftattention_b200.config import AttentionConfig
from thriftattention_b200.quant.formats import QuantFormat

SUPPORTED_BLOCK_SIZES = (64, 128)


class Sm100Backend:
    name = "sm100"

    def attention(self, q, k, v, *, selection, quant_format: QuantFormat, config: AttentionConfig,
                  is_bf16: bool, seq_major_out: bool = False) -> torch.Tensor:
        """``seq_major_out`` returns ``[B, Sq, Hq, D]`` straight from the kernel epilogue (tiled path) or as a
        view (single query) instead of ``[B, Hq, Sq, D]``."""
        check_qkv(q, k, v)
        if config.block_size not in SUPPORTED_BLOCK_SIZES:
            raise NotImplementedError("the sm100 attention kernels use 64- or 128-token KV blocks")
        if quant_format.name not in ("nvfp4", "mxfp4"):
            raise NotImplementedError(f"sm100 backend does not support quant format {quant_format.name!r}")
        if config.method not in ("thrift", "fp4"):
            raise ValueError(f"unsupported attention method {config.method!r}")
        if config.method == "thrift" and selection is None:
            raise ValueError("thrift attention requires a selection tensor")
        if _use_single_query(q, config.implementation):
            out = self._single_query_attention(q, k, v, selection, quant_format, config, is_bf16)
            return out.reshape(out.shape[0], 1, out.shape[1], out.shape[3]) if seq_major_out else out
        return self._tiled_attention(q, k, v, selection, quant_format, config, is_bf16, seq_major_out)

    # ------------------------------------------------------------------ decode
    def _single_query_attention(self, q, k, v, selection, quant_format, config, is_bf16):
        if config.block_size != 64:
            raise NotImplementedError("single-query attention selects 64-token pages")
        require_block_aligned("k", k.shape[2], config.block_size)
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        q_grouped = _group_single_query(q, k.shape[1])
        packed = quant_format.quantize_single_query_qkv(q_grouped, k, v, is_bf16=is_bf16)
        ext = get_extension()
        fmt = quant_format.name
        if config.method == "fp4":
            out = getattr(ext, f"fp4_attention_single_query_{fmt}_packed")(*packed, is_bf16)
        else:
            out = getattr(ext, f"thrift_attention_single_query_{fmt}_packed")(q_grouped, k, v, selection, *packed,
                                                                             is_bf16)
        return _ungroup_single_query(out, q.shape[1])

    # ------------------------------------------------------------------ prefill
    def _tiled_attention(self, q, k, v, selection, quant_format, config, is_bf16, seq_major_out=False):
        require_block_aligned("q", q.shape[2], 64)
        require_block_aligned("k", k.shape[2], config.block_size)
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        packed = quant_format.quantize_qkv(q, k, v, is_bf16=is_bf16)
        ext = get_extension()
        fmt = quant_format.name
        mode = "causal" if config.causal else "noncausal"
        if seq_major_out:
            sel = selection if config.method == "thrift" else None
            hi = (q, k, v) if sel is not None else (None, None, None)
            return ext.prefill_attention(*hi, sel, *packed, causal=config.causal, is_mx=(fmt == "mxfp4"),
                                         is_bf16=is_bf16, block_size=config.block_size, k_permuted=True,
                                         seq_major_out=True)
        if config.method == "fp4":
            return getattr(ext, f"fp4_attention_{mode}_{fmt}_packed")(*packed, is_bf16)
        if config.block_size == 64:
            return getattr(ext, f"thrift_attention_{mode}_{fmt}_packed")(q, k, v, selection, *packed, is_bf16)
        # 128-token selection blocks: extension entry point (the reference-named operators fix 64)
        return ext.prefill_attention(q, k, v, selection, *packed, causal=config.causal, is_mx=(fmt == "mxfp4"),
                                     is_bf16=is_bf16, block_size=config.block_size, k_permuted=True)


SM100_BACKEND = Sm100Backend()

"""Operator module: the callables the reference exports from its compiled
``thriftattention._C`` extension (csrc/bindings.cpp:1454-1671), implemented over the
C ABI of ``libthrift_sm100.so``.

Names, positional argument order, argument meaning and error conditions follow the
reference bindings; outputs and workspaces are allocated here with torch and handed
to the library as raw pointers together with the current CUDA stream.  Errors from
argument checks are ``RuntimeError`` like the reference's ``TORCH_CHECK`` failures.

Additions (no reference counterpart, used by the sm100 backend): ``block_stats``,
``select_prefill_blocks``, ``select_decode_blocks``, ``pack_topk_mask``,
``prefill_attention``, ``decode_attention`` and ``merge_decode_partials``.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

_lib.load()  # fail at import time when the CUDA library is missing


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _ptr(t: torch.Tensor | None):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(t: torch.Tensor):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _scale_dtype(is_mx: bool):
    return torch.float8_e8m0fnu if is_mx else torch.float8_e4m3fn


# ---------------------------------------------------------------------------------------------
# Quantisers  (bindings.cpp:893-1097)
# ---------------------------------------------------------------------------------------------
def _quantize(x: torch.Tensor, is_bf16: bool, is_mx: bool, layout: int):
    _check(x.is_cuda, "x must be a CUDA tensor")
    _check(x.is_contiguous(), "x must be contiguous")
    _check(x.dim() == 4, "x must be 4D [batch, heads, seq, head_dim]")
    b, h, s, d = x.shape
    _check(d in (64, 128), f"head_dim must be 64 or 128, got {d}")
    _check(x.dtype == (torch.bfloat16 if is_bf16 else torch.float16), "x dtype must match is_bf16")
    g = 32 if is_mx else 16
    if layout >= 2:
        padded = (s + 127) // 128 * 128
        codes = torch.empty(b, h, d, padded // 2, dtype=torch.uint8, device=x.device)
        scales = torch.empty(b, h, d, padded // g, dtype=torch.uint8, device=x.device)
    else:
        codes = torch.empty(b, h, s, d // 2, dtype=torch.uint8, device=x.device)
        scales = torch.empty(b, h, s, d // g, dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.load().ta100_quantize(_ptr(x), _ptr(codes), _ptr(scales), b * h, s, d, int(is_mx), int(is_bf16),
                                        layout, _stream(x))
    _lib.check(rc, "quantize")
    return [codes, scales.view(_scale_dtype(is_mx))]


def quantize_qkv(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, is_mx: bool, is_bf16: bool, k_permuted: bool):
    """Q (rows), K (rows, permuted for the prefill kernel if ``k_permuted``) and V (transposed) in one launch; returns
    ``(q_codes, k_codes, v_codes_t, q_scales, k_scales, v_scales_t)`` - the order of ``QuantFormat.quantize_qkv``
    (src/thriftattention/quant/formats.py:55-79 of the reference, three launches there)."""
    for name, x in (("q", q), ("k", k), ("v", v)):
        _check(x.is_cuda and x.is_contiguous() and x.dim() == 4, f"{name} must be a contiguous 4D CUDA tensor")
        _check(x.dtype == (torch.bfloat16 if is_bf16 else torch.float16), f"{name} dtype must match is_bf16")
    _check(k.shape == v.shape, "k and v must have the same shape")
    _check(q.shape[0] == k.shape[0] and q.shape[3] == k.shape[3], "q and k must agree in batch and head_dim")
    b, hq, sq, d = q.shape
    _, hkv, skv, _ = k.shape
    _check(d in (64, 128), f"head_dim must be 64 or 128, got {d}")
    g = 32 if is_mx else 16
    padded = (skv + 127) // 128 * 128
    u8 = dict(dtype=torch.uint8, device=q.device)
    q4, qs = torch.empty(b, hq, sq, d // 2, **u8), torch.empty(b, hq, sq, d // g, **u8)
    k4, ks = torch.empty(b, hkv, skv, d // 2, **u8), torch.empty(b, hkv, skv, d // g, **u8)
    v4, vs = torch.empty(b, hkv, d, padded // 2, **u8), torch.empty(b, hkv, d, padded // g, **u8)
    with torch.cuda.device(q.device):
        rc = _lib.load().ta100_quantize_qkv(_ptr(q), _ptr(k), _ptr(v), _ptr(q4), _ptr(qs), _ptr(k4), _ptr(ks), _ptr(v4),
                                            _ptr(vs), b * hq, sq, b * hkv, skv, d, int(is_mx), int(is_bf16),
                                            int(k_permuted), _stream(q))
    _lib.check(rc, "quantize_qkv")
    sd = _scale_dtype(is_mx)
    return q4, k4, v4, qs.view(sd), ks.view(sd), vs.view(sd)


def nvfp4_quantize(x, is_bf16=False):
    return _quantize(x, is_bf16, False, 0)


def nvfp4_quantize_permuted(x, is_bf16=False):
    return _quantize(x, is_bf16, False, 1)


def nvfp4_quantize_transposed(x, is_bf16=False):
    return _quantize(x, is_bf16, False, 2)


def nvfp4_quantize_transposed_permuted(x, is_bf16=False):
    return _quantize(x, is_bf16, False, 3)


def mxfp4_quantize(x, is_bf16=False):
    return _quantize(x, is_bf16, True, 0)


def mxfp4_quantize_permuted(x, is_bf16=False):
    return _quantize(x, is_bf16, True, 1)


def mxfp4_quantize_transposed(x, is_bf16=False):
    return _quantize(x, is_bf16, True, 2)


def mxfp4_quantize_transposed_permuted(x, is_bf16=False):
    return _quantize(x, is_bf16, True, 3)


# ---------------------------------------------------------------------------------------------
# Block statistics and selection  (bindings.cpp:1100-1452)
# ---------------------------------------------------------------------------------------------
def block_stats(x: torch.Tensor, block_size: int, *, mean=False, minmax=False):
    """Per-block fp32 mean (cast to x.dtype), min and max of ``x`` [B,H,S,D] in one pass.

    Fuses the PyTorch pre-reductions of the reference (selection/block_mean.py:44-54,
    selection/quest.py:11-24) without materialising an fp32 copy.  Returns a tuple
    ``(mean|None, min|None, max|None)`` of [B,H,S/block,D] tensors.
    """
    _check(x.is_cuda and x.is_contiguous() and x.dim() == 4, "x must be a contiguous 4D CUDA tensor")
    b, h, s, d = x.shape
    _check(d in (64, 128), f"head_dim must be 64 or 128, got {d}")
    _check(s % block_size == 0, f"sequence length must be divisible by {block_size}")
    nb = s // block_size
    mk = lambda: torch.empty(b, h, nb, d, dtype=x.dtype, device=x.device)
    o_mean = mk() if mean else None
    o_min = mk() if minmax else None
    o_max = mk() if minmax else None
    with torch.cuda.device(x.device):
        rc = _lib.load().ta100_block_stats(_ptr(x), _ptr(o_mean), _ptr(o_min), _ptr(o_max), b * h, s, d, block_size,
                                           int(x.dtype == torch.bfloat16), _stream(x))
    _lib.check(rc, "block_stats")
    return o_mean, o_min, o_max


def cache_append(k_new, v_new, k_hi, v_hi, k_codes, k_scales, v_codes_t, v_scales_t, *, start, k_count=None, v_count=None,
                 k_mean=None, k_min=None, k_max=None, is_mx=False, stat_block=64, keep_k=False, keep_v=False,
                 trusted=False):
    """Fused KV-cache append (one launch): stores ``k_new`` / ``v_new`` [B, H, T, D] at token positions
    ``[start, start + T)`` of the capacity-strided caches ``k_hi`` / ``v_hi`` [B, H, cap, D], quantises the
    new K rows, re-quantises the V groups they touch and refreshes the statistics of completed blocks.

    ``k_new`` / ``v_new`` may be ``None`` with an explicit count: zero rows are stored, or with
    ``keep_k`` / ``keep_v`` the cached rows are kept and only re-quantised.  Stands in for
    ``ThriftAttentionCacheLayer.update`` and its three helpers
    (integrations/transformers_cache.py:87-123, 308-351).  ``trusted`` skips the shape checks: the cache layer
    that owns all of these buffers calls it once per layer and token, where the checks cost more than the launch.
    """
    b, h, cap, d = k_hi.shape
    is_bf16 = k_hi.dtype == torch.bfloat16
    if trusted:
        vp = ctypes.c_void_p
        ptr = lambda t: None if t is None else vp(t.data_ptr())
        k_count = k_new.shape[2] if k_new is not None else int(k_count or 0)
        v_count = v_new.shape[2] if v_new is not None else int(v_count or 0)
        with torch.cuda.device(k_hi.device):
            rc = _lib.load().ta100_cache_append(ptr(k_new), ptr(v_new), ptr(k_hi), ptr(v_hi), ptr(k_codes), ptr(k_scales),
                                                ptr(v_codes_t), ptr(v_scales_t), ptr(k_mean), ptr(k_min), ptr(k_max),
                                                b * h, int(start), k_count, v_count, cap, d, stat_block, int(is_mx),
                                                int(is_bf16), (1 if keep_k else 0) | (2 if keep_v else 0),
                                                vp(torch.cuda.current_stream(k_hi.device).cuda_stream))
        if rc:
            _lib.check(rc, "cache_append")
        return
    _check(k_hi.is_cuda and k_hi.dim() == 4 and k_hi.is_contiguous(), "k cache must be a contiguous 4D CUDA tensor")
    _check(k_hi.dtype in (torch.float16, torch.bfloat16), "KV cache tensors must be float16 or bfloat16")
    g = 32 if is_mx else 16
    for name, new, count in (("key_states", k_new, k_count), ("value_states", v_new, v_count)):
        if new is not None:
            _check(new.is_cuda and new.is_contiguous() and new.dtype == k_hi.dtype, f"{name} must be contiguous CUDA tensors "
                   "of the cache dtype")
            _check(new.dim() == 4 and new.shape[0] == b and new.shape[1] == h and new.shape[3] == d,
                   f"{name} must be [batch, heads, tokens, head_dim] matching the cache")
            _check(count is None or count == new.shape[2], f"{name} count does not match its tensor")
    k_count = k_new.shape[2] if k_new is not None else int(k_count or 0)
    v_count = v_new.shape[2] if v_new is not None else int(v_count or 0)
    expect = {"v_hi": (v_hi, (b, h, cap, d)), "k_codes": (k_codes, (b, h, cap, d // 2)),
              "k_scales": (k_scales, (b, h, cap, d // g)), "v_codes_t": (v_codes_t, (b, h, d, cap // 2)),
              "v_scales_t": (v_scales_t, (b, h, d, cap // g))}
    for name, (t, shape) in expect.items():
        _check(t.is_cuda and t.is_contiguous() and tuple(t.shape) == shape, f"{name} must be contiguous {shape}")
    for name, t in (("k_mean", k_mean), ("k_min", k_min), ("k_max", k_max)):
        _check(t is None or (t.is_cuda and t.is_contiguous() and tuple(t.shape) == (b, h, cap // stat_block, d)
                             and t.dtype == k_hi.dtype), f"{name} must be contiguous [B, H, cap/{stat_block}, D] of the cache dtype")
    flags = (1 if keep_k else 0) | (2 if keep_v else 0)
    with torch.cuda.device(k_hi.device):
        rc = _lib.load().ta100_cache_append(_ptr(k_new), _ptr(v_new), _ptr(k_hi), _ptr(v_hi), _ptr(k_codes), _ptr(k_scales),
                                            _ptr(v_codes_t), _ptr(v_scales_t), _ptr(k_mean), _ptr(k_min), _ptr(k_max),
                                            b * h, int(start), k_count, v_count, cap, d, stat_block, int(is_mx),
                                            int(is_bf16), flags, _stream(k_hi))
    _lib.check(rc, "cache_append")


def cache_append_paged(k_new, v_new, k_hi, v_hi, k_codes, k_scales, v_codes, v_scales, page_table, *, start, k_count=None,
                       v_count=None, k_mean=None, k_min=None, k_max=None, is_mx=False, stat_block=64, keep_k=False,
                       keep_v=False):
    """``cache_append`` into page pools behind ``page_table`` int32 [B, max_pages] (the layout ``decode_attention``
    reads): ``k_hi`` / ``v_hi`` [pool, Hkv, 64, D], ``k_codes`` [pool, Hkv, 64, D/2], ``v_codes`` [pool, Hkv, D, 32] and
    their scales; statistics [B, Hkv, blocks, D] by logical block.  ``k_new`` / ``v_new`` [B, Hkv, T, D]."""
    _check(k_hi.is_cuda and k_hi.dim() == 4 and k_hi.is_contiguous() and k_hi.shape[2] == 64,
           "k pool must be a contiguous CUDA tensor [pool_pages, kv_heads, 64, head_dim]")
    pool, hkv, _, d = k_hi.shape
    _check(k_hi.dtype in (torch.float16, torch.bfloat16), "KV cache tensors must be float16 or bfloat16")
    is_bf16 = k_hi.dtype == torch.bfloat16
    g = 32 if is_mx else 16
    _check(page_table.is_cuda and page_table.dtype == torch.int32 and page_table.dim() == 2 and page_table.is_contiguous(),
           "page_table must be a contiguous int32 CUDA tensor [batch, max_pages]")
    b, max_pages = page_table.shape
    expect = {"v_hi": (v_hi, (pool, hkv, 64, d)), "k_codes": (k_codes, (pool, hkv, 64, d // 2)),
              "k_scales": (k_scales, (pool, hkv, 64, d // g)), "v_codes": (v_codes, (pool, hkv, d, 32)),
              "v_scales": (v_scales, (pool, hkv, d, 64 // g))}
    for name, (t, shape) in expect.items():
        _check(t.is_cuda and t.is_contiguous() and tuple(t.shape) == shape, f"{name} must be contiguous {shape}")
    for name, new, count in (("key_states", k_new, k_count), ("value_states", v_new, v_count)):
        if new is not None:
            _check(new.is_cuda and new.is_contiguous() and new.dtype == k_hi.dtype and new.dim() == 4
                   and new.shape[0] == b and new.shape[1] == hkv and new.shape[3] == d,
                   f"{name} must be contiguous [batch, kv_heads, tokens, head_dim] CUDA tensors of the cache dtype")
            _check(count is None or count == new.shape[2], f"{name} count does not match its tensor")
    k_count = k_new.shape[2] if k_new is not None else int(k_count or 0)
    v_count = v_new.shape[2] if v_new is not None else int(v_count or 0)
    _check(int(start) + max(k_count, v_count) <= max_pages * 64, "the token range exceeds the page table")
    stat_blocks = 1
    for name, t in (("k_mean", k_mean), ("k_min", k_min), ("k_max", k_max)):
        if t is not None:
            _check(t.is_cuda and t.is_contiguous() and t.dim() == 4 and t.shape[0] == b and t.shape[1] == hkv and t.shape[3] == d
                   and t.dtype == k_hi.dtype, f"{name} must be contiguous [B, Hkv, blocks, D] of the cache dtype")
            stat_blocks = t.shape[2]
    flags = (1 if keep_k else 0) | (2 if keep_v else 0)
    with torch.cuda.device(k_hi.device):
        rc = _lib.load().ta100_cache_append_paged(_ptr(k_new), _ptr(v_new), _ptr(k_hi), _ptr(v_hi), _ptr(k_codes),
                                                  _ptr(k_scales), _ptr(v_codes), _ptr(v_scales), _ptr(k_mean), _ptr(k_min),
                                                  _ptr(k_max), _ptr(page_table), max_pages, pool, b, hkv, stat_blocks,
                                                  int(start), k_count, v_count, d, stat_block, int(is_mx), int(is_bf16),
                                                  flags, _stream(k_hi))
    _lib.check(rc, "cache_append_paged")


def select_prefill_blocks(q_mean, k_a, k_b, topk_count, causal=True, is_bf16=False, sink=0, local=0):
    """Per-q-block selection.  ``k_b is None`` -> block-mean score with ``k_a = k_mean``;
    otherwise Quest with ``k_a = k_min``, ``k_b = k_max``.  K statistics may be given per
    KV head ([B,Hkv,nk,D]) or already expanded per Q head.  ``sink``/``local`` force the
    first/last valid blocks (extension; 0 reproduces the reference)."""
    ts = [q_mean, k_a] + ([k_b] if k_b is not None else [])
    _check(all(t.is_cuda for t in ts), "selection inputs must be CUDA tensors")
    _check(all(t.is_contiguous() for t in ts), "selection inputs must be contiguous")
    _check(all(t.dim() == 4 for t in ts), "selection inputs must be 4D tensors")
    _check(k_b is None or k_a.shape == k_b.shape, "k_min and k_max shapes must match")
    _check(q_mean.size(0) == k_a.size(0), "batch dimensions must match")
    _check(q_mean.size(1) % k_a.size(1) == 0, "q heads must be divisible by key stat heads")
    _check(q_mean.size(3) == k_a.size(3), "head_dim must match")
    b, hq, nq, d = q_mean.shape
    nk = k_a.size(2)
    _check(d in (64, 128), f"head_dim must be 64 or 128, got {d}")
    _check(nk <= 2048, f"block selector supports <= 2048 KV blocks, got {nk}")
    _check(0 <= topk_count <= nk, "topk_count must be in [0, num_kv_blocks]")
    width = sink + local + topk_count
    out = torch.empty(b * hq, nq, width, dtype=torch.int32, device=q_mean.device)
    if width == 0:
        return out
    with torch.cuda.device(q_mean.device):
        rc = _lib.load().ta100_select_prefill(_ptr(q_mean), _ptr(k_a), _ptr(k_b), _ptr(out), b * hq, hq // k_a.size(1),
                                              nq, nk, d, topk_count, int(causal), int(k_b is not None), int(is_bf16),
                                              sink, local, _stream(q_mean))
    _lib.check(rc, "select_prefill")
    return out


def block_mean_topk(q_mean, k_mean, topk_count, causal=True, is_bf16=False):
    return select_prefill_blocks(q_mean, k_mean, None, topk_count, causal, is_bf16)


def quest_block_topk(q_mean, k_min, k_max, topk_count, causal=True, is_bf16=False):
    return select_prefill_blocks(q_mean, k_min, k_max, topk_count, causal, is_bf16)


def select_decode_blocks(q_grouped, k_a, k_b, topk_count, num_kv_blocks, is_bf16=False, sink=0, local=0, out=None,
                         return_scores=False, scores_out=None, row_width=None):
    """Decode selection; with ``return_scores`` also the fp32 score of every pick (forced blocks +FLT_MAX,
    padding -FLT_MAX), bit-identical to what the kernel ranked by.  ``out`` / ``scores_out`` let the caller
    supply the two result buffers (e.g. the two planes of one buffer that is all-gathered afterwards);
    ``row_width`` >= sink + local + topk_count makes the rows that wide, the tail being padding."""
    ts = [q_grouped, k_a] + ([k_b] if k_b is not None else [])
    _check(all(t.is_cuda for t in ts), "selection inputs must be CUDA tensors")
    _check(all(t.is_contiguous() for t in ts), "selection inputs must be contiguous")
    _check(all(t.dim() == 4 for t in ts), "selection inputs must be 4D tensors")
    _check(k_b is None or k_a.shape == k_b.shape, "k_min and k_max shapes must match")
    _check(q_grouped.size(0) == k_a.size(0), "batch dimensions must match")
    _check(q_grouped.size(1) == k_a.size(1), "KV-head dimensions must match")
    _check(q_grouped.size(3) == k_a.size(3), "head_dim must match")
    b, hkv, groups, d = q_grouped.shape
    cap = k_a.size(2)
    _check(1 <= groups <= 16, f"grouped single-query selector expects groups in [1, 16], got {groups}")
    _check(d in (64, 128), f"head_dim must be 64 or 128, got {d}")
    _check(0 <= num_kv_blocks <= cap, "num_kv_blocks must be in [0, key stat capacity]")
    _check(num_kv_blocks <= 2048, f"single-query block selector supports <= 2048 KV blocks, got {num_kv_blocks}")
    _check(0 <= topk_count <= num_kv_blocks, "topk_count must be in [0, num_kv_blocks]")
    used = sink + local + topk_count
    width = used if row_width is None else row_width
    _check(width >= used, "row_width must cover sink + local + topk_count")
    if out is None:
        out = torch.empty(b * hkv, width, dtype=torch.int32, device=q_grouped.device)
    scores = None
    if return_scores:
        scores = scores_out if scores_out is not None else torch.empty(b * hkv, width, dtype=torch.float32,
                                                                      device=q_grouped.device)
        _check(scores.is_cuda and scores.dtype == torch.float32 and scores.is_contiguous()
               and tuple(scores.shape) == (b * hkv, width), "scores_out must be contiguous fp32 [batch * kv_heads, width]")
    _check(out.is_cuda and out.dtype == torch.int32 and out.is_contiguous() and tuple(out.shape) == (b * hkv, width),
           "out must be contiguous int32 [batch * kv_heads, width]")
    if used == 0:
        if width:
            out.fill_(-1)
            if scores is not None:
                scores.fill_(-3.4028234663852886e38)
        return (out, scores) if return_scores else out
    with torch.cuda.device(q_grouped.device):
        rc = _lib.load().ta100_select_decode(_ptr(q_grouped), _ptr(k_a), _ptr(k_b), _ptr(out), _ptr(scores), b * hkv, groups,
                                             num_kv_blocks, cap, d, topk_count, int(k_b is not None), int(is_bf16),
                                             sink, local, width, _stream(q_grouped))
    _lib.check(rc, "select_decode")
    return (out, scores) if return_scores else out


def merge_page_candidates(gathered, *, rank, total_pages, top_k, sink=0, local=0):
    """Global decode selection from the all-gathered candidate buffers of every KV-sequence shard.

    ``gathered`` int32 ``[world, 2, rows, width]``: per shard the page ids (local to the shard) and the bit
    patterns of their fp32 scores as written by ``select_decode_blocks(..., return_scores=True)``.  Returns int32
    ``[rows, sink + local + top_k]`` local page ids of shard ``rank``'s part of the global selection
    (its forced pages first, -1 where a pick belongs to another shard)."""
    _check(gathered.is_cuda and gathered.dtype == torch.int32 and gathered.is_contiguous() and gathered.dim() == 4
           and gathered.size(1) == 2, "gathered must be contiguous int32 [world, 2, rows, width]")
    world, _, rows, width = gathered.shape
    out = torch.empty(rows, sink + local + top_k, dtype=torch.int32, device=gathered.device)
    with torch.cuda.device(gathered.device):
        rc = _lib.load().ta100_merge_page_candidates(_ptr(gathered), _ptr(out), rows, world, width, rank, total_pages,
                                                     top_k, sink, local, _stream(gathered))
    _lib.check(rc, "merge_page_candidates")
    return out


def single_query_key_mean_topk(q_grouped, k_mean, topk_count, num_kv_blocks, is_bf16=False):
    return select_decode_blocks(q_grouped, k_mean, None, topk_count, num_kv_blocks, is_bf16)


def single_query_quest_topk(q_grouped, k_min, k_max, topk_count, num_kv_blocks, is_bf16=False):
    return select_decode_blocks(q_grouped, k_min, k_max, topk_count, num_kv_blocks, is_bf16)


def single_query_key_mean_topk_into(q_grouped, k_mean, topk, local_scores, local_indices, done_counts, num_kv_blocks,
                                    is_bf16=False):
    """Writes the selection into the caller's ``topk`` tensor.  The three workspace tensors of
    the reference's chunked variant are accepted and validated but not needed: one CTA per
    KV head scores all blocks and selects in place."""
    for t in (topk, local_scores, local_indices, done_counts):
        _check(t.is_cuda and t.is_contiguous(), "top-k workspace tensors must be contiguous CUDA tensors")
    _check(topk.dtype == torch.int32 and local_indices.dtype == torch.int32 and done_counts.dtype == torch.int32,
           "topk, local_indices, and done_counts must be int32")
    _check(local_scores.dtype == torch.float32, "local_scores must be float32")
    flat = q_grouped.size(0) * q_grouped.size(1)
    _check(topk.dim() == 2 and topk.size(0) == flat, "topk must be shaped [batch * kv_heads, topk_count]")
    _check(done_counts.dim() == 1 and done_counts.size(0) == flat, "done_counts must be shaped [batch * kv_heads]")
    return select_decode_blocks(q_grouped, k_mean, None, topk.size(1), num_kv_blocks, is_bf16, out=topk)


def local_block_topk(q, num_kv_blocks, topk_count, causal=True, block_size=64):
    _check(q.is_cuda, "q must be a CUDA tensor")
    _check(q.dim() == 4, "q must be 4D [batch, heads, seq, head_dim]")
    _check(block_size > 0 and q.size(2) % block_size == 0, "q sequence length must be divisible by block_size")
    _check(0 <= topk_count <= num_kv_blocks, "topk_count must be in [0, num_kv_blocks]")
    flat, nq = q.size(0) * q.size(1), q.size(2) // block_size
    out = torch.empty(flat, nq, topk_count, dtype=torch.int32, device=q.device)
    with torch.cuda.device(q.device):
        rc = _lib.load().ta100_local_block_topk(_ptr(out), flat, nq, num_kv_blocks, topk_count, int(causal), _stream(q))
    _lib.check(rc, "local_block_topk")
    return out


def single_query_local_topk(q_grouped, topk_count, num_kv_blocks):
    _check(q_grouped.is_cuda, "q_grouped must be a CUDA tensor")
    _check(q_grouped.dim() == 4, "q_grouped must be 4D [batch, kv_heads, groups, head_dim]")
    _check(0 <= topk_count <= num_kv_blocks, "topk_count must be in [0, num_kv_blocks]")
    flat = q_grouped.size(0) * q_grouped.size(1)
    out = torch.empty(flat, topk_count, dtype=torch.int32, device=q_grouped.device)
    with torch.cuda.device(q_grouped.device):
        rc = _lib.load().ta100_single_query_local_topk(_ptr(out), flat, num_kv_blocks, topk_count, _stream(q_grouped))
    _lib.check(rc, "single_query_local_topk")
    return out


def pack_topk_mask(selected_blocks: torch.Tensor, num_kv_blocks: int) -> torch.Tensor:
    """Index list [..., k] -> int64 bitset [..., ceil(nk/64)] (bindings.cpp:537-542)."""
    _check(selected_blocks.is_cuda and selected_blocks.is_contiguous() and selected_blocks.dtype == torch.int32,
           "selected_blocks must be a contiguous int32 CUDA tensor")
    words = (num_kv_blocks + 63) // 64
    _check(words <= 32, f"at most 2048 KV blocks are supported, got {num_kv_blocks}")
    k = selected_blocks.size(-1)
    rows = selected_blocks.numel() // k if k else int(torch.Size(selected_blocks.shape[:-1]).numel())
    mask = torch.zeros(*selected_blocks.shape[:-1], words, dtype=torch.int64, device=selected_blocks.device)
    if k == 0 or rows == 0:
        return mask
    with torch.cuda.device(mask.device):
        rc = _lib.load().ta100_pack_topk_mask(_ptr(selected_blocks), _ptr(mask), rows, k, num_kv_blocks, words,
                                              _stream(mask))
    _lib.check(rc, "pack_topk_mask")
    return mask


# ---------------------------------------------------------------------------------------------
# Prefill attention  (bindings.cpp:249-292, 487-695)
# ---------------------------------------------------------------------------------------------
def _check_hi(q, k, v):
    _check(q.is_cuda and k.is_cuda and v.is_cuda, "Q/K/V must be CUDA tensors")
    _check(q.dim() == 4 and k.dim() == 4 and v.dim() == 4, "Q/K/V must be 4D [batch, heads, seq, head_dim]")
    _check(q.size(0) == k.size(0) == v.size(0), "Q/K/V batch dimensions must match")
    _check(k.size(1) == v.size(1), "K and V head dimensions must match")
    _check(k.size(2) == v.size(2), "K and V sequence lengths must match")
    _check(q.size(3) == k.size(3) == v.size(3), "Q/K/V head dimensions must match")


def _check_packed(q_packed, k_packed, v_packed_t, q_scale, k_scale, v_scale_t):
    _check(q_packed.is_cuda and k_packed.is_cuda and v_packed_t.is_cuda, "packed Q/K/V must be CUDA tensors")
    _check(q_scale.is_cuda and k_scale.is_cuda and v_scale_t.is_cuda, "Q/K/V scales must be CUDA tensors")
    _check(q_packed.dim() == 4 and k_packed.dim() == 4 and v_packed_t.dim() == 4, "packed Q/K/V must be 4D tensors")
    _check(q_packed.size(0) == k_packed.size(0), "packed Q/K batch dimensions must match")
    _check(q_packed.size(1) % k_packed.size(1) == 0, "Q heads must be divisible by KV heads")
    _check(q_packed.size(3) == k_packed.size(3), "packed Q/K head dimensions must match")


_workspaces: dict = {}


def _workspace(device, nbytes: int) -> torch.Tensor:
    """Per-(device, stream) scratch buffer, grown on demand and reused across calls."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


_prefill_event_sink = None


def set_prefill_event_sink(sink) -> None:
    """``sink`` = a list: every later ``prefill_attention`` call appends a (start, end) pair of CUDA events recorded
    on the launching stream around the library call (scale re-tiling + the attention kernel), so that a caller of
    the public API can time the kernel itself.  ``None`` switches the recording off."""
    global _prefill_event_sink
    _prefill_event_sink = sink


def prefill_attention(q_hi, k_hi, v_hi, selected_blocks, q_packed, k_packed, v_packed_t, q_scale, k_scale, v_scale_t, *,
                      causal, is_mx, is_bf16=False, block_size=64, k_permuted=True, round_partial=True, max_ctas=0,
                      check_status=False, seq_major_out=False):
    """Fused mixed-precision prefill attention (one kernel for the FP4 pass and the 16-bit pass).

    ``selected_blocks`` is ``None`` (pure FP4) or int32 ``[B*Hq, Sq/block_size, W]`` with -1
    padding.  ``k_permuted`` says whether ``k_packed`` uses the reference's row-permuted layout.
    ``seq_major_out`` makes the kernel epilogue write ``[B, Sq, Hq, D]`` (what a Transformers attention
    function returns) instead of ``[B, Hq, Sq, D]``.
    """
    _check_packed(q_packed, k_packed, v_packed_t, q_scale, k_scale, v_scale_t)
    b, hq, sq, dh = q_packed.shape
    hkv, skv = k_packed.size(1), k_packed.size(2)
    d = dh * 2
    _check(q_packed.is_contiguous() and q_scale.is_contiguous(), "packed Q and its scales must be contiguous")
    _check(k_packed.stride(3) == 1 and k_packed.stride(2) == dh, "packed K rows must be dense")
    kv_cap = k_packed.stride(1) // dh if hkv > 1 or b > 1 else max(skv, k_packed.stride(1) // dh)
    width = 0
    if selected_blocks is not None:
        _check_hi(q_hi, k_hi, v_hi)
        _check(selected_blocks.is_cuda, "selected_blocks must be a CUDA tensor")
        _check(selected_blocks.dtype == torch.int32, "selected_blocks must be int32")
        _check(selected_blocks.is_contiguous(), "selected_blocks must be contiguous")
        _check(selected_blocks.dim() == 3, "selected_blocks must be [batch * heads, q_blocks, top_k]")
        _check(selected_blocks.size(0) == b * hq, "selected_blocks first dimension must equal batch * Q heads")
        _check(selected_blocks.size(1) == (sq + block_size - 1) // block_size,
               "selected_blocks second dimension must equal number of Q blocks")
        _check((skv + 63) // 64 <= 2048, f"ThriftAttention supports at most 2048 64-token KV blocks, got {(skv + 63) // 64}")
        width = selected_blocks.size(2)
        _check(q_hi.is_contiguous(), "Q must be contiguous")
        want = (hkv * kv_cap * d, kv_cap * d, d, 1)
        for t in (k_hi, v_hi):
            _check((t.is_contiguous() and t.size(2) == kv_cap) or tuple(t.stride()) == want,
                   "16-bit K/V must be contiguous or views of a cache with the packed K's capacity")
    out = torch.empty((b, sq, hq, d) if seq_major_out else (b, hq, sq, d),
                      dtype=torch.bfloat16 if is_bf16 else torch.float16, device=q_packed.device)
    lib = _lib.load()
    with torch.cuda.device(out.device):
        nbytes = lib.ta100_prefill_workspace_bytes(b, hq, hkv, sq, skv, d, int(is_mx))
        ws = _workspace(out.device, nbytes)
        sel = selected_blocks if width > 0 else None
        events = None
        if _prefill_event_sink is not None:
            events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            events[0].record()
        rc = lib.ta100_prefill_attention(
            _ptr(q_hi) if sel is not None else None, _ptr(k_hi) if sel is not None else None,
            _ptr(v_hi) if sel is not None else None, _ptr(sel), width, block_size, _ptr(q_packed), _ptr(k_packed),
            _ptr(v_packed_t), _ptr(q_scale), _ptr(k_scale), _ptr(v_scale_t), _ptr(out), _ptr(ws), ws.numel(), b, hq, hkv,
            sq, skv, kv_cap, d, int(causal), int(is_mx), int(is_bf16), int(k_permuted), int(round_partial), max_ctas,
            int(seq_major_out), _stream(out))
        _lib.check(rc, "prefill_attention")
        if events is not None:
            events[1].record()
            _prefill_event_sink.append(events)
        if check_status:
            _lib.check(lib.ta100_prefill_status(_ptr(ws), b, hq, hkv, sq, skv, d, int(is_mx), _stream(out)),
                       "prefill_attention (device)")
    return out


def _fp4_tiled(packed, causal, is_mx, is_bf16):
    q_packed, k_packed, v_packed_t, q_scale, k_scale, v_scale_t = packed
    return prefill_attention(None, None, None, None, q_packed, k_packed, v_packed_t, q_scale, k_scale, v_scale_t,
                             causal=causal, is_mx=is_mx, is_bf16=is_bf16)


def fp4_attention_causal_nvfp4_packed(q_packed, k_packed, v_packed_t, q_scale, k_scale, v_scale_t, is_bf16=False):
    return _fp4_tiled((q_packed, k_packed, v_packed_t, q_scale, k_scale, v_scale_t), True, False, is_bf16)


def fp4_attention_noncausal_nvfp4_packed(q_packed, k_packed, v_packed_t, q_scale, k_scale, v_scale_t, is_bf16=False):
    return _fp4_tiled((q_packed, k_packed, v_packed_t, q_scale, k_scale, v_scale_t), False, False, is_bf16)


def fp4_attention_causal_mxfp4_packed(q_packed, k_packed, v_packed_t, q_scale, k_scale, v_scale_t, is_bf16=False):
    return _fp4_tiled((q_packed, k_packed, v_packed_t, q_scale, k_scale, v_scale_t), True, True, is_bf16)


def fp4_attention_noncausal_mxfp4_packed(q_packed, k_packed, v_packed_t, q_scale, k_scale, v_scale_t, is_bf16=False):
    return _fp4_tiled((q_packed, k_packed, v_packed_t, q_scale, k_scale, v_scale_t), False, True, is_bf16)


def _thrift_tiled(args, causal, is_mx, is_bf16):
    q_hi, k_hi, v_hi, selected_blocks = args[:4]
    return prefill_attention(q_hi, k_hi, v_hi, selected_blocks, *args[4:], causal=causal, is_mx=is_mx, is_bf16=is_bf16)


def thrift_attention_causal_nvfp4_packed(q_hi, k_hi, v_hi, selected_blocks, q_packed, k_packed, v_packed_t, q_scale,
                                         k_scale, v_scale_t, is_bf16=False):
    return _thrift_tiled((q_hi, k_hi, v_hi, selected_blocks, q_packed, k_packed, v_packed_t, q_scale, k_scale,
                          v_scale_t), True, False, is_bf16)


def thrift_attention_noncausal_nvfp4_packed(q_hi, k_hi, v_hi, selected_blocks, q_packed, k_packed, v_packed_t, q_scale,
                                            k_scale, v_scale_t, is_bf16=False):
    return _thrift_tiled((q_hi, k_hi, v_hi, selected_blocks, q_packed, k_packed, v_packed_t, q_scale, k_scale,
                          v_scale_t), False, False, is_bf16)


def thrift_attention_causal_mxfp4_packed(q_hi, k_hi, v_hi, selected_blocks, q_packed, k_packed, v_packed_t, q_scale,
                                         k_scale, v_scale_t, is_bf16=False):
    return _thrift_tiled((q_hi, k_hi, v_hi, selected_blocks, q_packed, k_packed, v_packed_t, q_scale, k_scale,
                          v_scale_t), True, True, is_bf16)


def thrift_attention_noncausal_mxfp4_packed(q_hi, k_hi, v_hi, selected_blocks, q_packed, k_packed, v_packed_t, q_scale,
                                            k_scale, v_scale_t, is_bf16=False):
    return _thrift_tiled((q_hi, k_hi, v_hi, selected_blocks, q_packed, k_packed, v_packed_t, q_scale, k_scale,
                          v_scale_t), False, True, is_bf16)


# ---------------------------------------------------------------------------------------------
# Decode (single query) attention  (bindings.cpp:420-486, 731-891)
# ---------------------------------------------------------------------------------------------
def _check_decode_args(q_hi, k_hi, v_hi, selected_blocks, q_packed, k_packed, v_packed_t, q_scale, k_scale, v_scale_t,
                       kv_len, page_table, allow_padded_selection):
    """Argument checks shared by every decode entry (the conditions of bindings.cpp:731-810 plus the paged
    extension).  Returns (b, hkv, g, d, skv, kv_cap, max_pages, npages, width)."""
    _check(q_packed.is_cuda and k_packed.is_cuda and v_packed_t.is_cuda, "packed Q/K/V must be CUDA tensors")
    _check(q_scale.is_cuda and k_scale.is_cuda and v_scale_t.is_cuda, "Q/K/V scales must be CUDA tensors")
    _check(q_packed.dim() == 4, "packed Q must be 4D [batch, kv_heads, groups, head_dim / 2]")
    b, hkv, g, dh = q_packed.shape
    d = dh * 2
    _check(1 <= g <= 16, f"single-query ThriftAttention expects grouped query length in [1, 16], got {g}")
    _check(q_packed.is_contiguous() and q_scale.is_contiguous(), "packed Q and its scales must be contiguous")
    if page_table is None:
        _check(k_packed.dim() == 4 and k_packed.size(0) == b and k_packed.size(1) == hkv, "packed K shape mismatch")
        skv = k_packed.size(2) if kv_len is None else kv_len
        _check(k_packed.stride(3) == 1 and k_packed.stride(2) == dh, "packed K rows must be dense")
        kv_cap = max(skv, k_packed.stride(1) // dh)
        _check((kv_cap + 127) // 128 * 128 // 2 == v_packed_t.stride(2) or v_packed_t.size(3) * 1 == v_packed_t.stride(2),
               "packed V row stride must equal the padded cache capacity / 2")
        max_pages = 0
    else:
        _check(kv_len is not None, "kv_len is required with a page table")
        _check(page_table.is_cuda and page_table.dtype == torch.int32 and page_table.is_contiguous()
               and page_table.dim() == 2 and page_table.size(0) == b, "page_table must be int32 [batch, max_pages]")
        skv, kv_cap, max_pages = kv_len, kv_len, page_table.size(1)
        pool = k_packed.size(0)
        _check(k_packed.dim() == 4 and k_packed.size(1) == hkv and k_packed.size(2) == 64 and k_packed.is_contiguous(),
               "paged K codes must be a contiguous pool [pages, kv_heads, 64, head_dim / 2]")
        _check(v_packed_t.dim() == 4 and v_packed_t.size(0) == pool and v_packed_t.is_contiguous()
               and k_scale.size(0) == pool and v_scale_t.size(0) == pool and k_scale.is_contiguous()
               and v_scale_t.is_contiguous(), "the K/V code and scale pools must be contiguous and hold the same number of pages")
        _check(kv_len // 64 <= max_pages, "page_table has fewer columns than the sequence has pages")
    _check(skv % 64 == 0, "k sequence length must be divisible by 64")
    npages = skv // 64
    width = 0
    if selected_blocks is not None:
        _check(selected_blocks.is_cuda, "selected_blocks must be a CUDA tensor")
        _check(selected_blocks.dtype == torch.int32, "selected_blocks must be int32")
        _check(selected_blocks.is_contiguous(), "selected_blocks must be contiguous")
        _check(selected_blocks.dim() == 2, "selected_blocks must be [batch * grouped_heads, top_k]")
        _check(selected_blocks.size(0) == b * hkv, "selected_blocks first dimension must equal batch * grouped_heads")
        width = selected_blocks.size(1)
        # a shard of a longer sequence may receive a list wider than its own page count (entries of other
        # shards are -1)
        _check(allow_padded_selection or 0 <= width <= npages,
               "selected block count must be in [0, number of KV blocks]")
        if width:
            _check(q_hi is not None and q_hi.shape == (b, hkv, g, d), "q_hi shape must match packed Q")
            _check(q_hi.is_contiguous(), "Q must be contiguous")
            if page_table is None:
                # 16-bit K/V may be views of a longer cache, as long as they share the packed K's capacity
                want = (hkv * kv_cap * d, kv_cap * d, d, 1)
                for t in (k_hi, v_hi):
                    _check(t.dim() == 4 and (t.is_contiguous() and t.size(2) == kv_cap or tuple(t.stride()) == want),
                           "16-bit K/V must be contiguous or views of a cache with the packed K's capacity")
            else:
                _check(k_hi.is_contiguous() and v_hi.is_contiguous() and k_hi.size(0) == k_packed.size(0)
                       and v_hi.size(0) == k_packed.size(0),
                       "the 16-bit K/V pools must be contiguous and hold as many pages as the code pools")
    return b, hkv, g, d, skv, kv_cap, max_pages, npages, width


def decode_pick_splits(flat_kv_heads: int, num_pages: int) -> int:
    """Number of sequential KV chains per (sequence, KV head) the decode kernel uses by default."""
    return _lib.load().ta100_decode_pick_splits(flat_kv_heads, num_pages)


def decode_attention(q_hi, k_hi, v_hi, selected_blocks, q_packed, k_packed, v_packed_t, q_scale, k_scale, v_scale_t, *,
                     is_mx, is_bf16=False, num_splits=0, kv_len=None, page_table=None, return_partials=False,
                     allow_padded_selection=False, partials_out=None, check_status=False):
    """Split-KV decode attention over 64-token pages.

    q_* are grouped: [B, Hkv, G, ...] with G <= 16 query heads per KV head.  K/V are either the
    reference's contiguous, capacity-strided cache tensors (``page_table is None``) or page pools
    ``[n_pages, Hkv, 64, ...]`` (K rows, 16-bit K/V) and ``[n_pages, Hkv, D, 32]`` (V codes) addressed
    through ``page_table`` int32 [B, max_pages].  ``selected_blocks`` is ``None`` or int32 [B*Hkv, W].
    Returns [B, Hkv, G, D]; with ``return_partials`` also the un-merged ``(o, ml)`` partials
    ([B*Hkv, splits, G, D] in units of C and [B*Hkv, splits, G, 2] = (row max, row sum)).
    ``check_status`` synchronises and raises if the kernel skipped a page-table entry outside the pool or gave up
    a bounded wait (``decode_status``).
    """
    b, hkv, g, d, skv, kv_cap, max_pages, npages, width = _check_decode_args(
        q_hi, k_hi, v_hi, selected_blocks, q_packed, k_packed, v_packed_t, q_scale, k_scale, v_scale_t, kv_len, page_table,
        allow_padded_selection)
    pool_pages = k_packed.size(0) if page_table is not None else 0
    lib = _lib.load()
    dev = q_packed.device
    splits = num_splits if num_splits > 0 else lib.ta100_decode_pick_splits(b * hkv, npages)
    splits = max(1, min(splits, npages))
    out = torch.empty(b, hkv, g, d, dtype=torch.bfloat16 if is_bf16 else torch.float16, device=dev)
    if partials_out is not None:
        # caller-owned partials (e.g. two views of the buffer a rank all-gathers afterwards)
        part_o, part_ml = partials_out
        _check(tuple(part_o.shape) == (b * hkv, splits, g, d) and tuple(part_ml.shape) == (b * hkv, splits, g, 2)
               and part_o.dtype == part_ml.dtype == torch.float32 and part_o.is_contiguous() and part_ml.is_contiguous()
               and part_o.device == dev and part_ml.device == dev,
               f"partials_out must be contiguous fp32 [{b * hkv}, {splits}, {g}, {d}] and [.., 2] on the query's device")
    else:
        part_o = torch.empty(b * hkv, splits, g, d, dtype=torch.float32, device=dev)
        part_ml = torch.empty(b * hkv, splits, g, 2, dtype=torch.float32, device=dev)
    sel = selected_blocks if width else None
    with torch.cuda.device(dev):
        rc = lib.ta100_decode_attention(
            _ptr(q_hi) if sel is not None else None, _ptr(k_hi) if sel is not None else None,
            _ptr(v_hi) if sel is not None else None, _ptr(sel), width, _ptr(q_packed), _ptr(k_packed), _ptr(v_packed_t),
            _ptr(q_scale), _ptr(k_scale), _ptr(v_scale_t), _ptr(page_table), max_pages, pool_pages, _ptr(out), _ptr(part_o),
            _ptr(part_ml), b, hkv, g, skv, kv_cap, d, int(is_mx), int(is_bf16), splits, 1, _stream(out))
    _lib.check(rc, "decode_attention")
    if check_status:
        decode_status(dev)
    if return_partials:
        return out, part_o, part_ml
    return out


_decode_step_scratch: dict = {}
_decode_step_splits: dict = {}


def cached_decode_step(q_grouped, k_hi, v_hi, k_packed, k_scale, v_packed_t, v_scale_t, stat_a, stat_b, *, kv_len, n_select_blocks,
                       top_k, sink=0, local=0, is_mx=False, sel_out=None, page_table=None):
    """One decode step over a contiguous cache in ONE library call (quantise q, select, attend, merge).  With
    ``page_table`` (int32 [B, max_pages]) the cache tensors are the page pools of ``decode_attention``.

    ``q_grouped`` [B, Hkv, G, D]; the cache tensors are the capacity-sized buffers themselves (not views):
    ``k_hi`` / ``v_hi`` [B, Hkv, cap, D], ``k_packed`` [B, Hkv, cap, D/2], ``v_packed_t`` [B, Hkv, D, cap/2] and their
    scales, ``stat_a`` / ``stat_b`` [B, Hkv, cap/64, D] block means or (Quest) minima / maxima.  ``kv_len`` is the
    kernel length (a multiple of 64).  The caller owns the shapes: this entry validates only what the library
    cannot (it is the hot path of a batch-1 generation loop, where the host time per call exceeds the device
    time).  Returns ``(out [B, Hkv, G, D], selected [B*Hkv, top_k + sink + local])``."""
    b, hkv, g, d = q_grouped.shape
    dev = q_grouped.device
    is_bf16 = q_grouped.dtype == torch.bfloat16
    _check(q_grouped.is_cuda and q_grouped.is_contiguous() and kv_len % 64 == 0 and 1 <= g <= 16,
           "cached_decode_step expects a contiguous CUDA query [B, Hkv, G <= 16, D] and a kernel length in whole pages")
    cap = k_packed.shape[2]
    width = top_k + sink + local
    lib = _lib.load()
    key = (b * hkv, kv_len // 64)
    splits = _decode_step_splits.get(key)
    if splits is None:
        splits = max(1, min(lib.ta100_decode_pick_splits(b * hkv, kv_len // 64), kv_len // 64))
        _decode_step_splits[key] = splits
    skey = (dev.index, b, hkv, g, d, splits, is_mx)
    scratch = _decode_step_scratch.get(skey)
    if scratch is None:
        grp = 32 if is_mx else 16
        scratch = (torch.empty(b, hkv, g, d // 2, dtype=torch.uint8, device=dev),
                   torch.empty(b, hkv, g, d // grp, dtype=torch.uint8, device=dev),
                   torch.empty(b * hkv, splits, g, d, dtype=torch.float32, device=dev),
                   torch.empty(b * hkv, splits, g, 2, dtype=torch.float32, device=dev))
        _decode_step_scratch[skey] = scratch
    q4, qs, part_o, part_ml = scratch
    if sel_out is None or tuple(sel_out.shape) != (b * hkv, width):
        sel_out = torch.empty(b * hkv, width, dtype=torch.int32, device=dev)
    out = torch.empty(b, hkv, g, d, dtype=q_grouped.dtype, device=dev)
    vp = ctypes.c_void_p
    if page_table is not None:
        with torch.cuda.device(dev):
            rc = lib.ta100_cached_decode_step_paged(
                vp(q_grouped.data_ptr()), vp(q4.data_ptr()), vp(qs.data_ptr()), vp(k_hi.data_ptr()), vp(v_hi.data_ptr()),
                vp(k_packed.data_ptr()), vp(k_scale.data_ptr()), vp(v_packed_t.data_ptr()), vp(v_scale_t.data_ptr()),
                vp(page_table.data_ptr()), page_table.shape[1], k_packed.shape[0],
                vp(stat_a.data_ptr()) if width else None, vp(stat_b.data_ptr()) if (width and stat_b is not None) else None,
                vp(sel_out.data_ptr()), vp(out.data_ptr()), vp(part_o.data_ptr()), vp(part_ml.data_ptr()), b, hkv, g, kv_len,
                stat_a.shape[2] if stat_a is not None else 0, n_select_blocks, top_k, sink, local, d, int(is_mx),
                int(is_bf16), splits, vp(torch.cuda.current_stream(dev).cuda_stream))
        if rc:
            _lib.check(rc, "cached_decode_step")
        return out, sel_out
    with torch.cuda.device(dev):
        rc = lib.ta100_cached_decode_step(
            vp(q_grouped.data_ptr()), vp(q4.data_ptr()), vp(qs.data_ptr()), vp(k_hi.data_ptr()), vp(v_hi.data_ptr()),
            vp(k_packed.data_ptr()), vp(k_scale.data_ptr()), vp(v_packed_t.data_ptr()), vp(v_scale_t.data_ptr()),
            vp(stat_a.data_ptr()) if width else None, vp(stat_b.data_ptr()) if (width and stat_b is not None) else None,
            vp(sel_out.data_ptr()), vp(out.data_ptr()), vp(part_o.data_ptr()), vp(part_ml.data_ptr()), b, hkv, g, kv_len,
            cap, stat_a.shape[2] if stat_a is not None else 0, n_select_blocks, top_k, sink, local, d, int(is_mx),
            int(is_bf16), splits, vp(torch.cuda.current_stream(dev).cuda_stream))
    if rc:
        _lib.check(rc, "cached_decode_step")
    return out, sel_out


def _check_length(length: torch.Tensor, device, batch: int | None = None) -> int:
    """The device-side length: int32 on the cache's device, one element (every sequence has that length) or one per
    sequence (a ragged batch).  Returns the element count."""
    _check(isinstance(length, torch.Tensor) and length.is_cuda and length.device == device and length.dtype == torch.int32
           and length.is_contiguous() and (length.numel() == 1 or batch is None or length.numel() == batch),
           "the device-side length must be a contiguous int32 CUDA tensor on the cache's device with one element, or one per sequence")
    return int(length.numel())


def cache_append_at(k_new, v_new, k_hi, v_hi, k_codes, k_scales, v_codes, v_scales, length, *, offset=0, page_table=None,
                    k_mean=None, k_min=None, k_max=None, is_mx=False, stat_block=64):
    """``cache_append`` (or, with ``page_table``, ``cache_append_paged``) at token position ``length[0] + offset``, where
    ``length`` is an int32 tensor ON THE GPU (one element, or one per sequence for a ragged batch): the launch is the
    same whatever the position, so it can be captured in a CUDA graph and replayed for every token.  A range that would end beyond the capacity is not stored.
    ``k_new`` / ``v_new`` [B, Hkv, T, D]."""
    _check(k_hi.is_cuda and k_hi.dim() == 4 and k_hi.is_contiguous() and k_hi.dtype in (torch.float16, torch.bfloat16),
           "k cache must be a contiguous 4D float16 / bfloat16 CUDA tensor")
    paged = page_table is not None
    g = 32 if is_mx else 16
    d = k_hi.shape[3]
    if paged:
        pool, hkv = k_hi.shape[0], k_hi.shape[1]
        _check(k_hi.shape[2] == 64 and page_table.is_cuda and page_table.dtype == torch.int32 and page_table.dim() == 2
               and page_table.is_contiguous(), "paged append expects pools [pool, Hkv, 64, D] and an int32 page table")
        b, max_pages = page_table.shape
        cap = 0
        expect = {"v_hi": (v_hi, (pool, hkv, 64, d)), "k_codes": (k_codes, (pool, hkv, 64, d // 2)),
                  "k_scales": (k_scales, (pool, hkv, 64, d // g)), "v_codes": (v_codes, (pool, hkv, d, 32)),
                  "v_scales": (v_scales, (pool, hkv, d, 64 // g))}
    else:
        b, hkv, cap, _ = k_hi.shape
        pool = max_pages = 0
        expect = {"v_hi": (v_hi, (b, hkv, cap, d)), "k_codes": (k_codes, (b, hkv, cap, d // 2)),
                  "k_scales": (k_scales, (b, hkv, cap, d // g)), "v_codes": (v_codes, (b, hkv, d, cap // 2)),
                  "v_scales": (v_scales, (b, hkv, d, cap // g))}
    for name, (t, shape) in expect.items():
        _check(t.is_cuda and t.is_contiguous() and tuple(t.shape) == shape, f"{name} must be contiguous {shape}")
    for name, new in (("key_states", k_new), ("value_states", v_new)):
        _check(new is not None and new.is_cuda and new.is_contiguous() and new.dtype == k_hi.dtype and new.dim() == 4
               and new.shape[0] == b and new.shape[1] == hkv and new.shape[3] == d,
               f"{name} must be contiguous [batch, kv_heads, tokens, head_dim] CUDA tensors of the cache dtype")
    n_len = _check_length(length, k_hi.device, b)
    stat_blocks = 1
    for name, t in (("k_mean", k_mean), ("k_min", k_min), ("k_max", k_max)):
        if t is not None:
            _check(t.is_cuda and t.is_contiguous() and t.dim() == 4 and t.shape[0] == b and t.shape[1] == hkv
                   and t.shape[3] == d and t.dtype == k_hi.dtype and (paged or t.shape[2] == cap // stat_block),
                   f"{name} must be contiguous [B, Hkv, blocks, D] of the cache dtype")
            stat_blocks = t.shape[2]
    with torch.cuda.device(k_hi.device):
        rc = _lib.load().ta100_cache_append_at(
            _ptr(k_new), _ptr(v_new), _ptr(k_hi), _ptr(v_hi), _ptr(k_codes), _ptr(k_scales), _ptr(v_codes), _ptr(v_scales),
            _ptr(k_mean), _ptr(k_min), _ptr(k_max), _ptr(page_table), max_pages, pool, b, hkv, stat_blocks, cap, _ptr(length),
            n_len, int(offset), k_new.shape[2], v_new.shape[2], d, stat_block, int(is_mx), int(k_hi.dtype == torch.bfloat16), 0,
            _stream(k_hi))
    _lib.check(rc, "cache_append_at")


def advance_length(length: torch.Tensor, count: int, limit: int) -> None:
    """``length[i] = min(length[i] + count, limit)`` for every element, in stream order (one tiny launch): the end of a
    generation step whose kernels read the length on the GPU."""
    n_len = _check_length(length, length.device)
    with torch.cuda.device(length.device):
        rc = _lib.load().ta100_advance_length(_ptr(length), n_len, int(count), int(limit), _stream(length))
    _lib.check(rc, "advance_length")


def decode_step_row_width(max_len: int, *, top_k=None, fraction=None, sink=0, local=0) -> int:
    """Width of the selection rows ``cached_decode_step_at`` needs for sequences of up to ``max_len`` tokens."""
    from .selection.counts import resolve_top_k

    n = max_len // 64
    return max(1, resolve_top_k(n, causal=False, top_k=top_k, fraction=fraction) + int(sink) + int(local))


def cached_decode_step_at(q_grouped, k_hi, v_hi, k_packed, k_scale, v_packed, v_scale, stat_a, stat_b, length, *, offset,
                          max_len, top_k=None, fraction=None, sink=0, local=0, is_mx=False, splits=None, sel_out=None,
                          out=None, page_table=None):
    """``cached_decode_step`` over ``length[0] + offset`` cached tokens, ``length`` being an int32 tensor ON THE GPU
    with one element - or one per sequence: sequence ``i`` of a ragged batch then holds ``length[i] + offset`` tokens.  The kernels derive the page count, the number of complete blocks and the selected / forced block counts
    (the rule of ``cached_decode_attention``: ``top_k`` blocks or ``fraction`` of the complete ones, ``local`` then
    ``sink`` forced blocks as far as there is room) from it when they start, so the same launches serve every length
    up to ``max_len`` (a multiple of 64) and replay from one CUDA graph across tokens.  Contiguous cache tensors as
    for ``cached_decode_step``; with ``page_table`` the page pools.  ``splits`` chains per KV head (default: the
    choice for ``max_len``).  Returns ``(out [B, Hkv, G, D], selected [B*Hkv, row width])``, rows -1 padded."""
    b, hkv, g, d = q_grouped.shape
    dev = q_grouped.device
    is_bf16 = q_grouped.dtype == torch.bfloat16
    _check(q_grouped.is_cuda and q_grouped.is_contiguous() and max_len % 64 == 0 and max_len > 0 and 1 <= g <= 16,
           "cached_decode_step_at expects a contiguous CUDA query [B, Hkv, G <= 16, D] and max_len in whole pages")
    n_len = _check_length(length, dev, b)
    _check(stat_a is not None and k_hi is not None and v_hi is not None, "the statistics and the 16-bit caches are required")
    paged = page_table is not None
    cap = max_len if paged else k_packed.shape[2]
    _check(cap >= max_len, "max_len exceeds the cache capacity")
    width = decode_step_row_width(max_len, top_k=top_k, fraction=fraction, sink=sink, local=local)
    lib = _lib.load()
    pages = max_len // 64
    if splits is None:
        splits = max(1, min(lib.ta100_decode_pick_splits(b * hkv, pages), pages))
    skey = (dev.index, b, hkv, g, d, splits, is_mx)
    scratch = _decode_step_scratch.get(skey)
    if scratch is None:
        grp = 32 if is_mx else 16
        scratch = (torch.empty(b, hkv, g, d // 2, dtype=torch.uint8, device=dev),
                   torch.empty(b, hkv, g, d // grp, dtype=torch.uint8, device=dev),
                   torch.empty(b * hkv, splits, g, d, dtype=torch.float32, device=dev),
                   torch.empty(b * hkv, splits, g, 2, dtype=torch.float32, device=dev))
        _decode_step_scratch[skey] = scratch
    q4, qs, part_o, part_ml = scratch
    if sel_out is None or tuple(sel_out.shape) != (b * hkv, width):
        sel_out = torch.empty(b * hkv, width, dtype=torch.int32, device=dev)
    if out is None:
        out = torch.empty(b, hkv, g, d, dtype=q_grouped.dtype, device=dev)
    vp = ctypes.c_void_p
    with torch.cuda.device(dev):
        rc = lib.ta100_cached_decode_step_at(
            vp(q_grouped.data_ptr()), vp(q4.data_ptr()), vp(qs.data_ptr()), vp(k_hi.data_ptr()), vp(v_hi.data_ptr()),
            vp(k_packed.data_ptr()), vp(k_scale.data_ptr()), vp(v_packed.data_ptr()), vp(v_scale.data_ptr()),
            _ptr(page_table), page_table.shape[1] if paged else 0, k_packed.shape[0] if paged else 0,
            vp(stat_a.data_ptr()), _ptr(stat_b), vp(sel_out.data_ptr()), width, vp(out.data_ptr()), vp(part_o.data_ptr()),
            vp(part_ml.data_ptr()), b, hkv, g, vp(length.data_ptr()), n_len, int(offset), max_len, cap, stat_a.shape[2],
            -1 if top_k is None else int(top_k), float(0.05 if fraction is None else fraction), int(sink), int(local), d,
            int(is_mx), int(is_bf16), splits, vp(torch.cuda.current_stream(dev).cuda_stream))
    if rc:
        _lib.check(rc, "cached_decode_step_at")
    return out, sel_out


def debug_set_wait(budget_cycles: int = 0, skip_loads: bool = False) -> None:
    """Diagnostics: the cycle budget of the bounded device-side waits of later launches (0 = default) and a switch
    that makes the attention kernels' producer warps copy nothing, so that the waits run out (tests of the
    give-up path).  Process-wide."""
    _lib.check(_lib.load().ta100_debug_set_wait(int(budget_cycles), int(bool(skip_loads))), "debug_set_wait")


def decode_status(device=None) -> None:
    """Raises ``RuntimeError`` if a bounded wait inside a decode kernel ran out on ``device`` since the
    last call (synchronises with the current stream)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        rc = _lib.load().ta100_decode_status(ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    _lib.check(rc, "decode_attention (device)")


def reduce_decode_partials(part_o: torch.Tensor, part_ml: torch.Tensor, out=None):
    """One producer's chains reduced to a single partial per head: ``[heads, splits, G, D]`` / ``[.., 2]`` ->
    ``[heads, 1, G, D]`` / ``[heads, 1, G, 2]`` (fp32; same meaning as the inputs).  ``out`` = the two result
    tensors, e.g. two views of the buffer that is all-gathered next."""
    _check(part_o.is_cuda and part_ml.is_cuda and part_o.is_contiguous() and part_ml.is_contiguous()
           and part_o.dim() == 4 and part_ml.dim() == 4, "partials must be contiguous 4-D CUDA tensors")
    _check(part_o.dtype == torch.float32 and part_ml.dtype == torch.float32, "partials must be float32")
    heads, splits, g, d = part_o.shape
    if out is None:
        out = (torch.empty(heads, 1, g, d, dtype=torch.float32, device=part_o.device),
               torch.empty(heads, 1, g, 2, dtype=torch.float32, device=part_o.device))
    out_o, out_ml = out
    _check(tuple(out_o.shape) == (heads, 1, g, d) and tuple(out_ml.shape) == (heads, 1, g, 2) and out_o.is_contiguous()
           and out_ml.is_contiguous() and out_o.dtype == out_ml.dtype == torch.float32,
           "out must be contiguous fp32 [heads, 1, G, D] and [heads, 1, G, 2]")
    with torch.cuda.device(part_o.device):
        rc = _lib.load().ta100_reduce_partials(_ptr(part_o), _ptr(part_ml), _ptr(out_o), _ptr(out_ml), heads, splits, g, d,
                                               _stream(part_o))
    _lib.check(rc, "reduce_partials")
    return out_o, out_ml


def merge_decode_partials(part_o: torch.Tensor, part_ml: torch.Tensor, *, is_mx: bool, is_bf16: bool = False):
    """LSE merge of decode partials gathered from several shards.

    part_o [shards, heads, splits, G, D] fp32 (units of C), part_ml [shards, heads, splits, G, 2]
    -> [heads, G, D] 16-bit.  Same formula as the in-kernel merge of the reference
    (csrc/cuda/sm120/nvfp4/single_query_attention.cu:1562-1593).
    """
    _check(part_o.is_cuda and part_ml.is_cuda and part_o.dim() == 5 and part_ml.dim() == 5,
           "partials must be 5-D CUDA tensors")
    # each shard's block must be dense; the shards themselves may be any distance apart (two views of one
    # all-gathered buffer per shard)
    _check(part_o[0].is_contiguous() and part_ml[0].is_contiguous(), "each shard's partials must be contiguous")
    _check(part_o.dtype == torch.float32 and part_ml.dtype == torch.float32, "partials must be float32")
    shards, heads, splits, g, d = part_o.shape
    out = torch.empty(heads, g, d, dtype=torch.bfloat16 if is_bf16 else torch.float16, device=part_o.device)
    so = part_o.stride(0) if shards > 1 else 0
    sml = part_ml.stride(0) if shards > 1 else 0
    with torch.cuda.device(out.device):
        rc = _lib.load().ta100_merge_partials(_ptr(part_o), _ptr(part_ml), _ptr(out), shards, so, sml, heads, splits, g,
                                              d, int(is_mx), int(is_bf16), _stream(out))
    _lib.check(rc, "merge_partials")
    return out


def _fp4_single(packed, is_mx, is_bf16):
    q_packed, k_packed, v_packed_t, q_scale, k_scale, v_scale_t = packed
    _check_packed(q_packed, k_packed, v_packed_t, q_scale, k_scale, v_scale_t)
    return decode_attention(None, None, None, None, q_packed, k_packed, v_packed_t, q_scale, k_scale, v_scale_t,
                            is_mx=is_mx, is_bf16=is_bf16)


def fp4_attention_single_query_nvfp4_packed(q_packed, k_packed, v_packed_t, q_scale, k_scale, v_scale_t, is_bf16=False):
    return _fp4_single((q_packed, k_packed, v_packed_t, q_scale, k_scale, v_scale_t), False, is_bf16)


def fp4_attention_single_query_mxfp4_packed(q_packed, k_packed, v_packed_t, q_scale, k_scale, v_scale_t, is_bf16=False):
    return _fp4_single((q_packed, k_packed, v_packed_t, q_scale, k_scale, v_scale_t), True, is_bf16)


def _thrift_single(q_hi, k_hi, v_hi, selected_blocks, packed, is_mx, is_bf16):
    _check_hi(q_hi, k_hi, v_hi)
    _check_packed(*packed)
    return decode_attention(q_hi, k_hi, v_hi, selected_blocks, *packed, is_mx=is_mx, is_bf16=is_bf16)


def thrift_attention_single_query_nvfp4_packed(q_hi, k_hi, v_hi, selected_blocks, q_packed, k_packed, v_packed_t, q_scale,
                                               k_scale, v_scale_t, is_bf16=False):
    return _thrift_single(q_hi, k_hi, v_hi, selected_blocks, (q_packed, k_packed, v_packed_t, q_scale, k_scale,
                                                              v_scale_t), False, is_bf16)


def thrift_attention_single_query_mxfp4_packed(q_hi, k_hi, v_hi, selected_blocks, q_packed, k_packed, v_packed_t, q_scale,
                                               k_scale, v_scale_t, is_bf16=False):
    return _thrift_single(q_hi, k_hi, v_hi, selected_blocks, (q_packed, k_packed, v_packed_t, q_scale, k_scale,
                                                              v_scale_t), True, is_bf16)


def decode_attention_noalloc(q_hi, k_hi, v_hi, selected_blocks, q_packed, k_packed, v_packed_t, q_scale, k_scale,
                             v_scale_t, out, *, is_mx, is_bf16=False, num_splits=0):
    """Decode attention that allocates nothing: the caller passes ``out`` ([B, Hkv, G, D], 16-bit) and
    the split-KV partials live in a fixed 16 MiB array inside the CUDA library.

    For processes that cannot allocate device memory at call time — all free HBM already belongs to
    their own pool, or a ``cudaMalloc`` stall is not acceptable inside the decode loop.  Same result
    as ``decode_attention`` with the same ``num_splits``.  Calls on one device share the scratch, so
    do not let two of them overlap on the GPU; make the first call on a device outside stream
    capture.  Raises ``RuntimeError`` when the problem needs more scratch than the fixed array holds.
    Contiguous (non-paged) caches only in this wrapper.
    """
    b, hkv, g, d, skv, kv_cap, _, _, width = _check_decode_args(
        q_hi, k_hi, v_hi, selected_blocks, q_packed, k_packed, v_packed_t, q_scale, k_scale, v_scale_t, None, None, False)
    _check(out.is_cuda and out.is_contiguous() and tuple(out.shape) == (b, hkv, g, d), "out must be contiguous [B, Hkv, G, D]")
    _check(out.dtype == (torch.bfloat16 if is_bf16 else torch.float16), "out dtype must match is_bf16")
    _check(out.device == q_packed.device, "out must live on the query's device")
    lib = _lib.load()
    splits = num_splits if num_splits > 0 else lib.ta100_decode_pick_splits(b * hkv, skv // 64)
    splits = max(1, min(splits, skv // 64))
    sel = selected_blocks if width else None
    with torch.cuda.device(out.device):
        rc = lib.ta100_decode_attention_static(
            _ptr(q_hi) if sel is not None else None, _ptr(k_hi) if sel is not None else None,
            _ptr(v_hi) if sel is not None else None, _ptr(sel), width, _ptr(q_packed), _ptr(k_packed), _ptr(v_packed_t),
            _ptr(q_scale), _ptr(k_scale), _ptr(v_scale_t), None, 0, 0, _ptr(out), b, hkv, g, skv, kv_cap, d, int(is_mx),
            int(is_bf16), splits, _stream(out))
    _lib.check(rc, "decode_attention_noalloc")
    return out

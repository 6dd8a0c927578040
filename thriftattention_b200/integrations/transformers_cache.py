"""Generation cache for Hugging Face Transformers models: 16-bit K/V plus the FP4 codes, block
scales and per-block key statistics that the decode kernel reads, kept current by ONE fused
kernel launch per layer and step.

Interface and semantics follow the reference's ``integrations/transformers_cache.py``
(``ThriftAttentionCacheLayer`` :70-475, ``ThriftAttentionCache`` :478-567, ``cached_decode_attention``
:570-619, ``cached_prefill_attention`` :622-680, the selection helpers :683-831):

* physical capacity is a multiple of 128 tokens, grown by doubling or fixed by ``max_cache_len``;
* ``seq_len`` is the logical length; the packed views handed to the kernels are rounded up to 64
  tokens (V to 128) and the rounded tail holds zero rows;
* only complete 64-token blocks can be promoted to 16-bit — the trailing partial block stays FP4;
* ``crop`` zeroes and re-quantises the rounded tail.

Beyond the reference: MXFP4 caches, Quest selection (block minima / maxima are maintained next to
the means), forced sink / local blocks, and a prefill that reads the cache's own FP4 tensors
instead of quantising K and V a second time.
"""
from __future__ import annotations

from contextlib import contextmanager
from contextvars import ContextVar
from dataclasses import dataclass
from typing import Any, Iterator

import weakref

import torch

from .._extension import get_extension
from ..backends.single_query import _group_single_query, _ungroup_single_query
from ..config import AttentionConfig
from ..quant.formats import get_quant_format
from ..selection import resolve_top_k
from ..selection.local import select_local_block_pairs

PAGE = 64            # tokens per selectable KV block of the decode kernel
CAPACITY_QUANTUM = 128

_ACTIVE_CACHE: ContextVar["ThriftAttentionCache | None"] = ContextVar("thriftattention_active_cache", default=None)


def get_active_thriftattention_cache() -> "ThriftAttentionCache | None":
    return _ACTIVE_CACHE.get()


@contextmanager
def use_thriftattention_cache(cache: "ThriftAttentionCache") -> Iterator["ThriftAttentionCache"]:
    """Make ``cache`` the one the registered attention function routes through (context-local)."""
    token = _ACTIVE_CACHE.set(cache)
    try:
        yield cache
    finally:
        _ACTIVE_CACHE.reset(token)


def is_thriftattention_cache(value: object) -> bool:
    return isinstance(value, ThriftAttentionCache)


def _round_up(value: int, multiple: int) -> int:
    return -(-value // multiple) * multiple


def _cache_position_start(cache_kwargs: dict[str, Any] | None, fallback: int) -> int:
    """First position of an update: ``cache_kwargs['cache_position']`` (must be consecutive) or ``fallback``."""
    position = (cache_kwargs or {}).get("cache_position")
    if position is None:
        return fallback
    if not isinstance(position, torch.Tensor):
        return int(position)
    flat = position.reshape(-1)
    if flat.numel() == 0:
        return fallback
    # Reading a device tensor synchronises with the GPU.  A model passes the SAME tensor object to every layer
    # of a forward pass, so the value read for the first layer serves the others (checked by object identity
    # and version counter, not by address: the allocator reuses addresses from step to step).
    memo = _POSITION_MEMO
    if memo[0] is not None and memo[0]() is position and memo[1] == position._version:
        return memo[2]
    first = int(flat[0].item())
    if flat.numel() > 1:
        expected = torch.arange(first, first + flat.numel(), device=flat.device, dtype=flat.dtype)
        if not torch.equal(flat, expected):
            raise ValueError("ThriftAttentionCache requires contiguous cache_position values")
    try:
        memo[0], memo[1], memo[2] = weakref.ref(position), position._version, first
    except TypeError:
        memo[0] = None
    return first


_POSITION_MEMO: list = [None, 0, 0]


def _scale_dtype(quant_format: str) -> torch.dtype:
    return torch.float8_e8m0fnu if quant_format == "mxfp4" else torch.float8_e4m3fn


def _group_size(quant_format: str) -> int:
    return 32 if quant_format == "mxfp4" else 16


@dataclass
class ThriftAttentionCacheLayer:
    """K/V of one attention layer: 16-bit rows, FP4 codes + scales (K by rows, V transposed) and
    per-64-token-block key statistics, all ``[batch, kv_heads, capacity, ...]``-strided."""

    max_cache_len: int | None = None
    quant_format: str = "nvfp4"
    track_minmax: bool = False

    k_fp16: torch.Tensor | None = None
    v_fp16: torch.Tensor | None = None
    k_packed: torch.Tensor | None = None
    k_scale: torch.Tensor | None = None
    v_packed_t: torch.Tensor | None = None
    v_scale_t: torch.Tensor | None = None
    k_mean: torch.Tensor | None = None
    k_min: torch.Tensor | None = None
    k_max: torch.Tensor | None = None
    selected_blocks: torch.Tensor | None = None
    seq_len: int = 0
    capacity: int = 0

    # ------------------------------------------------------------------------------------------ update
    def update(self, key_states: torch.Tensor, value_states: torch.Tensor,
               cache_kwargs: dict[str, Any] | None = None) -> tuple[torch.Tensor, torch.Tensor]:
        """Append (or overwrite from ``cache_position``) and return the logical 16-bit K/V views.

        The whole update — 16-bit stores, K quantisation, V group re-quantisation, block statistics —
        is one kernel launch (the reference issues slice copies plus three extension calls,
        transformers_cache.py:87-123)."""
        if key_states.ndim != 4 or value_states.ndim != 4:
            raise ValueError("KV cache tensors must be [batch, heads, seq, head_dim]")
        if key_states.shape != value_states.shape:
            raise ValueError("key_states and value_states must have identical shapes")
        if key_states.dtype not in (torch.float16, torch.bfloat16):
            raise ValueError("KV cache tensors must be float16 or bfloat16")
        if key_states.dtype != value_states.dtype:
            raise ValueError("key_states and value_states must have the same dtype")

        start = _cache_position_start(cache_kwargs, self.seq_len)
        token_count = key_states.shape[2]
        end = start + token_count
        if self.max_cache_len is not None and end > self.max_cache_len:
            raise ValueError(f"ThriftAttentionCache length {end} exceeds max_cache_len={self.max_cache_len}")

        self._ensure_capacity(key_states, end)
        self.seq_len = max(self.seq_len, end)
        if token_count:
            self._append(key_states.contiguous(), value_states.contiguous(), start)
        return self.key_view(), self.value_view()

    def _append(self, key_states: torch.Tensor | None, value_states: torch.Tensor | None, start: int, *,
                k_count: int | None = None, v_count: int | None = None, keep_k: bool = False, keep_v: bool = False,
                stats: bool = True) -> None:
        get_extension().cache_append(
            key_states, value_states, self.k_fp16, self.v_fp16, self.k_packed, self.k_scale, self.v_packed_t,
            self.v_scale_t, start=start, k_count=k_count, v_count=v_count,
            k_mean=self.k_mean if stats else None, k_min=self.k_min if stats else None,
            k_max=self.k_max if stats else None, is_mx=self.quant_format == "mxfp4", stat_block=PAGE,
            keep_k=keep_k, keep_v=keep_v, **({"trusted": True} if self._trusted_append(key_states, value_states) else {}))

    def _trusted_append(self, key_states, value_states) -> bool:
        """The layer allocated every cache buffer itself (``_ensure_capacity``), so only the new rows need a
        look before the unchecked entry point is used."""
        like = self.k_fp16
        if like is None or not like.is_cuda:
            return False
        for t in (key_states, value_states):
            if t is not None and not (t.is_cuda and t.is_contiguous() and t.dtype == like.dtype and t.dim() == 4
                                      and t.shape[0] == like.shape[0] and t.shape[1] == like.shape[1]
                                      and t.shape[3] == like.shape[3]):
                return False
        return True

    # ------------------------------------------------------------------------------------------- views
    def key_view(self) -> torch.Tensor:
        if self.k_fp16 is None:
            raise RuntimeError("ThriftAttention cache layer has not been initialized")
        return self.k_fp16[:, :, : self.seq_len]

    def value_view(self) -> torch.Tensor:
        if self.v_fp16 is None:
            raise RuntimeError("ThriftAttention cache layer has not been initialized")
        return self.v_fp16[:, :, : self.seq_len]

    def kernel_len(self) -> int:
        """Tokens the kernels walk: ``seq_len`` rounded up to whole 64-token blocks (at least one)."""
        return max(PAGE, _round_up(self.seq_len, PAGE))

    def packed_views(self) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
        """``(k_packed, v_packed_t, k_scale, v_scale_t)`` cut to the kernel length (V to a multiple of
        128 tokens).  The rows between ``seq_len`` and the rounded length are zero rows."""
        if self.k_packed is None or self.k_scale is None:
            raise RuntimeError("ThriftAttention packed K cache has not been initialized")
        if self.v_packed_t is None or self.v_scale_t is None:
            raise RuntimeError("ThriftAttention packed V cache has not been initialized")
        kernel_len = self.kernel_len()
        v_len = _round_up(kernel_len, CAPACITY_QUANTUM)
        g = _group_size(self.quant_format)
        return (self.k_packed[:, :, :kernel_len], self.v_packed_t[:, :, :, : v_len // 2],
                self.k_scale[:, :, :kernel_len], self.v_scale_t[:, :, :, : v_len // g])

    def hi_kernel_views(self) -> tuple[torch.Tensor, torch.Tensor]:
        """16-bit K/V cut to the kernel length (the rounded tail is zero)."""
        if self.k_fp16 is None or self.v_fp16 is None:
            raise RuntimeError("ThriftAttention cache layer has not been initialized")
        n = self.kernel_len()
        return self.k_fp16[:, :, :n], self.v_fp16[:, :, :n]

    # --------------------------------------------------------------------------------------- selection
    def select_key_blocks(self, q_grouped: torch.Tensor, *, top_k: int | None, fraction: float | None,
                          block_size: int, selection: str = "block_mean", sink_blocks: int = 0,
                          local_blocks: int = 0) -> torch.Tensor:
        """Blocks of this layer to read in 16-bit for one decode step: int32 ``[batch * kv_heads, width]``.

        Candidates are the COMPLETE blocks only (the trailing partial block stays FP4); the count comes
        from ``resolve_top_k`` with the non-causal rule (transformers_cache.py:152-212).  ``selection``
        is ``"block_mean"`` (score = q . mean(K block), the reference's policy) or ``"quest"``."""
        complete_blocks = self.seq_len // block_size
        selected_count = resolve_top_k(complete_blocks, causal=False, top_k=top_k, fraction=fraction)
        batch, kv_heads, _, _ = q_grouped.shape
        if selected_count == 0:
            return torch.empty(batch * kv_heads, 0, device=q_grouped.device, dtype=torch.int32)
        quest = selection == "quest"
        stat_a, stat_b = (self.k_min, self.k_max) if quest else (self.k_mean, None)
        if stat_a is None or (quest and stat_b is None):
            raise RuntimeError("ThriftAttention K block means have not been initialized" if not quest else
                               "ThriftAttention K block minima/maxima have not been initialized")
        if q_grouped.dtype != stat_a.dtype:
            raise ValueError("q_grouped and cached K means must have the same dtype")
        is_bf16 = q_grouped.dtype == torch.bfloat16
        # forced blocks never push the list beyond the number of candidates
        local = max(0, min(local_blocks, complete_blocks - selected_count))
        sink = max(0, min(sink_blocks, complete_blocks - selected_count - local))
        if complete_blocks <= 2048:
            width = selected_count + sink + local
            shape = (batch * kv_heads, width)
            if (self.selected_blocks is None or tuple(self.selected_blocks.shape) != shape
                    or self.selected_blocks.device != q_grouped.device):
                self.selected_blocks = torch.empty(shape, device=q_grouped.device, dtype=torch.int32)
            return get_extension().select_decode_blocks(q_grouped, stat_a, stat_b, selected_count, complete_blocks,
                                                        is_bf16, sink=sink, local=local, out=self.selected_blocks)
        # longer than the selection kernel's 2048-block limit: tensor code, as the reference does
        qf = q_grouped.float().unsqueeze(3)                                     # [B, Hkv, G, 1, D]
        if quest:
            bound = torch.where(qf >= 0, self.k_max[:, :, :complete_blocks].float().unsqueeze(2),
                                self.k_min[:, :, :complete_blocks].float().unsqueeze(2))
            scores = (qf * bound).sum(-1)
        else:
            scores = torch.matmul(q_grouped.float(), self.k_mean[:, :, :complete_blocks].float().transpose(-1, -2))
        scores = scores.amax(dim=2).reshape(batch * kv_heads, complete_blocks)
        return scores.topk(selected_count, dim=-1).indices.to(torch.int32).contiguous()

    # ------------------------------------------------------------------------- batch-dimension surgery
    def reorder(self, beam_idx: torch.Tensor) -> None:
        self._index_select_batch(beam_idx)

    def batch_select_indices(self, indices: torch.Tensor) -> None:
        self._index_select_batch(indices)

    def batch_repeat_interleave(self, repeats: int) -> None:
        for name in self._tensor_names():
            tensor = getattr(self, name)
            if tensor is not None:
                setattr(self, name, tensor.repeat_interleave(repeats, dim=0))
        self.selected_blocks = None

    def _index_select_batch(self, indices: torch.Tensor) -> None:
        for name in self._tensor_names():
            tensor = getattr(self, name)
            if tensor is not None:
                setattr(self, name, tensor.index_select(0, indices.to(tensor.device)))
        self.selected_blocks = None

    @staticmethod
    def _tensor_names() -> tuple[str, ...]:
        return ("k_fp16", "v_fp16", "k_packed", "k_scale", "v_packed_t", "v_scale_t", "k_mean", "k_min", "k_max")

    # ------------------------------------------------------------------------------------ crop / reset
    def crop(self, max_length: int) -> None:
        """Shorten the logical length (negative = drop that many tokens) and return the rounded physical
        tail to zero rows, so that the kernels' rounded views stay well defined."""
        if max_length < 0:
            max_length = max(self.seq_len + max_length, 0)
        new_len = min(self.seq_len, max_length)
        if new_len < self.seq_len:
            self._zero_physical_tail(new_len)
        self.seq_len = new_len

    def reset(self) -> None:
        self.seq_len = 0

    def _zero_physical_tail(self, logical_len: int) -> None:
        # K is cleared up to the next 64-token boundary, V up to the next 128-token boundary
        # (transformers_cache.py:237-253); both ranges are then re-quantised.
        if self.k_fp16 is None or self.v_fp16 is None:
            return
        key_end = min(max(PAGE, _round_up(logical_len, PAGE)), self.k_fp16.shape[2])
        value_end = min(_round_up(key_end, CAPACITY_QUANTUM), self.v_fp16.shape[2])
        if logical_len < key_end:
            self.k_fp16[:, :, logical_len:key_end].zero_()
            if self.k_packed is not None and self.k_scale is not None:
                self._quantize_k_range(self.k_fp16[:, :, logical_len:key_end].contiguous(), logical_len, key_end)
        if logical_len < value_end:
            self.v_fp16[:, :, logical_len:value_end].zero_()
            if self.v_packed_t is not None and self.v_scale_t is not None:
                self._quantize_v_range(logical_len, value_end)

    def _quantize_k_range(self, key_states: torch.Tensor, start: int, end: int) -> None:
        """Store and quantise K rows ``[start, end)``; no statistics refresh."""
        self._append(key_states, None, start, v_count=0, stats=False)

    def _quantize_v_range(self, start: int, end: int) -> None:
        """Re-quantise every V group overlapping ``[start, end)`` from the 16-bit cache."""
        self._append(None, None, start, k_count=0, v_count=end - start, keep_v=True, stats=False)

    def _refresh_k_means(self, start: int, end: int) -> None:
        """Recompute the statistics of the 64-token blocks lying entirely inside ``[start // 64 * 64, end)``."""
        self._append(None, None, start, k_count=end - start, v_count=0, keep_k=True)

    # ---------------------------------------------------------------------------------------- capacity
    def reserve(self, tokens: int) -> None:
        """Room for ``tokens`` tokens now, so that later appends neither move nor re-allocate anything (what a
        generation step captured in a CUDA graph needs).  The layer must already hold its first tokens."""
        if self.k_fp16 is None:
            raise RuntimeError("ThriftAttention cache layer has not been initialized")
        b, h, _, d = self.k_fp16.shape
        self._ensure_capacity(torch.empty(b, h, 0, d, dtype=self.k_fp16.dtype, device=self.k_fp16.device), tokens)

    def _ensure_capacity(self, like: torch.Tensor, required: int) -> None:
        """Allocate or grow every tensor to hold ``required`` tokens.  The first allocation takes
        ``max_cache_len`` when it is known, else 64 tokens; later ones double; the result is rounded up to
        128 tokens and never exceeds ``max_cache_len`` rounded up to 128 (transformers_cache.py:255-306)."""
        if self.k_fp16 is not None:
            if like.shape[0] != self.k_fp16.shape[0] or like.shape[1] != self.k_fp16.shape[1]:
                raise ValueError("ThriftAttentionCache batch/head shape changed unexpectedly")
            if like.dtype != self.k_fp16.dtype:
                raise ValueError("ThriftAttentionCache dtype changed unexpectedly")
            if required <= self.capacity:
                return

        batch, heads, _, head_dim = like.shape
        limit = self.max_cache_len
        if self.capacity == 0:
            wanted = limit if limit is not None else PAGE
        else:
            wanted = self.capacity * 2
        wanted = max(wanted, required)
        if limit is not None:
            wanted = min(wanted, limit)
        new_capacity = _round_up(wanted, CAPACITY_QUANTUM)
        if limit is not None:
            new_capacity = min(new_capacity, _round_up(limit, CAPACITY_QUANTUM))
        if new_capacity < required:
            raise ValueError("could not grow ThriftAttentionCache to required length")

        g = _group_size(self.quant_format)
        dev = like.device
        fresh = {
            "k_fp16": torch.zeros(batch, heads, new_capacity, head_dim, device=dev, dtype=like.dtype),
            "v_fp16": torch.zeros(batch, heads, new_capacity, head_dim, device=dev, dtype=like.dtype),
            "k_packed": torch.zeros(batch, heads, new_capacity, head_dim // 2, device=dev, dtype=torch.uint8),
            "k_scale": torch.zeros(batch, heads, new_capacity, head_dim // g, device=dev, dtype=torch.uint8)
            .view(_scale_dtype(self.quant_format)),
            "v_packed_t": torch.zeros(batch, heads, head_dim, new_capacity // 2, device=dev, dtype=torch.uint8),
            "v_scale_t": torch.zeros(batch, heads, head_dim, new_capacity // g, device=dev, dtype=torch.uint8)
            .view(_scale_dtype(self.quant_format)),
            "k_mean": torch.zeros(batch, heads, new_capacity // PAGE, head_dim, device=dev, dtype=like.dtype),
        }
        if self.track_minmax:
            fresh["k_min"] = torch.zeros_like(fresh["k_mean"])
            fresh["k_max"] = torch.zeros_like(fresh["k_mean"])

        if self.k_fp16 is not None:
            old = self.capacity
            for name in ("k_fp16", "v_fp16", "k_packed"):
                fresh[name][:, :, :old] = getattr(self, name)
            fresh["v_packed_t"][:, :, :, : old // 2] = self.v_packed_t
            fresh["v_scale_t"].view(torch.uint8)[:, :, :, : old // g] = self.v_scale_t.view(torch.uint8)
            for name in ("k_mean", "k_min", "k_max"):
                if name in fresh and getattr(self, name) is not None:
                    fresh[name][:, :, : old // PAGE] = getattr(self, name)
            # fp8 tensors do not support slice assignment on every build: go through uint8 views
            fresh["k_scale"].view(torch.uint8)[:, :, :old] = self.k_scale.view(torch.uint8)

        for name, tensor in fresh.items():
            setattr(self, name, tensor)
        self.capacity = new_capacity
        self.selected_blocks = None


def _raw(tensor: torch.Tensor) -> torch.Tensor:
    """fp8 scale tensors as bytes (indexing, concatenation and fills are not implemented for fp8 on every build)."""
    return tensor if tensor.dtype in (torch.float16, torch.bfloat16, torch.uint8) else tensor.view(torch.uint8)


@dataclass
class PagedThriftAttentionCacheLayer(ThriftAttentionCacheLayer):
    """The same layer over POOLS of 64-token pages behind a page table - the layout the decode kernel reads
    (``decode_attention(..., page_table=)``) and ``cache_append_paged`` writes.

    * pools (one set per layer): 16-bit K/V ``[pages, Hkv, 64, D]``, K codes ``[pages, Hkv, 64, D/2]`` + scales,
      V codes transposed inside a page ``[pages, Hkv, D, 32]`` + scales; ``page_table`` int32 ``[B, max_pages]``.
      With ``max_cache_len`` the pool holds every sequence at that length from the first append on; otherwise it
      starts small and doubles (the one place a copy is made) when the free list runs dry;
    * a sequence grows by taking page ids from the free list - nothing is moved (the reference, and the
      capacity-strided layer above, copy the whole slab: transformers_cache.py:255-306);
    * free pages hold zeros, so the rows behind the logical length read as zero rows, as the kernels expect;
      physical page 0 is never handed out and stays zero (what a gather reads where a sequence has no page);
    * block statistics stay indexed by logical block (``[B, Hkv, blocks, D]``, grown by doubling: 1/64 of K);
    * the decode step reads the pools in place.  Whatever wants contiguous tensors (a prefill over the cache,
      ``key_view`` / ``value_view``, the legacy-cache export) gets them by a gather, cached until the next change.
    """

    k_pool: torch.Tensor | None = None
    v_pool: torch.Tensor | None = None
    k4_pool: torch.Tensor | None = None
    ks_pool: torch.Tensor | None = None
    v4_pool: torch.Tensor | None = None
    vs_pool: torch.Tensor | None = None
    page_table: torch.Tensor | None = None          # device int32 [B, max_pages]; -1 = no page
    _pages: list | None = None                      # host mirror: per sequence, its page ids in order
    _free: list | None = None
    _gathered: dict | None = None

    # ------------------------------------------------------------------------------------------ shape helpers
    def _pools(self) -> tuple[torch.Tensor, ...]:
        return (self.k_pool, self.v_pool, self.k4_pool, self.ks_pool, self.v4_pool, self.vs_pool)

    def batch_size(self) -> int | None:
        return None if self._pages is None else len(self._pages)

    def kv_heads(self) -> int:
        if self.k_pool is None:
            raise RuntimeError("ThriftAttention cache layer has not been initialized")
        return int(self.k_pool.shape[1])

    # ------------------------------------------------------------------------------------------ page management
    def _new_pools(self, pages: int, heads: int, head_dim: int, dtype: torch.dtype, device) -> dict[str, torch.Tensor]:
        g = _group_size(self.quant_format)
        u8 = dict(device=device, dtype=torch.uint8)
        return {"k_pool": torch.zeros(pages, heads, PAGE, head_dim, device=device, dtype=dtype),
                "v_pool": torch.zeros(pages, heads, PAGE, head_dim, device=device, dtype=dtype),
                "k4_pool": torch.zeros(pages, heads, PAGE, head_dim // 2, **u8),
                "ks_pool": torch.zeros(pages, heads, PAGE, head_dim // g, **u8).view(_scale_dtype(self.quant_format)),
                "v4_pool": torch.zeros(pages, heads, head_dim, PAGE // 2, **u8),
                "vs_pool": torch.zeros(pages, heads, head_dim, PAGE // g, **u8).view(_scale_dtype(self.quant_format))}

    def _grow_pool(self, extra_pages: int) -> None:
        old = int(self.k_pool.shape[0])
        fresh = self._new_pools(extra_pages, self.k_pool.shape[1], self.k_pool.shape[3], self.k_pool.dtype, self.k_pool.device)
        for name, tensor in fresh.items():
            cur = getattr(self, name)
            setattr(self, name, torch.cat([_raw(cur), _raw(tensor)]).view(cur.dtype))
        self._free.extend(range(old, old + extra_pages))

    def _take_pages(self, count: int) -> list[int]:
        if count > len(self._free):
            self._grow_pool(max(count - len(self._free), int(self.k_pool.shape[0])))
        taken, self._free = self._free[:count], self._free[count:]
        return taken

    def _release_pages(self, pages: list[int]) -> None:
        """Back to the free list, as zeros."""
        if not pages:
            return
        idx = torch.tensor(pages, device=self.k_pool.device, dtype=torch.long)
        for pool in self._pools():
            _raw(pool).index_fill_(0, idx, 0)
        self._free.extend(pages)

    def _upload_table(self) -> None:
        """Host page lists -> device table.  The table is as wide as ``max_cache_len`` needs when that is known, else
        it doubles when a sequence outgrows it."""
        need = max(2, max(len(row) for row in self._pages))
        width = int(self.page_table.shape[1]) if self.page_table is not None else 0
        if self.max_cache_len is not None:
            width = max(width, (self.max_cache_len + PAGE - 1) // PAGE)
        if width < need:
            width = max(need, 2 * width)
        host = torch.full((len(self._pages), width), -1, dtype=torch.int32)
        for b, row in enumerate(self._pages):
            if row:
                host[b, : len(row)] = torch.tensor(row, dtype=torch.int32)
        if self.page_table is not None and tuple(self.page_table.shape) == tuple(host.shape):
            self.page_table.copy_(host)      # in place: launches captured in a CUDA graph keep reading this tensor
        else:
            self.page_table = host.to(self.k_pool.device)

    def reserve(self, tokens: int) -> None:
        """Pages for ``tokens`` tokens per sequence now (taken from the pool and entered in the page table), so that
        later appends change nothing on the host side.  The layer must already hold its first tokens."""
        if self.k_pool is None:
            raise RuntimeError("ThriftAttention cache layer has not been initialized")
        _, h, _, d = self.k_pool.shape
        capacity = self.capacity
        self._ensure_capacity(torch.empty(len(self._pages), h, 0, d, dtype=self.k_pool.dtype, device=self.k_pool.device), tokens)
        self.capacity = max(capacity, self.capacity)

    def _ensure_capacity(self, like: torch.Tensor, required: int) -> None:
        batch, heads, _, head_dim = like.shape
        if self.k_pool is None:
            per_seq = (self.max_cache_len + PAGE - 1) // PAGE if self.max_cache_len is not None else 2 * ((required + PAGE - 1) // PAGE)
            for name, tensor in self._new_pools(1 + batch * max(per_seq, 1), heads, head_dim, like.dtype, like.device).items():
                setattr(self, name, tensor)
            self._pages = [[] for _ in range(batch)]
            self._free = list(range(1, int(self.k_pool.shape[0])))          # page 0: the zero page
        else:
            if batch != len(self._pages) or heads != self.k_pool.shape[1]:
                raise ValueError("ThriftAttentionCache batch/head shape changed unexpectedly")
            if like.dtype != self.k_pool.dtype:
                raise ValueError("ThriftAttentionCache dtype changed unexpectedly")
        need = max(1, (required + PAGE - 1) // PAGE)
        changed = self.page_table is None
        for row in self._pages:
            if len(row) < need:
                row.extend(self._take_pages(need - len(row)))
                changed = True
        if changed:
            self._upload_table()
        # statistics by logical block
        blocks = int(self.page_table.shape[1])
        if self.k_mean is None or self.k_mean.shape[2] < blocks:
            names = ("k_mean", "k_min", "k_max") if self.track_minmax else ("k_mean",)
            for name in names:
                fresh = torch.zeros(batch, heads, blocks, head_dim, device=like.device, dtype=like.dtype)
                cur = getattr(self, name)
                if cur is not None:
                    fresh[:, :, : cur.shape[2]] = cur
                setattr(self, name, fresh)
        self.capacity = need * PAGE
        self.selected_blocks = None

    # ------------------------------------------------------------------------------------------ update
    def update(self, key_states: torch.Tensor, value_states: torch.Tensor,
               cache_kwargs: dict[str, Any] | None = None) -> tuple[torch.Tensor, torch.Tensor]:
        """Append through the page table (one launch).  Returns the logical 16-bit K/V - gathered, which costs a
        copy of the layer; callers that read the cache in place (the registered attention function does) should
        pass ``cache_kwargs={"thrift_return_new_states": True}`` or use ``append``, and get the new rows back."""
        self.append(key_states, value_states, cache_kwargs)
        if cache_kwargs is not None and cache_kwargs.get("thrift_return_new_states"):
            return key_states, value_states
        return self.key_view(), self.value_view()

    def append(self, key_states: torch.Tensor, value_states: torch.Tensor, cache_kwargs: dict[str, Any] | None = None) -> None:
        if key_states.ndim != 4 or value_states.ndim != 4:
            raise ValueError("KV cache tensors must be [batch, heads, seq, head_dim]")
        if key_states.shape != value_states.shape:
            raise ValueError("key_states and value_states must have identical shapes")
        if key_states.dtype not in (torch.float16, torch.bfloat16):
            raise ValueError("KV cache tensors must be float16 or bfloat16")
        if key_states.dtype != value_states.dtype:
            raise ValueError("key_states and value_states must have the same dtype")
        start = _cache_position_start(cache_kwargs, self.seq_len)
        token_count = key_states.shape[2]
        end = start + token_count
        if self.max_cache_len is not None and end > self.max_cache_len:
            raise ValueError(f"ThriftAttentionCache length {end} exceeds max_cache_len={self.max_cache_len}")
        self._ensure_capacity(key_states, end)
        self.seq_len = max(self.seq_len, end)
        if token_count:
            self._append(key_states.contiguous(), value_states.contiguous(), start)

    def _append(self, key_states: torch.Tensor | None, value_states: torch.Tensor | None, start: int, *,
                k_count: int | None = None, v_count: int | None = None, keep_k: bool = False, keep_v: bool = False,
                stats: bool = True) -> None:
        self._gathered = None
        get_extension().cache_append_paged(
            key_states, value_states, self.k_pool, self.v_pool, self.k4_pool, self.ks_pool, self.v4_pool, self.vs_pool,
            self.page_table, start=start, k_count=k_count, v_count=v_count,
            k_mean=self.k_mean if stats else None, k_min=self.k_min if stats else None,
            k_max=self.k_max if stats else None, is_mx=self.quant_format == "mxfp4", stat_block=PAGE,
            keep_k=keep_k, keep_v=keep_v)

    # ------------------------------------------------------------------------------------------- views (gathers)
    def _gather(self, name: str, tokens: int) -> torch.Tensor:
        """Contiguous ``[B, Hkv, tokens, X]`` (or ``[B, Hkv, D, tokens/2 | tokens/G]`` for V codes and scales) of the
        first ``tokens`` token positions; positions without a page read as zeros."""
        if self.k_pool is None or self.page_table is None:
            raise RuntimeError("ThriftAttention cache layer has not been initialized")
        self._gathered = self._gathered or {}
        key = (name, tokens)
        if key in self._gathered:
            return self._gathered[key]
        pool = getattr(self, name)
        n = (tokens + PAGE - 1) // PAGE
        have = min(n, int(self.page_table.shape[1]))
        picked = _raw(pool)[self.page_table[:, :have].long().clamp_min(0)]      # [B, have, Hkv, 64 | D, X]; no page -> page 0
        if have < n:
            pad = torch.zeros(picked.shape[0], n - have, *picked.shape[2:], device=picked.device, dtype=picked.dtype)
            picked = torch.cat([picked, pad], dim=1)
        if name in ("v4_pool", "vs_pool"):
            if tokens % PAGE:
                raise ValueError("transposed V views are cut at page boundaries")
            out = picked.permute(0, 2, 3, 1, 4).reshape(picked.shape[0], picked.shape[2], picked.shape[3], -1)
        else:
            out = picked.permute(0, 2, 1, 3, 4).reshape(picked.shape[0], picked.shape[2], n * PAGE, picked.shape[4])[:, :, :tokens]
        out = out.contiguous().view(pool.dtype)
        self._gathered[key] = out
        return out

    def key_view(self) -> torch.Tensor:
        return self._gather("k_pool", self.seq_len)

    def value_view(self) -> torch.Tensor:
        return self._gather("v_pool", self.seq_len)

    def packed_views(self) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
        kernel_len = self.kernel_len()
        v_len = _round_up(kernel_len, CAPACITY_QUANTUM)
        return (self._gather("k4_pool", kernel_len), self._gather("v4_pool", v_len),
                self._gather("ks_pool", kernel_len), self._gather("vs_pool", v_len))

    def hi_kernel_views(self) -> tuple[torch.Tensor, torch.Tensor]:
        n = self.kernel_len()
        return self._gather("k_pool", n), self._gather("v_pool", n)

    # ------------------------------------------------------------------------- batch-dimension surgery
    def batch_repeat_interleave(self, repeats: int) -> None:
        if self._pages is None:
            return
        self._index_select_batch(torch.arange(len(self._pages)).repeat_interleave(repeats))

    def _index_select_batch(self, indices: torch.Tensor) -> None:
        """New sequence i becomes a COPY of old sequence indices[i] (beams diverge afterwards, so pages are not shared)."""
        if self._pages is None:
            return
        self._gathered = None
        rows = [int(i) for i in indices.tolist()]
        new_pages = [self._take_pages(len(self._pages[src])) for src in rows]
        dst = [pg for row in new_pages for pg in row]
        src = [pg for r in rows for pg in self._pages[r]]
        if dst:
            di = torch.tensor(dst, device=self.k_pool.device, dtype=torch.long)
            si = torch.tensor(src, device=self.k_pool.device, dtype=torch.long)
            for pool in self._pools():
                raw = _raw(pool)
                raw.index_copy_(0, di, raw.index_select(0, si))
        old = [pg for row in self._pages for pg in row]
        self._pages = new_pages
        self._release_pages(old)
        sel = indices.to(self.k_pool.device)
        for name in ("k_mean", "k_min", "k_max"):
            tensor = getattr(self, name)
            if tensor is not None:
                setattr(self, name, tensor.index_select(0, sel))
        self._upload_table()
        self.selected_blocks = None

    # ------------------------------------------------------------------------------------ crop / reset
    def crop(self, max_length: int) -> None:
        if max_length < 0:
            max_length = max(self.seq_len + max_length, 0)
        new_len = min(self.seq_len, max_length)
        if new_len < self.seq_len and self._pages is not None:
            self._gathered = None
            keep = max(1, (new_len + PAGE - 1) // PAGE)
            dropped = [pg for row in self._pages for pg in row[keep:]]
            self._pages = [row[:keep] for row in self._pages]
            self._release_pages(dropped)
            self._upload_table()
            key_end = keep * PAGE
            if new_len < key_end:
                # zero rows behind the new length inside the last page, codes and scales re-derived from them
                self._append(None, None, new_len, k_count=key_end - new_len, v_count=key_end - new_len, stats=False)
            self.capacity = keep * PAGE
        self.seq_len = new_len

    def reset(self) -> None:
        if self._pages is not None:
            self._gathered = None
            dropped = [pg for row in self._pages for pg in row]
            self._pages = [[] for _ in self._pages]
            self._release_pages(dropped)
            self.page_table = None
        self.seq_len = 0
        self.capacity = 0

    def _zero_physical_tail(self, logical_len: int) -> None:       # the slab layer's helper; crop above does the work
        raise NotImplementedError


class ThriftAttentionCache:
    """Cache object handed to ``model(..., past_key_values=cache)``: one ``ThriftAttentionCacheLayer``
    per attention layer plus the Transformers cache protocol (``update``, ``get_seq_length``,
    ``get_mask_sizes``, ``crop``, ``reset``, ``reorder_cache``, ``batch_*``).  It implements the protocol
    directly instead of subclassing, because the base-class constructor differs between
    Transformers releases (transformers_cache.py:478-567)."""

    def __init__(self, *, config: AttentionConfig | None = None, max_cache_len: int | None = None,
                 paged: bool = False) -> None:
        """``paged=True`` keeps every layer in pools of 64-token pages behind a page table
        (``PagedThriftAttentionCacheLayer``) instead of capacity-strided slabs."""
        self.config = config or AttentionConfig()
        self._max_cache_len = max_cache_len
        self.paged = bool(paged)
        self.layers: list[ThriftAttentionCacheLayer] = []
        self._seen_tokens = 0
        self.prefill_real_seq_len: int | None = None
        # device-length mode (enable_device_length): the number of cached tokens lives in this one-element int32
        # CUDA tensor and the decode launches no longer depend on it
        self.device_length: torch.Tensor | None = None
        self.device_max_len = 0
        self.device_splits: int | None = None

    # ------------------------------------------------------------------------- length in device memory
    def enable_device_length(self, max_len: int | None = None, splits: int | None = None) -> torch.Tensor:
        """Switch the decode steps of this cache to a sequence length kept ON THE GPU, so that a whole single-token
        forward pass of the model - every layer's append + attention through the registered attention function - can
        be captured in a CUDA graph once and replayed for every token.

        Call it after the prefill.  Every layer gets room for ``max_len`` tokens now (default: ``max_cache_len``
        rounded up to whole 64-token pages).  From here on ``update`` with one new token (while this cache is the
        active one) stores nothing and hands the new rows on, and the attention function appends and attends through
        ``device_length_decode_step``; the caller feeds the model ``position_ids`` / ``cache_position`` derived from
        the returned tensor (``device_positions``) and ends every forward pass with ``advance_device_length()``.
        The Python-side lengths go stale meanwhile; ``sync_device_length`` / ``disable_device_length`` refresh them.
        An attention mask handed to a single-token step is ignored in this mode (all sequences of the cache have the
        same length, every cached token is visible).
        ``splits``: chains per KV head of the attention kernel (default: the choice for ``max_len``)."""
        if not self.layers or self.layers[0].seq_len == 0:
            raise RuntimeError("enable_device_length needs a filled cache (call it after the prefill)")
        tokens = self.layers[0].seq_len
        if any(layer.seq_len != tokens for layer in self.layers):
            raise RuntimeError("the layers of the cache hold different numbers of tokens")
        if max_len is None:
            if self._max_cache_len is None:
                raise ValueError("enable_device_length needs max_len or a cache built with max_cache_len")
            max_len = self._max_cache_len
        max_len = _round_up(int(max_len), PAGE)
        if max_len < tokens:
            raise ValueError(f"max_len={max_len} is below the {tokens} tokens already cached")
        for layer in self.layers:
            layer.reserve(max_len)
        first = self.layers[0]
        device = (first.k_pool if isinstance(first, PagedThriftAttentionCacheLayer) else first.k_fp16).device
        self.device_length = torch.tensor([tokens], dtype=torch.int32, device=device)
        self.device_max_len = max_len
        self.device_splits = splits
        return self.device_length

    def device_positions(self) -> torch.Tensor:
        """``cache_position`` of the next token, ``[1]`` int64, computed on the GPU from the device-side length
        (``.view(1, 1)`` of it is the ``position_ids`` of a batch whose sequences have the same length)."""
        if self.device_length is None:
            raise RuntimeError("the cache is not in device-length mode")
        return self.device_length.to(torch.long)

    def advance_device_length(self, count: int = 1) -> None:
        """End of a forward pass in device-length mode: length += count (one tiny launch, capturable)."""
        if self.device_length is None:
            raise RuntimeError("the cache is not in device-length mode")
        get_extension().advance_length(self.device_length, count, self.device_max_len)

    def sync_device_length(self) -> int:
        """Read the device-side length back (a synchronisation) and bring the Python-side lengths up to date."""
        if self.device_length is None:
            raise RuntimeError("the cache is not in device-length mode")
        tokens = int(self.device_length.item())
        for layer in self.layers:
            layer.seq_len = tokens
            if isinstance(layer, PagedThriftAttentionCacheLayer):
                layer._gathered = None
        self._seen_tokens = tokens
        return tokens

    def disable_device_length(self) -> int:
        """Back to lengths kept in Python; returns the number of cached tokens."""
        tokens = self.sync_device_length()
        self.device_length = None
        return tokens

    @classmethod
    def from_model(cls, model: object, *, config: AttentionConfig | None = None,
                   max_cache_len: int | None = None, paged: bool = False) -> "ThriftAttentionCache":
        if max_cache_len is None:
            max_cache_len = getattr(getattr(model, "config", None), "max_position_embeddings", None)
        return cls(config=config, max_cache_len=max_cache_len, paged=paged)

    # ------------------------------------------------------------------------------------ properties
    @property
    def seen_tokens(self) -> int:
        return self._seen_tokens

    @property
    def max_cache_len(self) -> int | None:
        return self._max_cache_len

    @property
    def is_compileable(self) -> bool:
        return False

    @property
    def is_initialized(self) -> bool:
        return len(self.layers) > 0

    @property
    def is_sliding(self) -> list[bool]:
        return [False for _ in self.layers]

    @property
    def max_batch_size(self) -> int | None:
        for layer in self.layers:
            if isinstance(layer, PagedThriftAttentionCacheLayer):
                if layer.batch_size() is not None:
                    return layer.batch_size()
            elif layer.k_fp16 is not None:
                return int(layer.k_fp16.shape[0])
        return None

    # -------------------------------------------------------------------------------------- protocol
    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int | None = None,
               cache_kwargs: dict[str, Any] | None = None, **_: Any) -> tuple[torch.Tensor, torch.Tensor]:
        if layer_idx is None:
            raise ValueError("ThriftAttentionCache.update requires layer_idx")
        layer = self.layer(layer_idx)
        if self.device_length is not None:
            if key_states.shape[2] != 1 or layer.seq_len == 0 or get_active_thriftattention_cache() is not self:
                raise RuntimeError("the cache is in device-length mode, which serves single-token steps through the registered "
                                   "attention function only (the Python-side lengths are stale): call disable_device_length() "
                                   "before any other update")
            # the registered attention function appends these rows itself, at the position it reads on the GPU
            # (device_length_decode_step)
            return key_states, value_states
        if self.paged and get_active_thriftattention_cache() is self:
            # the registered attention function reads the pools in place: spare the gather of the full K/V
            cache_kwargs = dict(cache_kwargs or {}, thrift_return_new_states=True)
        key, value = layer.update(key_states, value_states, cache_kwargs)
        if layer_idx == 0:
            self._seen_tokens = layer.seq_len
        return key, value

    def layer(self, layer_idx: int) -> ThriftAttentionCacheLayer:
        kind = PagedThriftAttentionCacheLayer if self.paged else ThriftAttentionCacheLayer
        while len(self.layers) <= layer_idx:
            self.layers.append(kind(
                max_cache_len=self._max_cache_len,
                quant_format=self.config.quant_format,
                track_minmax=self.config.selection == "quest"))
        return self.layers[layer_idx]

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self.layers[layer_idx].seq_len if layer_idx < len(self.layers) else 0

    def get_mask_sizes(self, query_length: int, layer_idx: int) -> tuple[int, int]:
        if layer_idx >= len(self.layers):
            return query_length, 0
        return self.layers[layer_idx].seq_len + query_length, 0

    def get_max_cache_shape(self) -> int | None:
        return self._max_cache_len

    def get_max_length(self) -> int | None:
        return self._max_cache_len

    def get_usable_length(self, new_seq_length: int, layer_idx: int = 0) -> int:
        previous = self.get_seq_length(layer_idx)
        if self._max_cache_len is None or previous + new_seq_length <= self._max_cache_len:
            return previous
        return max(self._max_cache_len - new_seq_length, 0)

    def reorder_cache(self, beam_idx: torch.Tensor) -> None:
        for layer in self.layers:
            layer.reorder(beam_idx)

    def batch_select_indices(self, indices: torch.Tensor) -> None:
        for layer in self.layers:
            layer.batch_select_indices(indices)

    def batch_repeat_interleave(self, repeats: int) -> None:
        for layer in self.layers:
            layer.batch_repeat_interleave(repeats)

    def crop(self, max_length: int) -> None:
        for layer in self.layers:
            layer.crop(max_length)
        self._seen_tokens = self.get_seq_length(0)

    def reset(self) -> None:
        for layer in self.layers:
            layer.reset()
        self._seen_tokens = 0

    def to_legacy_cache(self) -> tuple[tuple[torch.Tensor, torch.Tensor], ...]:
        return tuple((layer.key_view(), layer.value_view()) for layer in self.layers)

    def __getitem__(self, layer_idx: int) -> tuple[torch.Tensor, torch.Tensor]:
        layer = self.layer(layer_idx)
        return layer.key_view(), layer.value_view()

    def __len__(self) -> int:
        return len(self.layers)


# ------------------------------------------------------------------------------------------------
# Attention over the cache
# ------------------------------------------------------------------------------------------------
def _layer_format(layer: ThriftAttentionCacheLayer, config: AttentionConfig):
    quant_format = get_quant_format(config.quant_format)          # NotImplementedError for unknown names
    if quant_format.name != layer.quant_format:
        raise ValueError(f"cache layer holds {layer.quant_format!r} codes but the call asks for {quant_format.name!r}")
    return quant_format


def cached_decode_attention(query: torch.Tensor, cache: ThriftAttentionCache, layer_idx: int,
                            config: AttentionConfig) -> torch.Tensor:
    """One decode step ``[B, Hq, 1, D]`` over layer ``layer_idx`` of ``cache``; returns ``[B, Hq, 1, D]``.

    Launches: quantise the grouped query, select blocks, split-KV attention (+ its merge) — queued by one
    library call on the common path, operator by operator otherwise.  K and V are read in place through
    capacity strides — nothing is copied (transformers_cache.py:570-619)."""
    layer = cache.layer(layer_idx)
    if layer.seq_len == 0:
        raise RuntimeError("ThriftAttention decode cache is empty")
    quant_format = _layer_format(layer, config)

    q = query.contiguous()
    is_bf16 = q.dtype == torch.bfloat16
    paged = isinstance(layer, PagedThriftAttentionCacheLayer)
    kv_heads = layer.kv_heads() if paged else layer.key_view().shape[1]
    q_grouped = _group_single_query(q, kv_heads)
    fmt = quant_format.name
    if paged:
        fused = _fused_decode_step(q_grouped, layer, config, fmt) if config.method == "thrift" else None
        if fused is None:
            fused = _paged_decode_step(q_grouped, layer, config, quant_format)
        return _ungroup_single_query(fused, q.shape[1])
    if config.method == "thrift":
        fused = _fused_decode_step(q_grouped, layer, config, fmt)
        if fused is not None:
            return _ungroup_single_query(fused, q.shape[1])
    q_packed, q_scale = quant_format.quantize(q_grouped, is_bf16=is_bf16)
    k_packed, v_packed_t, k_scale, v_scale_t = layer.packed_views()
    ext = get_extension()

    if config.method == "fp4":
        out = getattr(ext, f"fp4_attention_single_query_{fmt}_packed")(q_packed, k_packed, v_packed_t, q_scale, k_scale,
                                                                       v_scale_t, is_bf16)
        return _ungroup_single_query(out, q.shape[1])
    if config.method != "thrift":
        raise ValueError(f"unsupported ThriftAttention method {config.method!r}")

    selected_blocks = select_cached_decode_blocks(q_grouped, layer, config)
    out = getattr(ext, f"thrift_attention_single_query_{fmt}_packed")(
        q_grouped, layer.key_view(), layer.value_view(), selected_blocks, q_packed, k_packed, v_packed_t, q_scale,
        k_scale, v_scale_t, is_bf16)
    return _ungroup_single_query(out, q.shape[1])


def _paged_decode_step(q_grouped: torch.Tensor, layer: "PagedThriftAttentionCacheLayer", config: AttentionConfig,
                       quant_format) -> torch.Tensor:
    """The decode step over a paged layer: quantise q, select blocks from the (logical) statistics, then split-KV
    attention that reads the page pools in place through the layer's page table."""
    if config.method not in ("thrift", "fp4"):
        raise ValueError(f"unsupported ThriftAttention method {config.method!r}")
    is_bf16 = q_grouped.dtype == torch.bfloat16
    q_packed, q_scale = quant_format.quantize(q_grouped, is_bf16=is_bf16)
    selected = select_cached_decode_blocks(q_grouped, layer, config) if config.method == "thrift" else None
    return get_extension().decode_attention(
        q_grouped, layer.k_pool, layer.v_pool, selected, q_packed, layer.k4_pool, layer.v4_pool, q_scale, layer.ks_pool,
        layer.vs_pool, is_mx=quant_format.name == "mxfp4", is_bf16=is_bf16, kv_len=layer.kernel_len(),
        page_table=layer.page_table)


def _fused_decode_step(q_grouped: torch.Tensor, layer: ThriftAttentionCacheLayer, config: AttentionConfig,
                       fmt: str) -> torch.Tensor | None:
    """Quantise q + select + attend + merge through one library call when the step is the common one (score-based
    selection over at most 2048 complete blocks of a 64-token-block cache); ``None`` sends the caller down the
    operator-by-operator path, which computes the same thing."""
    ext = get_extension()
    step = getattr(ext, "cached_decode_step", None)
    if step is None or config.selection not in ("block_mean", "quest") or config.block_size != PAGE:
        return None
    quest = config.selection == "quest"
    stat_a, stat_b = (layer.k_min, layer.k_max) if quest else (layer.k_mean, None)
    complete_blocks = layer.seq_len // PAGE
    if stat_a is None or (quest and stat_b is None) or complete_blocks > 2048 or q_grouped.dtype != stat_a.dtype:
        return None
    selected_count = resolve_top_k(complete_blocks, causal=False, top_k=config.top_k, fraction=config.fraction)
    local = max(0, min(getattr(config, "local_blocks", 0), complete_blocks - selected_count))
    sink = max(0, min(getattr(config, "sink_blocks", 0), complete_blocks - selected_count - local))
    if selected_count == 0:
        sink = local = 0
    if isinstance(layer, PagedThriftAttentionCacheLayer):
        out, layer.selected_blocks = step(q_grouped, layer.k_pool, layer.v_pool, layer.k4_pool, layer.ks_pool, layer.v4_pool,
                                          layer.vs_pool, stat_a, stat_b, kv_len=layer.kernel_len(),
                                          n_select_blocks=complete_blocks, top_k=selected_count, sink=sink, local=local,
                                          is_mx=fmt == "mxfp4", sel_out=layer.selected_blocks, page_table=layer.page_table)
        return out
    out, layer.selected_blocks = step(q_grouped, layer.k_fp16, layer.v_fp16, layer.k_packed, layer.k_scale,
                                      layer.v_packed_t, layer.v_scale_t, stat_a, stat_b, kv_len=layer.kernel_len(),
                                      n_select_blocks=complete_blocks, top_k=selected_count, sink=sink, local=local,
                                      is_mx=fmt == "mxfp4", sel_out=layer.selected_blocks)
    return out


def device_length_decode_step(query: torch.Tensor, key_states: torch.Tensor, value_states: torch.Tensor,
                              cache: ThriftAttentionCache, layer_idx: int, config: AttentionConfig, length: torch.Tensor, *,
                              max_len: int, splits: int | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """One layer of one generation step with the sequence length kept ON THE GPU: stores the token's
    ``key_states`` / ``value_states`` ``[B, Hkv, 1, D]`` at position ``length[0]`` of layer ``layer_idx`` and returns
    the attention of ``query`` ``[B, Hq, 1, D]`` over the ``length[0] + 1`` cached tokens.

    ``length`` is a one-element int32 CUDA tensor.  No launch depends on its value (the kernels read it), so the
    calls of all layers followed by one ``advance_length(length, 1, max_len)`` can be captured in a CUDA graph once
    and replayed for every token; the result is bit for bit the one of ``update`` + ``cached_decode_attention`` run
    with the same chain count.  The reference keeps the length in Python (transformers_cache.py:64-84), which rules
    that out.  Requirements: the layer holds its prompt (filled through ``update``) and room for ``max_len`` tokens
    (``reserve``; ``max_len`` a multiple of 64); ``method="thrift"`` with block-mean or Quest selection over 64-token
    blocks.  The layer's Python-side ``seq_len`` is not touched: set it from ``length`` when leaving the graph."""
    layer = cache.layer(layer_idx)
    quant_format = _layer_format(layer, config)
    if config.method != "thrift" or config.selection not in ("block_mean", "quest") or config.block_size != PAGE:
        raise ValueError("the device-length step supports method='thrift' with block_mean / quest selection and 64-token blocks")
    paged = isinstance(layer, PagedThriftAttentionCacheLayer)
    quest = config.selection == "quest"
    stat_a, stat_b = (layer.k_min, layer.k_max) if quest else (layer.k_mean, None)
    if stat_a is None or (quest and stat_b is None):
        raise RuntimeError("ThriftAttention cache layer has not been initialized")
    if paged:
        bufs = (layer.k_pool, layer.v_pool, layer.k4_pool, layer.ks_pool, layer.v4_pool, layer.vs_pool)
        table = layer.page_table
        room = min(len(row) for row in layer._pages) * PAGE
        layer._gathered = None
    else:
        bufs = (layer.k_fp16, layer.v_fp16, layer.k_packed, layer.k_scale, layer.v_packed_t, layer.v_scale_t)
        table = None
        room = layer.capacity
    if max_len % PAGE != 0 or max_len <= 0 or room < max_len:
        raise ValueError(f"the layer holds room for {room} tokens, max_len={max_len} asked (a multiple of {PAGE}): call reserve()")
    q = query.contiguous()
    q_grouped = _group_single_query(q, bufs[0].shape[1])
    ext = get_extension()
    is_mx = quant_format.name == "mxfp4"
    ext.cache_append_at(key_states.contiguous(), value_states.contiguous(), *bufs, length, offset=0, page_table=table,
                        k_mean=layer.k_mean, k_min=layer.k_min, k_max=layer.k_max, is_mx=is_mx, stat_block=PAGE)
    grouped_out = None if out is None else _group_single_query(out, bufs[0].shape[1])
    result, layer.selected_blocks = ext.cached_decode_step_at(
        q_grouped, *bufs, stat_a, stat_b, length, offset=key_states.shape[2], max_len=max_len, top_k=config.top_k,
        fraction=config.fraction, sink=getattr(config, "sink_blocks", 0), local=getattr(config, "local_blocks", 0),
        is_mx=is_mx, splits=splits, sel_out=layer.selected_blocks, out=grouped_out, page_table=table)
    return _ungroup_single_query(result, q.shape[1])


def cached_prefill_attention(query: torch.Tensor, cache: ThriftAttentionCache, layer_idx: int,
                             config: AttentionConfig, *, seq_major_out: bool = False) -> torch.Tensor:
    """Prefill ``[B, Hq, Sq, D]`` against the K/V that ``update`` has just stored in layer ``layer_idx``;
    the result is ``[B, Hq, Sq, D]``, or ``[B, Sq, Hq, D]`` with ``seq_major_out``.

    The reference re-quantises the whole K and V into the tiled kernel's own layouts here
    (transformers_cache.py:622-680).  The sm_100a prefill kernel reads plain K rows and capacity
    strides, so only the query is quantised and K/V codes, scales and block statistics come straight
    from the cache."""
    layer = cache.layer(layer_idx)
    quant_format = _layer_format(layer, config)
    q = query.contiguous()
    is_bf16 = q.dtype == torch.bfloat16
    q_packed, q_scale = quant_format.quantize(q, is_bf16=is_bf16)
    k_packed, v_packed_t, k_scale, v_scale_t = layer.packed_views()
    k_hi, v_hi = layer.hi_kernel_views()
    ext = get_extension()
    common = dict(causal=config.causal, is_mx=quant_format.name == "mxfp4", is_bf16=is_bf16,
                  block_size=config.block_size, k_permuted=False)
    if seq_major_out:
        common["seq_major_out"] = True

    if config.method == "fp4":
        out = ext.prefill_attention(None, None, None, None, q_packed, k_packed, v_packed_t, q_scale, k_scale,
                                    v_scale_t, **common)
    elif config.method != "thrift":
        raise ValueError(f"unsupported ThriftAttention method {config.method!r}")
    else:
        selected_blocks = select_cached_prefill_blocks(q, layer.key_view(), layer, config,
                                                       real_q_len=cache.prefill_real_seq_len, is_bf16=is_bf16)
        out = ext.prefill_attention(q, k_hi, v_hi, selected_blocks, q_packed, k_packed, v_packed_t, q_scale, k_scale,
                                    v_scale_t, **common)
    if isinstance(layer, PagedThriftAttentionCacheLayer):
        layer._gathered = None          # the contiguous copies made for this call (the stream keeps them alive until it ran)
    return out


# ------------------------------------------------------------------------------------------------
# Selection over the cache
# ------------------------------------------------------------------------------------------------
def select_cached_decode_blocks(q_grouped: torch.Tensor, layer: ThriftAttentionCacheLayer,
                                config: AttentionConfig) -> torch.Tensor:
    if config.selection in ("block_mean", "quest"):
        return select_topk_key_blocks(q_grouped, layer, config)
    if config.selection == "local":
        return select_local_key_blocks(q_grouped, layer, config)
    raise ValueError(f"unsupported cached decode selection {config.selection!r}")


def select_topk_key_blocks(q_grouped: torch.Tensor, layer: ThriftAttentionCacheLayer,
                           config: AttentionConfig) -> torch.Tensor:
    extra = {}
    if config.selection == "quest":
        extra["selection"] = "quest"
    if getattr(config, "sink_blocks", 0) or getattr(config, "local_blocks", 0):
        extra.update(sink_blocks=config.sink_blocks, local_blocks=config.local_blocks)
    return layer.select_key_blocks(q_grouped, top_k=config.top_k, fraction=config.fraction,
                                   block_size=config.block_size, **extra)


def select_local_key_blocks(q_grouped: torch.Tensor, layer: ThriftAttentionCacheLayer,
                            config: AttentionConfig) -> torch.Tensor:
    """The most recent complete blocks (transformers_cache.py:714-731)."""
    complete_blocks = layer.seq_len // config.block_size
    selected_count = resolve_top_k(complete_blocks, causal=False, top_k=config.top_k, fraction=config.fraction)
    flat_heads = q_grouped.shape[0] * q_grouped.shape[1]
    if selected_count == 0:
        return torch.empty(flat_heads, 0, device=q_grouped.device, dtype=torch.int32)
    return get_extension().single_query_local_topk(q_grouped, selected_count, complete_blocks)


def select_cached_prefill_blocks(q: torch.Tensor, k: torch.Tensor, layer: ThriftAttentionCacheLayer,
                                 config: AttentionConfig, real_q_len: int | None = None,
                                 is_bf16: bool = False) -> torch.Tensor:
    if config.selection in ("block_mean", "quest"):
        return _select_block_pairs_from_cached_stats(q, layer, config, real_q_len=real_q_len, is_bf16=is_bf16)
    if config.selection == "local":
        return select_local_block_pairs(q, k, causal=config.causal, top_k=config.top_k, fraction=config.fraction,
                                        block_size=config.block_size, is_bf16=is_bf16)
    raise ValueError(f"unsupported cached prefill selection {config.selection!r}")


def _query_block_means(q: torch.Tensor, block_size: int, real_q_len: int | None) -> torch.Tensor:
    """Mean query of every q block, 16-bit ``[B, Hq, Sq/block, D]``.  With ``real_q_len`` shorter than the
    (padded) query, padding rows are left out: the partial block averages its real rows only and blocks
    made of padding alone are zero (transformers_cache.py:789-808)."""
    batch, q_heads, q_len, head_dim = q.shape
    q_mean, _, _ = get_extension().block_stats(q, block_size, mean=True)
    if real_q_len is None or real_q_len >= q_len:
        return q_mean
    real_q_len = max(0, int(real_q_len))
    full_blocks, tail = divmod(real_q_len, block_size)
    if tail:
        rows = q[:, :, full_blocks * block_size: full_blocks * block_size + tail].float()
        q_mean[:, :, full_blocks] = (rows.sum(dim=2) / tail).to(q_mean.dtype)
        q_mean[:, :, full_blocks + 1:] = 0
    else:
        q_mean[:, :, full_blocks:] = 0
    return q_mean


def _select_block_pairs_from_cached_stats(q: torch.Tensor, layer: ThriftAttentionCacheLayer, config: AttentionConfig,
                                          real_q_len: int | None = None, is_bf16: bool = False) -> torch.Tensor:
    """Per-q-block top-k from the statistics the cache already holds (transformers_cache.py:761-831);
    ``[B * Hq, Sq/block, width]`` int32, -1 padded under the causal mask."""
    quest = config.selection == "quest"
    if (layer.k_min is None or layer.k_max is None) if quest else layer.k_mean is None:
        raise RuntimeError("ThriftAttention K block means have not been initialized")
    block_size = config.block_size
    batch, q_heads, q_len, head_dim = q.shape
    num_q_blocks = q_len // block_size
    num_kv_blocks = layer.seq_len // block_size
    selected_count = resolve_top_k(num_kv_blocks, causal=config.causal, top_k=config.top_k, fraction=config.fraction)
    if selected_count == 0:
        return torch.empty(batch * q_heads, num_q_blocks, 0, device=q.device, dtype=torch.int32)

    q_mean = _query_block_means(q, block_size, real_q_len)
    ext = get_extension()
    if block_size == PAGE:
        stats = [t[:, :, :num_kv_blocks].contiguous() for t in ((layer.k_min, layer.k_max) if quest else (layer.k_mean,))]
    else:   # statistics of wider blocks are recomputed from the 16-bit keys
        k = layer.key_view()[:, :, : num_kv_blocks * block_size].contiguous()
        mean, k_min, k_max = ext.block_stats(k, block_size, mean=not quest, minmax=quest)
        stats = [k_min, k_max] if quest else [mean]

    if num_kv_blocks > 2048:
        raise NotImplementedError("ThriftAttention currently supports at most 2048 selected KV blocks")
    sink = getattr(config, "sink_blocks", 0)
    local = getattr(config, "local_blocks", 0)
    if sink or local:
        return ext.select_prefill_blocks(q_mean, stats[0], stats[1] if quest else None, selected_count, config.causal,
                                         is_bf16, sink=sink, local=local)
    if quest:
        return ext.quest_block_topk(q_mean, stats[0], stats[1], selected_count, config.causal, is_bf16)
    return ext.block_mean_topk(q_mean, stats[0], selected_count, config.causal, is_bf16)

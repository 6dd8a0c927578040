"""Multi-GPU partitioning of the attention path (one process per GPU, ``torch.distributed``).

The reference has no distributed code; these are the two decompositions the path admits:

* prefill — KV-head groups are independent (statistics, selection, quantisation and attention of
  one KV head and its query heads never look at another group), so ranks take whole groups and
  the only collective is an optional ``all_gather`` of the outputs;
* decode — the KV sequence is split into contiguous page ranges, one per rank.  Each rank scores
  its own pages with the selection kernel (which also returns its fp32 scores), the ranks exchange their
  local top-k candidates (a global top-k element is always inside its shard's top-k), every rank derives
  the same global selection — bit-identical to the single-GPU one —, runs the split-KV kernel
  over its pages and contributes un-normalised partials ``(o, m, l)``; after an ``all_gather`` the
  log-sum-exp merge kernel produces the output on every rank.

The planning helpers are pure Python / device-agnostic tensor code so that they can be exercised
with the ``gloo`` backend on CPU; the kernels themselves need a GPU.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


class PeerExchange:
    """All-gather of small per-rank buffers by this library's own kernel over NVLink peer memory
    (``ta100_peer_all_gather``): every rank stores its rows straight into every peer's region and waits, with a
    budget, for the peers' flags - one launch per rank and exchange instead of a latency-bound library collective.

    Collective constructor (every rank of ``group`` calls it): allocates this rank's region for payloads of up to
    ``max_bytes`` per rank, exchanges the CUDA IPC handles through ``torch.distributed`` and maps the peers' regions.
    One process per GPU; the ranks' kernels wait for each other.  ``all_gather`` must be called the same number of
    times on every rank; it is a plain kernel launch and can be captured in a CUDA graph."""

    def __init__(self, max_bytes: int, group=None, device=None) -> None:
        import ctypes

        from thriftattention_b200 import _lib

        self._lib = _lib.load()
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ValueError("PeerExchange serves at most 8 ranks")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.slot_bytes = (int(max_bytes) + 15) // 16 * 16
        own = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        with torch.cuda.device(self.device):
            _lib.check(self._lib.ta100_peer_exchange_create(self.world, self.slot_bytes, ctypes.byref(own), handle),
                       "peer_exchange_create")
        self._own = own
        mine = torch.frombuffer(bytearray(handle.raw), dtype=torch.uint8).to(self.device)
        handles = torch.empty(self.world, 64, dtype=torch.uint8, device=self.device)
        dist.all_gather_into_tensor(handles.view(-1), mine, group=group)
        handles = handles.cpu()
        self._opened: list = []
        regions = (ctypes.c_void_p * self.world)()
        for r in range(self.world):
            if r == self.rank:
                regions[r] = own.value
                continue
            ptr = ctypes.c_void_p()
            with torch.cuda.device(self.device):
                _lib.check(self._lib.ta100_peer_exchange_open(bytes(handles[r].tolist()), ctypes.byref(ptr)),
                           "peer_exchange_open")
            regions[r] = ptr.value
            self._opened.append(ptr)
        self._regions = regions
        dist.barrier(group=group)            # every region is mapped everywhere before the first store

    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        """``x`` (contiguous, CUDA, a multiple of 16 bytes, the same shape on every rank) -> ``[world, *x.shape]``."""
        import ctypes

        from thriftattention_b200 import _lib

        nbytes = x.numel() * x.element_size()
        if not (x.is_cuda and x.is_contiguous()) or nbytes % 16 or nbytes > self.slot_bytes or nbytes == 0:
            raise ValueError("PeerExchange.all_gather needs a contiguous CUDA tensor of 16..slot_bytes bytes (multiple of 16)")
        out = torch.empty((self.world, *x.shape), dtype=x.dtype, device=x.device)
        with torch.cuda.device(x.device):
            rc = self._lib.ta100_peer_all_gather(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(out.data_ptr()), nbytes,
                                                 self.slot_bytes, self.world, self.rank, self._regions,
                                                 ctypes.c_void_p(torch.cuda.current_stream(x.device).cuda_stream))
        _lib.check(rc, "peer_all_gather")
        return out

    def check(self) -> None:
        """Synchronises; raises if a wait for a peer ran out since the last check."""
        import ctypes

        from thriftattention_b200 import _lib

        with torch.cuda.device(self.device):
            rc = self._lib.ta100_peer_exchange_status(self._own, self.world, self.slot_bytes,
                                                      ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream))
        _lib.check(rc, "peer_all_gather (device)")

    def close(self) -> None:
        """Collective: unmaps the peers' regions and frees this rank's (after every rank is done with them)."""
        if self._own is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        with torch.cuda.device(self.device):
            for ptr in self._opened:
                self._lib.ta100_peer_exchange_close(ptr)
            dist.barrier(group=self.group)
            self._lib.ta100_peer_exchange_destroy(self._own)
        self._own, self._opened = None, []


def _all_gather_stack(x: torch.Tensor, group=None, exchange: "PeerExchange | None" = None) -> torch.Tensor:
    """``all_gather`` of equally shaped tensors, stacked on a new leading rank dimension (through ``exchange``'s
    peer-memory kernel when one is given and the tensor fits it, else the process group's collective)."""
    if exchange is not None and x.is_cuda and x.is_contiguous():
        nbytes = x.numel() * x.element_size()
        if 0 < nbytes <= exchange.slot_bytes and nbytes % 16 == 0:
            return exchange.all_gather(x)
    world = dist.get_world_size(group)
    x = x.contiguous()
    flat = torch.empty((world * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(flat, x, group=group)
    return flat.view((world,) + tuple(x.shape))


# --------------------------------------------------------------------------------------------- prefill
@dataclass(frozen=True)
class HeadShard:
    """Heads owned by one rank: KV heads [kv_begin, kv_end) and their query heads."""

    rank: int
    world: int
    kv_begin: int
    kv_end: int
    q_begin: int
    q_end: int


def plan_head_shards(num_q_heads: int, num_kv_heads: int, world: int) -> list[HeadShard]:
    """Contiguous, balanced split of the KV-head groups over ``world`` ranks."""
    if num_q_heads % num_kv_heads:
        raise ValueError("q heads must be divisible by KV heads")
    if world < 1 or num_kv_heads % world:
        raise ValueError(f"the number of ranks ({world}) must divide the number of KV heads ({num_kv_heads})")
    group = num_q_heads // num_kv_heads
    per = num_kv_heads // world
    return [HeadShard(r, world, r * per, (r + 1) * per, r * per * group, (r + 1) * per * group) for r in range(world)]


def shard_heads(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, shard: HeadShard):
    """Slices of full ``[B,H,S,D]`` tensors owned by ``shard`` (views, no copy)."""
    return (q[:, shard.q_begin:shard.q_end], k[:, shard.kv_begin:shard.kv_end], v[:, shard.kv_begin:shard.kv_end])


def gather_heads(local_out: torch.Tensor, group=None) -> torch.Tensor:
    """``all_gather`` of per-rank outputs ``[B, Hq/N, S, D]`` into ``[B, Hq, S, D]`` (rank order = head order)."""
    world = dist.get_world_size(group)
    if world == 1:
        return local_out
    buf = _all_gather_stack(local_out, group)
    b, h, s, d = local_out.shape
    return buf.permute(1, 0, 2, 3, 4).reshape(b, world * h, s, d)


def attention_head_sharded(q, k, v, *, config=None, group=None, gather: bool = True):
    """``attention`` on this rank's KV-head groups of replicated (or pre-sliced) inputs.

    ``q, k, v`` are the FULL tensors; each rank computes its slice.  With ``gather`` the full
    output is returned on every rank, otherwise the local slice.
    """
    from thriftattention_b200.functional import attention

    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    shard = plan_head_shards(q.shape[1], k.shape[1], world)[rank]
    ql, kl, vl = shard_heads(q, k, v, shard)
    out = attention(ql.contiguous(), kl.contiguous(), vl.contiguous(), config=config)
    return gather_heads(out, group) if (gather and world > 1) else out


# --------------------------------------------------------------------------------------------- decode
@dataclass(frozen=True)
class PageShard:
    """Pages (64-token blocks) of every sequence owned by one rank: [page_begin, page_end)."""

    rank: int
    world: int
    page_begin: int
    page_end: int

    @property
    def num_pages(self) -> int:
        return self.page_end - self.page_begin


def _shard_page_begin(r: int, world: int, num_pages: int) -> int:
    """Start of shard ``r``: the even split ``r * n / N`` with every inner boundary moved to the nearest multiple of
    32 pages (the rule of ``merge_page_candidates``).  The selection kernel orders exact ties by (bit-reversed page
    mod 32, page div 32) of its LOCAL page ids; a shard start that is a multiple of 32 makes that the order of the
    global ids, so a tie at a shard's own cut is resolved as the single-GPU kernel resolves it."""
    if r <= 0:
        return 0
    if r >= world:
        return num_pages
    return min((r * num_pages // world + 16) // 32 * 32, num_pages)


def plan_page_shards(num_pages: int, world: int) -> list[PageShard]:
    """Contiguous split of ``num_pages`` pages with shard starts at multiples of 32 pages (see
    ``_shard_page_begin``).  With fewer than about 32 pages per rank some shards are empty; they take part in the
    exchanges with no candidates and a neutral partial."""
    if world < 1:
        raise ValueError("world must be positive")
    return [PageShard(r, world, _shard_page_begin(r, world, num_pages), _shard_page_begin(r + 1, world, num_pages))
            for r in range(world)]


def _max_shard_pages(total_pages: int, world: int) -> int:
    return max(s.num_pages for s in plan_page_shards(total_pages, world))


def _bitrev5(x: torch.Tensor) -> torch.Tensor:
    r = torch.zeros_like(x)
    for i in range(5):
        r |= ((x >> i) & 1) << (4 - i)
    return r


def merge_topk_candidates(scores: torch.Tensor, pages: torch.Tensor, k: int) -> torch.Tensor:
    """Global top-k from gathered per-shard candidates.

    ``scores`` / ``pages``: ``[rows, n_candidates]`` (fp32 scores, global page ids, -1 for padding).
    Returns int32 ``[rows, k]`` in rank order.  Ties are broken the way the selection kernel breaks
    them on a single GPU: smallest 5-bit bit-reversal of ``page mod 32``, then smallest ``page div 32``
    — so every rank derives the same list, equal to the single-GPU result.
    """
    valid = pages >= 0
    s = torch.where(valid, scores, torch.full_like(scores, float("-inf")))
    pg = pages.to(torch.int64)
    tie = _bitrev5(pg & 31) * 65536 + (pg >> 5)
    # sort by (score desc, tie asc): stable sort on the secondary key first, then on the primary
    order = torch.argsort(tie, dim=1, stable=True)
    s_sorted = torch.gather(s, 1, order)
    order2 = torch.argsort(s_sorted, dim=1, descending=True, stable=True)
    final = torch.gather(order, 1, order2)[:, :k]
    out = torch.gather(pages, 1, final).to(torch.int32)
    ok = torch.gather(valid, 1, final)
    return torch.where(ok, out, torch.full_like(out, -1))


def exchange_candidates(local_scores: torch.Tensor, local_pages: torch.Tensor, group=None):
    """``all_gather`` of per-rank candidate lists ``[rows, c]`` -> ``[rows, world*c]`` (scores, pages)."""
    world = dist.get_world_size(group)
    if world == 1:
        return local_scores, local_pages
    s_buf = _all_gather_stack(local_scores, group)
    p_buf = _all_gather_stack(local_pages, group)
    rows = local_scores.shape[0]
    return s_buf.permute(1, 0, 2).reshape(rows, -1), p_buf.permute(1, 0, 2).reshape(rows, -1)


def exchange_partials(part_o: torch.Tensor, part_ml: torch.Tensor, group=None):
    """``all_gather`` of decode partials -> ``[world, heads, splits, G, D]`` and ``[world, heads, splits, G, 2]``."""
    world = dist.get_world_size(group)
    if world == 1:
        return part_o.unsqueeze(0), part_ml.unsqueeze(0)
    return _all_gather_stack(part_o, group), _all_gather_stack(part_ml, group)


def select_pages_sharded(q_grouped, k_a, k_b, *, shard: PageShard, total_pages: int, top_k: int, sink: int = 0,
                         local: int = 0, group=None, exchange: "PeerExchange | None" = None) -> torch.Tensor:
    """Global page selection when every rank holds the statistics of its own pages only.

    ``k_a`` / ``k_b`` ``[B, Hkv, shard.num_pages(+), D]``: block means (``k_b is None``) or Quest minima / maxima
    of the LOCAL pages.  Each rank runs the selection kernel on its pages — forcing the sink pages that fall at
    the start of its range and the recent pages that fall at its end — and receives the kernel's own fp32
    scores; the ranks exchange their top-k candidates and merge them with the kernel's tie-break, so the result
    equals the single-GPU selection bit for bit.  Returns int32 ``[B*Hkv, sink + local + top_k]`` LOCAL page ids
    of this rank's share (forced pages first), -1 elsewhere.
    """
    from thriftattention_b200._extension import get_extension

    ext = get_extension()
    n_local = shard.num_pages
    rows = q_grouped.shape[0] * q_grouped.shape[1]
    dev = q_grouped.device
    n_sink = min(sink, total_pages)
    local_lo = max(total_pages - local, n_sink)
    my_sink = max(0, min(n_sink, shard.page_end) - shard.page_begin)             # forced at the start of my range
    my_local = max(0, shard.page_end - max(local_lo, shard.page_begin))          # forced at its end
    k_glob = min(top_k, max(total_pages - n_sink - (total_pages - local_lo), 0))
    cand = min(k_glob, max(n_local - my_sink - my_local, 0))
    world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
    # every rank sends a list of the same width: forced pages + candidates, padded
    send_width = min(n_sink, _max_shard_pages(total_pages, shard.world)) + \
        min(total_pages - local_lo, _max_shard_pages(total_pages, shard.world)) + \
        min(k_glob, _max_shard_pages(total_pages, shard.world))
    if shard.page_begin % 32 and shard.num_pages:
        raise ValueError("a KV-sequence shard must start at a multiple of 32 pages (use plan_page_shards)")
    if q_grouped.is_cuda and world * send_width <= 2048:
        # one buffer, one all-gather, one merge kernel
        buf = torch.empty(2, rows, send_width, dtype=torch.int32, device=dev)
        if n_local == 0:
            buf[0].fill_(-1)                                            # an empty shard: no candidates
            buf[1].view(torch.float32).fill_(-torch.finfo(torch.float32).max)
        else:
            ext.select_decode_blocks(q_grouped, k_a, k_b, cand, n_local, q_grouped.dtype == torch.bfloat16, sink=my_sink,
                                     local=my_local, out=buf[0], return_scores=True,
                                     scores_out=buf[1].view(torch.float32), row_width=send_width)
        gathered = _all_gather_stack(buf, group, exchange) if world > 1 else buf.unsqueeze(0)
        return ext.merge_page_candidates(gathered.contiguous(), rank=shard.rank, total_pages=total_pages, top_k=top_k,
                                         sink=sink, local=local)
    if n_local == 0:
        sel = torch.full((rows, 0), -1, dtype=torch.int32, device=dev)
        scores = torch.zeros(rows, 0, dtype=torch.float32, device=dev)
    else:
        sel, scores = ext.select_decode_blocks(q_grouped, k_a, k_b, cand, n_local, q_grouped.dtype == torch.bfloat16,
                                               sink=my_sink, local=my_local, return_scores=True)
    forced = sel[:, : my_sink + my_local]
    c_pages = sel[:, my_sink + my_local: my_sink + my_local + cand]
    c_scores = scores[:, my_sink + my_local: my_sink + my_local + cand]
    # fixed-width candidate lists (k_glob per rank) for the exchange
    pad_p = torch.full((rows, k_glob), -1, dtype=torch.int32, device=dev)
    pad_s = torch.full((rows, k_glob), float("-inf"), dtype=torch.float32, device=dev)
    if cand:
        pad_p[:, :cand] = torch.where(c_pages >= 0, c_pages + shard.page_begin, c_pages)
        pad_s[:, :cand] = torch.where(c_pages >= 0, c_scores, torch.full_like(c_scores, float("-inf")))
    all_s, all_p = exchange_candidates(pad_s, pad_p, group)
    global_sel = merge_topk_candidates(all_s, all_p, k_glob) if k_glob else pad_p
    mine = (global_sel >= shard.page_begin) & (global_sel < shard.page_end)
    local_topk = torch.where(mine, global_sel - shard.page_begin, torch.full_like(global_sel, -1))
    out = torch.full((rows, sink + local + top_k), -1, dtype=torch.int32, device=dev)
    out[:, : my_sink + my_local] = forced
    out[:, sink + local: sink + local + k_glob] = local_topk
    return out.contiguous()


def decode_kv_sharded(q, k_local, v_local, *, shard: PageShard, total_pages: int, top_k: int, quant_format="nvfp4",
                      num_splits: int = 0, group=None, selection: str = "quest", sink_blocks: int = 0,
                      local_blocks: int = 0, exchange: "PeerExchange | None" = None):
    """One decode step with the KV sequence sharded over ranks.

    ``q`` ``[B, Hq, 1, D]`` replicated; ``k_local`` / ``v_local`` ``[B, Hkv, shard.num_pages*64, D]`` are this
    rank's slice of the cache.  Selection of ``top_k`` pages (+ forced sink / recent pages) over the WHOLE
    sequence, mixed attention over the local pages, LSE merge across ranks.  Returns ``[B, Hq, 1, D]`` on
    every rank, equal to the single-GPU result up to the split-dependent fp32 rounding of the merge.
    """
    from thriftattention_b200._extension import get_extension

    ext = get_extension()
    is_bf16 = q.dtype == torch.bfloat16
    is_mx = quant_format == "mxfp4"
    b, hq, _, d = q.shape
    hkv = k_local.shape[1]
    q_grouped = q.reshape(b, hkv, hq // hkv, d).contiguous()
    k_local, v_local = k_local.contiguous(), v_local.contiguous()
    # 1. local page statistics, 2. kernel-scored candidates + exchange, 3. identical global selection everywhere
    empty = shard.num_pages == 0
    if empty:
        k_a = k_b = None
    elif selection == "quest":
        _, k_a, k_b = ext.block_stats(k_local, 64, minmax=True)
    else:
        k_a, _, _ = ext.block_stats(k_local, 64, mean=True)
        k_b = None
    local_sel = select_pages_sharded(q_grouped, k_a, k_b, shard=shard, total_pages=total_pages, top_k=top_k,
                                     sink=sink_blocks, local=local_blocks, group=group, exchange=exchange)
    # 4. local split-KV attention -> partials, 5. exchange + merge
    run_decode = None                    # an empty shard contributes a neutral partial
    if not empty:
        quant = getattr(ext, f"{quant_format}_quantize")
        quant_t = getattr(ext, f"{quant_format}_quantize_transposed")
        q4, qs = quant(q_grouped, is_bf16)
        k4, ks = quant(k_local, is_bf16)
        v4, vs = quant_t(v_local, is_bf16)
        run_decode = lambda **kw: ext.decode_attention(q_grouped, k_local, v_local, local_sel, q4, k4, v4, qs, ks, vs,  # noqa: E731
                                                       is_mx=is_mx, is_bf16=is_bf16, allow_padded_selection=True, **kw)
    out = decode_partials_exchange_merge(
        run_decode,
        heads=b * hkv, group_size=hq // hkv, head_dim=d, shard=shard, total_pages=total_pages, num_splits=num_splits,
        is_mx=is_mx, is_bf16=is_bf16, device=q.device, group=group, exchange=exchange)
    return out.reshape(b, hq, 1, d)


def decode_partials_exchange_merge(run_decode, *, heads: int, group_size: int, head_dim: int, shard: PageShard,
                                   total_pages: int, num_splits: int, is_mx: bool, is_bf16: bool, device, group=None,
                                   exchange: "PeerExchange | None" = None):
    """Local split-KV attention, the rank's chains reduced to one partial per head, ONE ``all_gather`` of that
    buffer, LSE merge on every rank.

    ``run_decode(num_splits=, return_partials=True)`` launches the local decode kernel and returns
    ``(out, part_o, part_ml)``; every rank may use its own chain count.  ``run_decode=None`` (a rank without pages)
    contributes the neutral partial o = 0, m = -FLT_MAX, l = 0.  Returns ``[heads, group_size, head_dim]``."""
    from thriftattention_b200._extension import get_extension

    ext = get_extension()
    world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
    # this rank's chains are reduced to one partial per head first: the exchange then carries
    # heads x G x (D + 2) floats per rank whatever the chain count
    n_o, n_ml = heads * group_size * head_dim, heads * group_size * 2
    flat = torch.empty(n_o + n_ml, dtype=torch.float32, device=device)
    mine_o = flat[:n_o].view(heads, 1, group_size, head_dim)
    mine_ml = flat[n_o:].view(heads, 1, group_size, 2)
    if run_decode is None:
        flat.zero_()
        mine_ml[..., 0] = -torch.finfo(torch.float32).max
    else:
        _, part_o, part_ml = run_decode(num_splits=num_splits, return_partials=True)
        ext.reduce_decode_partials(part_o, part_ml, out=(mine_o, mine_ml))
    gathered = _all_gather_stack(flat, group, exchange) if world > 1 else flat.unsqueeze(0)   # [world, n_o + n_ml]
    all_o = gathered[:, :n_o].view(world, heads, 1, group_size, head_dim)
    all_ml = gathered[:, n_o:].view(world, heads, 1, group_size, 2)
    return ext.merge_decode_partials(all_o, all_ml, is_mx=is_mx, is_bf16=is_bf16)

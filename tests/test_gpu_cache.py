"""GPU tests of the generation cache: the fused append kernel is bit-exact against the CPU oracle's
quantisers and block statistics however the sequence is cut into appends; crop re-zeroes the rounded
tail; decode and prefill over the cache match the oracle's attention on the same (zero-padded) K/V."""
import pytest
import torch

import oracle
import thriftattention_b200 as ta
from thriftattention_b200.integrations import transformers_cache as tc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _u8(t):
    return t.view(torch.uint8).cpu()


def _check_layer_against_oracle(layer, k_ref, v_ref, fmt):
    """Every derived tensor of ``layer`` equals the oracle's function of its 16-bit content ``k_ref`` / ``v_ref``
    ([B,H,n,D] CPU tensors, n = layer.seq_len)."""
    n = layer.seq_len
    g = 32 if fmt == "mxfp4" else 16
    assert torch.equal(layer.key_view().cpu(), k_ref) and torch.equal(layer.value_view().cpu(), v_ref)
    k_packed, v_packed_t, k_scale, v_scale_t = layer.packed_views()      # strided views of a slab layer, gathers of a paged one
    codes, scales = oracle.quantize(k_ref, fmt, "plain")
    assert torch.equal(k_packed[:, :, :n].cpu(), codes)
    assert torch.equal(_u8(k_scale[:, :, :n]), _u8(scales))
    # V groups: tokens beyond n inside the last group are zero rows of the cache
    ng = -(-n // g) * g
    v_pad = torch.zeros(v_ref.shape[0], v_ref.shape[1], ng, v_ref.shape[3], dtype=v_ref.dtype)
    v_pad[:, :, :n] = v_ref
    vcodes, vscales = oracle.quantize(v_pad, fmt, "transposed")
    assert torch.equal(v_packed_t[:, :, :, : ng // 2].cpu(), vcodes[:, :, :, : ng // 2])
    assert torch.equal(_u8(v_scale_t[:, :, :, : ng // g]), _u8(vscales[:, :, :, : ng // g]))
    # ... and the rest of the rounded views are zero rows
    assert k_packed[:, :, n:].sum() == 0 and v_packed_t[:, :, :, ng // 2:].sum() == 0
    nb = n // 64
    if nb:
        mean, lo, hi = oracle.block_stats(k_ref[:, :, : nb * 64], 64)
        assert torch.equal(layer.k_mean[:, :, :nb].cpu(), mean)
        if layer.k_min is not None:
            assert torch.equal(layer.k_min[:, :, :nb].cpu(), lo) and torch.equal(layer.k_max[:, :, :nb].cpu(), hi)


@pytest.mark.parametrize("paged", [False, True])
@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("d", [128, 64])
def test_append_any_chunking_is_bit_exact(fmt, dtype, d, paged):
    torch.manual_seed(5)
    total = 700
    k = (torch.randn(2, 3, total, d) * 1.5).to(dtype)
    v = torch.randn(2, 3, total, d).to(dtype)
    k[0, 0, 100:116] = 0                      # an all-zero group -> scale byte 0, codes 0
    v[1, 2, 32:64, 5] = 0
    k[0, 1, 7, :16] = 5000.0                  # beyond 448 * 6: the scale saturates
    for chunks in ([700], [1] * 40 + [660], [70, 1, 1, 57, 3, 200, 33, 31, 1, 303], [64, 64, 128, 444]):
        kind = tc.PagedThriftAttentionCacheLayer if paged else tc.ThriftAttentionCacheLayer
        layer = kind(quant_format=fmt, track_minmax=True)
        pos = 0
        for c in chunks:
            layer.update(k[:, :, pos:pos + c].to(DEV), v[:, :, pos:pos + c].to(DEV))
            pos += c
            if c > 1 or pos % 16 == 0:
                _check_layer_against_oracle(layer, k[:, :, :pos], v[:, :, :pos], fmt)
        assert pos == total and layer.capacity in ((704,) if paged else (768, 1024))
        _check_layer_against_oracle(layer, k, v, fmt)
        if paged:
            # every sequence has its own 11 pages, none of them the zero page, and the table says so
            table = layer.page_table.cpu()
            used = table[:, :11].flatten().tolist()
            assert len(set(used)) == 22 and min(used) >= 1 and bool((table[:, 11:] == -1).all())


def test_append_with_fixed_capacity_and_positions():
    torch.manual_seed(6)
    k = torch.randn(1, 2, 200, 128).half()
    v = torch.randn(1, 2, 200, 128).half()
    layer = tc.ThriftAttentionCacheLayer(max_cache_len=200)
    layer.update(k[:, :, :150].to(DEV), v[:, :, :150].to(DEV), {"cache_position": torch.arange(150, device=DEV)})
    assert layer.capacity == 256
    # overwrite a range in the middle, then continue at the end
    k2, v2 = k.clone(), v.clone()
    k2[:, :, 60:90] = torch.randn(1, 2, 30, 128).half()
    v2[:, :, 60:90] = torch.randn(1, 2, 30, 128).half()
    layer.update(k2[:, :, 60:90].to(DEV), v2[:, :, 60:90].to(DEV), {"cache_position": torch.arange(60, 90)})
    assert layer.seq_len == 150
    layer.update(k2[:, :, 150:].to(DEV), v2[:, :, 150:].to(DEV))
    n = layer.seq_len
    assert n == 200
    codes, scales = oracle.quantize(k2, "nvfp4", "plain")
    assert torch.equal(layer.k_packed[:, :, :n].cpu(), codes) and torch.equal(_u8(layer.k_scale[:, :, :n]), _u8(scales))
    v_pad = torch.zeros(1, 2, 208, 128).half()
    v_pad[:, :, :200] = v2
    vcodes, _ = oracle.quantize(v_pad, "nvfp4", "transposed")
    assert torch.equal(layer.v_packed_t[:, :, :, :104].cpu(), vcodes[:, :, :, :104])
    # statistics are refreshed for the blocks that END inside the written range: block 0 here
    # (tokens 60..63 changed); block 1 keeps its old statistics although tokens 64..89 changed
    mean = oracle.block_stats(k2[:, :, :64], 64, ("mean",))[0]
    assert torch.equal(layer.k_mean[:, :, :1].cpu(), mean)


def test_crop_rezeroes_tail_and_requantises():
    torch.manual_seed(7)
    k = torch.randn(1, 2, 128, 128).half()
    v = torch.randn(1, 2, 128, 128).half()
    layer = tc.ThriftAttentionCacheLayer()
    layer.update(k.to(DEV), v.to(DEV))
    layer.crop(70)
    assert layer.seq_len == 70
    assert layer.k_fp16[:, :, 70:128].abs().sum() == 0 and layer.v_fp16[:, :, 70:128].abs().sum() == 0
    assert layer.k_packed[:, :, 70:128].sum() == 0 and _u8(layer.k_scale[:, :, 70:128]).sum() == 0
    _check_layer_against_oracle(layer, k[:, :, :70], v[:, :, :70], "nvfp4")
    assert layer.v_packed_t[:, :, :, 40:64].sum() == 0           # groups entirely beyond token 80
    # decode continues from the cropped length
    layer.update(k[:, :, 100:101].to(DEV), v[:, :, 100:101].to(DEV))
    k3 = torch.cat([k[:, :, :70], k[:, :, 100:101]], 2)
    v3 = torch.cat([v[:, :, :70], v[:, :, 100:101]], 2)
    _check_layer_against_oracle(layer, k3, v3, "nvfp4")


def test_cache_append_argument_errors():
    ext = ta._extension.get_extension()
    layer = tc.ThriftAttentionCacheLayer()
    layer.update(torch.zeros(1, 1, 10, 128, device=DEV).half(), torch.zeros(1, 1, 10, 128, device=DEV).half())
    args = (layer.k_fp16, layer.v_fp16, layer.k_packed, layer.k_scale, layer.v_packed_t, layer.v_scale_t)
    new = torch.zeros(1, 1, 200, 128, device=DEV).half()
    with pytest.raises(RuntimeError, match="cache_append"):
        ext.cache_append(new, new, *args, start=0)                # 200 rows into a 128-row cache
    with pytest.raises(RuntimeError):
        ext.cache_append(new[:, :, :4].bfloat16(), new[:, :, :4].bfloat16(), *args, start=0)
    with pytest.raises(RuntimeError):
        ext.cache_append(new[:, :, :4], new[:, :, :4], *args, start=0, k_mean=torch.zeros(1, 1, 1, 128, device=DEV).half())


# ------------------------------------------------------------------------------- attention over the cache
def _filled_cache(cfg, k, v, chunks):
    cache = ta.ThriftAttentionCache(config=cfg)
    pos = 0
    for c in chunks:
        cache.update(k[:, :, pos:pos + c].to(DEV), v[:, :, pos:pos + c].to(DEV), 0)
        pos += c
    return cache


def _zero_padded(x, multiple=64):
    n = x.shape[2]
    p = max(multiple, -(-n // multiple) * multiple)
    out = torch.zeros(x.shape[0], x.shape[1], p, x.shape[3], dtype=x.dtype)
    out[:, :, :n] = x
    return out


@pytest.mark.parametrize("fmt,selection,dtype", [("nvfp4", "block_mean", torch.float16), ("nvfp4", "quest", torch.bfloat16),
                                                 ("mxfp4", "quest", torch.float16), ("nvfp4", "local", torch.float16)])
def test_cached_decode_matches_oracle(fmt, selection, dtype):
    torch.manual_seed(11)
    b, hq, hkv, n, d = 2, 8, 2, 64 * 9 + 17, 128
    k = torch.randn(b, hkv, n, d).to(dtype)
    v = torch.randn(b, hkv, n, d).to(dtype)
    q = torch.randn(b, hq, 1, d).to(dtype)
    cfg = ta.AttentionConfig(selection=selection, top_k=3, quant_format=fmt)
    cache = _filled_cache(cfg, k, v, [500, 1, 1, n - 502])
    out = tc.cached_decode_attention(q.to(DEV), cache, 0, cfg)
    assert out.shape == (b, hq, 1, d) and out.dtype == dtype

    # oracle: same K/V, zero rows up to the next multiple of 64; only the 9 complete blocks are candidates
    kp, vp = _zero_padded(k), _zero_padded(v)
    qg = q.reshape(b, hkv, hq // hkv, d)
    if selection == "local":
        sel = oracle.local_decode(b * hkv, 9, 3)
    else:
        mean, lo, hi = oracle.block_stats(kp, 64)
        sel = (oracle.select_decode(qg, lo, hi, k=3, num_kv_blocks=9) if selection == "quest"
               else oracle.select_decode(qg, mean, k=3, num_kv_blocks=9))
    got_sel = tc.select_cached_decode_blocks(qg.to(DEV), cache.layers[0], cfg).cpu()
    assert torch.equal(got_sel, sel)
    splits = ta._extension.get_extension().decode_pick_splits(b * hkv, 10)
    ref = oracle.decode_attention(qg, kp, vp, sel, fmt=fmt, splits=min(splits, 10)).reshape(b, hq, 1, d)
    err = (out.float().cpu() - ref.float()).abs()
    tol = 2e-3 if dtype == torch.float16 else max(2e-3, 2.0 ** -7 * ref.float().abs().max().item())
    assert err.max().item() <= tol, err.max().item()

    # pure FP4 over the same cache
    cfg4 = ta.AttentionConfig(method="fp4", quant_format=fmt)
    out4 = tc.cached_decode_attention(q.to(DEV), cache, 0, cfg4)
    ref4 = oracle.decode_attention(qg, kp, vp, None, fmt=fmt, splits=min(splits, 10)).reshape(b, hq, 1, d)
    assert (out4.float().cpu() - ref4.float()).abs().max().item() <= tol


@pytest.mark.parametrize("fmt,selection,block", [("nvfp4", "block_mean", 64), ("mxfp4", "quest", 64), ("nvfp4", "quest", 128)])
def test_cached_prefill_matches_oracle(fmt, selection, block):
    torch.manual_seed(12)
    b, hq, hkv, n, d = 1, 4, 2, 512, 128
    q = torch.randn(b, hq, n, d).half()
    k = torch.randn(b, hkv, n, d).half()
    v = torch.randn(b, hkv, n, d).half()
    cfg = ta.AttentionConfig(selection=selection, top_k=2, quant_format=fmt, block_size=block)
    cache = ta.ThriftAttentionCache(config=cfg, max_cache_len=n + 100)      # capacity 640 > n: strided views
    cache.update(k.to(DEV), v.to(DEV), 0)
    assert cache.layers[0].capacity == 640
    out = tc.cached_prefill_attention(q.to(DEV), cache, 0, cfg)
    qm, = oracle.block_stats(q, block, ("mean",))
    mean, lo, hi = oracle.block_stats(k, block)
    sel = (oracle.select_prefill(qm, lo, hi, k=2, causal=True) if selection == "quest"
           else oracle.select_prefill(qm, mean, k=2, causal=True))
    ref = oracle.prefill_attention(q, k, v, sel, fmt=fmt, block=block, causal=True)
    err = (out.float().cpu() - ref.float()).abs()
    assert err.max().item() <= 2e-3 and err.mean().item() <= 2e-4, (err.max().item(), err.mean().item())
    # the route without a cache (K/V quantised again, K in the permuted layout) agrees
    again = ta.attention(q.to(DEV), k.to(DEV), v.to(DEV), config=cfg)
    assert (again.float() - out.float()).abs().max().item() <= 1e-3


def test_cached_prefill_ignores_prompt_padding_in_selection():
    torch.manual_seed(13)
    n, real = 256, 150
    q = torch.randn(1, 2, n, 128).half()
    k = torch.randn(1, 2, n, 128).half()
    v = torch.randn(1, 2, n, 128).half()
    cfg = ta.AttentionConfig(top_k=1)
    cache = ta.ThriftAttentionCache(config=cfg)
    cache.prefill_real_seq_len = real
    cache.update(k.to(DEV), v.to(DEV), 0)
    sel = tc.select_cached_prefill_blocks(q.to(DEV), cache.layers[0].key_view(), cache.layers[0], cfg, real_q_len=real).cpu()
    qm, = oracle.block_stats(q, 64, ("mean",))
    qm[:, :, 2] = (q[:, :, 128:150].float().sum(2) / 22).half()
    qm[:, :, 3] = 0
    mean, = oracle.block_stats(k, 64, ("mean",))
    ref = oracle.select_prefill(qm, mean, k=1, causal=True)
    assert torch.equal(sel[:, :2], ref[:, :2])          # blocks made only of real rows: identical arithmetic
    assert sel.shape == ref.shape


@pytest.mark.parametrize("fmt,selection,dtype,sink,local", [("nvfp4", "block_mean", torch.float16, 0, 0),
                                                          ("mxfp4", "quest", torch.bfloat16, 1, 2),
                                                          ("nvfp4", "quest", torch.float16, 2, 0)])
def test_fused_decode_step_equals_the_operator_path(monkeypatch, fmt, selection, dtype, sink, local):
    """cached_decode_attention queues quantise q + selection + attention through one library call; with that entry
    hidden it goes operator by operator.  Both give the same bytes, over several appended tokens and a ragged
    last block."""
    from thriftattention_b200 import _C
    from thriftattention_b200.integrations import transformers_cache as tc

    torch.manual_seed(31)
    cfg = ta.AttentionConfig(selection=selection, top_k=3, quant_format=fmt, sink_blocks=sink, local_blocks=local)
    caches = [tc.ThriftAttentionCache(config=cfg, max_cache_len=1024) for _ in range(2)]
    k = torch.randn(2, 2, 700, 128, device=DEV).to(dtype)
    v = torch.randn(2, 2, 700, 128, device=DEV).to(dtype)
    for c in caches:
        c.update(k, v, 0, {"cache_position": torch.arange(700, device=DEV)})
    for step in range(3):
        q = torch.randn(2, 8, 1, 128, device=DEV).to(dtype)
        k1 = torch.randn(2, 2, 1, 128, device=DEV).to(dtype)
        v1 = torch.randn(2, 2, 1, 128, device=DEV).to(dtype)
        for c in caches:
            c.update(k1, v1, 0, {"cache_position": torch.tensor([700 + step], device=DEV)})
        fused = tc.cached_decode_attention(q, caches[0], 0, cfg)
        with monkeypatch.context() as m:
            m.delattr(_C, "cached_decode_step")
            plain = tc.cached_decode_attention(q, caches[1], 0, cfg)
        assert torch.equal(fused, plain)
        assert torch.equal(caches[0].layer(0).selected_blocks, caches[1].layer(0).selected_blocks)
    _C.decode_status(DEV)


# ------------------------------------------------------------------------------- the paged layout
def test_paged_layer_positions_crop_reset_and_batch_surgery():
    """Overwrites by position, crop (pages go back to the free list as zeros), decode after a crop, reset, and the
    beam / batch operations (a selected sequence becomes a copy on pages of its own)."""
    torch.manual_seed(21)
    k = torch.randn(2, 2, 300, 128).half()
    v = torch.randn(2, 2, 300, 128).half()
    layer = tc.PagedThriftAttentionCacheLayer(max_cache_len=320, track_minmax=True)
    layer.update(k[:, :, :150].to(DEV), v[:, :, :150].to(DEV), {"cache_position": torch.arange(150, device=DEV)})
    pool_pages = layer.k_pool.shape[0]
    assert pool_pages == 1 + 2 * 5 and layer.page_table.shape == (2, 5)
    k2, v2 = k.clone(), v.clone()
    k2[:, :, 60:90] = torch.randn(2, 2, 30, 128).half()
    v2[:, :, 60:90] = torch.randn(2, 2, 30, 128).half()
    layer.update(k2[:, :, 60:90].to(DEV), v2[:, :, 60:90].to(DEV), {"cache_position": torch.arange(60, 90)})
    layer.update(k2[:, :, 150:].to(DEV), v2[:, :, 150:].to(DEV))
    assert layer.seq_len == 300 and layer.k_pool.shape[0] == pool_pages          # grown by page ids, not by copying
    n = layer.seq_len
    kp, vp, ks, _ = layer.packed_views()
    codes, scales = oracle.quantize(k2, "nvfp4", "plain")
    assert torch.equal(kp[:, :, :n].cpu(), codes) and torch.equal(_u8(ks[:, :, :n]), _u8(scales))
    v_pad = torch.zeros(2, 2, 304, 128).half()
    v_pad[:, :, :300] = v2
    assert torch.equal(vp[:, :, :, :152].cpu(), oracle.quantize(v_pad, "nvfp4", "transposed")[0][:, :, :, :152])

    layer.crop(70)
    assert layer.seq_len == 70 and len(layer._free) == 10 - 2 * 2
    _check_layer_against_oracle(layer, k2[:, :, :70], v2[:, :, :70], "nvfp4")
    free = torch.tensor(layer._free, device=DEV)
    assert all(_u8(pool[free]).sum() == 0 for pool in layer._pools())               # released pages hold zeros
    layer.update(k2[:, :, 100:101].to(DEV), v2[:, :, 100:101].to(DEV))
    k3 = torch.cat([k2[:, :, :70], k2[:, :, 100:101]], 2)
    v3 = torch.cat([v2[:, :, :70], v2[:, :, 100:101]], 2)
    _check_layer_against_oracle(layer, k3, v3, "nvfp4")

    layer.batch_repeat_interleave(2)                                                 # [s0, s0, s1, s1]
    assert layer.batch_size() == 4
    _check_layer_against_oracle(layer, k3.repeat_interleave(2, 0), v3.repeat_interleave(2, 0), "nvfp4")
    used = layer.page_table[:, :2].flatten().tolist()
    assert len(set(used)) == 8                                                       # no page is shared
    layer.reorder(torch.tensor([3, 0]))
    _check_layer_against_oracle(layer, k3[[1, 0]], v3[[1, 0]], "nvfp4")
    layer.update(k2[[1, 0], :, 200:203].to(DEV), v2[[1, 0], :, 200:203].to(DEV))   # the copies grow on their own pages
    _check_layer_against_oracle(layer, torch.cat([k3[[1, 0]], k2[[1, 0], :, 200:203]], 2),
                                torch.cat([v3[[1, 0]], v2[[1, 0], :, 200:203]], 2), "nvfp4")
    layer.reset()
    assert layer.seq_len == 0 and sorted(layer._free) == list(range(1, layer.k_pool.shape[0]))
    layer.update(k[:, :, :10].to(DEV), v[:, :, :10].to(DEV))
    _check_layer_against_oracle(layer, k[:, :, :10], v[:, :, :10], "nvfp4")


def test_paged_layer_without_a_length_bound_grows_its_pool():
    torch.manual_seed(22)
    k = torch.randn(1, 2, 1000, 64).to(torch.bfloat16)
    v = torch.randn(1, 2, 1000, 64).to(torch.bfloat16)
    layer = tc.PagedThriftAttentionCacheLayer(quant_format="mxfp4")
    pos = 0
    for c in (10, 200, 1, 789):
        layer.update(k[:, :, pos:pos + c].to(DEV), v[:, :, pos:pos + c].to(DEV))
        pos += c
    assert layer.k_pool.shape[0] >= 17 and layer.page_table.shape[1] >= 16
    _check_layer_against_oracle(layer, k, v, "mxfp4")


@pytest.mark.parametrize("fmt,selection,dtype", [("nvfp4", "block_mean", torch.float16), ("mxfp4", "quest", torch.bfloat16)])
def test_paged_cache_decode_and_prefill_equal_the_slab_cache(fmt, selection, dtype):
    """Same appends into a slab cache and a paged cache: the decode step (which reads the pools through the page
    table) and the prefill over the cache return the same bytes."""
    torch.manual_seed(23)
    b, hq, hkv, n, d = 2, 8, 2, 64 * 9 + 17, 128
    k = torch.randn(b, hkv, n, d).to(dtype)
    v = torch.randn(b, hkv, n, d).to(dtype)
    cfg = ta.AttentionConfig(selection=selection, top_k=3, quant_format=fmt, sink_blocks=1, local_blocks=1)
    caches = [ta.ThriftAttentionCache(config=cfg, paged=paged) for paged in (False, True)]
    for cache in caches:
        pos = 0
        for c in (500, 1, 1, n - 502):
            cache.update(k[:, :, pos:pos + c].to(DEV), v[:, :, pos:pos + c].to(DEV), 0)
            pos += c
    assert isinstance(caches[1].layers[0], tc.PagedThriftAttentionCacheLayer)
    q = torch.randn(b, hq, 1, d).to(dtype).to(DEV)
    outs = [tc.cached_decode_attention(q, cache, 0, cfg) for cache in caches]
    assert torch.equal(outs[0], outs[1])
    cfg4 = ta.AttentionConfig(method="fp4", quant_format=fmt)
    outs = [tc.cached_decode_attention(q, cache, 0, cfg4) for cache in caches]
    assert torch.equal(outs[0], outs[1])
    ta._extension.get_extension().decode_status(DEV)

    qp = torch.randn(b, hq, 64 * 10, d).to(dtype).to(DEV)
    pre = []
    for cache in caches:
        cache.crop(0)
        cache.update(k[:, :, :640].to(DEV), v[:, :, :640].to(DEV), 0)
        pre.append(tc.cached_prefill_attention(qp, cache, 0, cfg))
    assert torch.equal(pre[0], pre[1])


# ------------------------------------------------------------------------------- the length in device memory
def _layer_buffers(layer):
    names = (("k_pool", "v_pool", "k4_pool", "ks_pool", "v4_pool", "vs_pool") if isinstance(layer, tc.PagedThriftAttentionCacheLayer)
             else ("k_fp16", "v_fp16", "k_packed", "k_scale", "v_packed_t", "v_scale_t"))
    return {n: getattr(layer, n) for n in names + ("k_mean", "k_min", "k_max") if getattr(layer, n) is not None}


@pytest.mark.parametrize("paged,fmt,selection,dtype,d,prompt,steps,max_len",
                         [(False, "nvfp4", "block_mean", torch.float16, 128, 40, 150, 1024),
                          (True, "nvfp4", "quest", torch.bfloat16, 128, 40, 150, 1024),
                          (True, "mxfp4", "block_mean", torch.float16, 64, 40, 150, 1024),
                          (False, "mxfp4", "quest", torch.bfloat16, 64, 40, 150, 1024),
                          # around 256 complete blocks, where the selection kernel changes from one exact pass to
                          # tensor-core scores + exact re-scoring of the candidates
                          (True, "nvfp4", "block_mean", torch.float16, 128, 64 * 256 - 30, 100, 64 * 264),
                          (False, "nvfp4", "quest", torch.float16, 128, 64 * 256 - 30, 100, 64 * 264)])
def test_generation_step_with_device_length_replays_from_one_graph(monkeypatch, paged, fmt, selection, dtype, d, prompt,
                                                                   steps, max_len):
    """append + decode step of a layer, with the sequence length read from device memory, are captured in ONE CUDA
    graph and replayed for 100 - 150 tokens - across page boundaries, growing selected / forced block counts, a prompt
    shorter than one block - and give, token by token, the bytes of update + cached_decode_attention (whose
    launches take the length from the host) run with the same chain count; the caches end up identical too."""
    from thriftattention_b200 import _C

    torch.manual_seed(5)
    b, hq, hkv, chains = 2, 8, 2, 4
    cfg = ta.AttentionConfig(selection=selection, fraction=0.3, quant_format=fmt, sink_blocks=1, local_blocks=1)
    caches = [ta.ThriftAttentionCache(config=cfg, max_cache_len=max_len, paged=paged) for _ in range(2)]
    k0 = torch.randn(b, hkv, prompt, d, device=DEV).to(dtype)
    v0 = torch.randn(b, hkv, prompt, d, device=DEV).to(dtype)
    for c in caches:
        c.update(k0, v0, 0)
    host, graphed = caches
    layer = graphed.layer(0)
    layer.reserve(max_len)
    for pages in range(1, max_len // 64 + 1):      # the host-length path: same chains as the graph's launch
        monkeypatch.setitem(_C._decode_step_splits, (b * hkv, pages), min(chains, pages))

    length = torch.tensor([prompt], dtype=torch.int32, device=DEV)
    q_in = torch.zeros(b, hq, 1, d, device=DEV, dtype=dtype)
    k_in = torch.zeros(b, hkv, 1, d, device=DEV, dtype=dtype)
    v_in = torch.zeros(b, hkv, 1, d, device=DEV, dtype=dtype)
    out_buf = torch.zeros(b, hq, 1, d, device=DEV, dtype=dtype)

    def step():
        res = tc.device_length_decode_step(q_in, k_in, v_in, graphed, 0, cfg, length, max_len=max_len, splits=chains, out=out_buf)
        _C.advance_length(length, 1, max_len)
        return res

    # one eager step on throw-away state (kernel attributes, scratch buffers), then restore and capture
    saved = {n: t.clone() for n, t in _layer_buffers(layer).items()}
    step()
    torch.cuda.synchronize()
    for n, t in _layer_buffers(layer).items():
        t.view(torch.uint8).copy_(saved[n].view(torch.uint8))
    length.fill_(prompt)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        res = step()
    assert res.data_ptr() == out_buf.data_ptr()
    length.fill_(prompt)
    for n, t in _layer_buffers(layer).items():
        t.view(torch.uint8).copy_(saved[n].view(torch.uint8))

    for t in range(steps):
        q = torch.randn(b, hq, 1, d, device=DEV).to(dtype)
        k1 = torch.randn(b, hkv, 1, d, device=DEV).to(dtype)
        v1 = torch.randn(b, hkv, 1, d, device=DEV).to(dtype)
        q_in.copy_(q); k_in.copy_(k1); v_in.copy_(v1)
        graph.replay()
        host.update(k1, v1, 0)
        want = tc.cached_decode_attention(q, host, 0, cfg)
        assert torch.equal(out_buf, want), f"token {prompt + t}"
        want_sel = host.layer(0).selected_blocks
        got_sel = layer.selected_blocks
        if want_sel is not None and want_sel.numel():
            assert torch.equal(got_sel[:, : want_sel.shape[1]], want_sel), f"token {prompt + t}"
            assert bool((got_sel[:, want_sel.shape[1]:] == -1).all())
    assert int(length.item()) == prompt + steps
    a, g = _layer_buffers(host.layer(0)), _layer_buffers(layer)
    if paged:
        tokens = (prompt + steps + 63) // 64 * 64
        layer._gathered = None
        for n in ("k_pool", "v_pool", "k4_pool", "ks_pool", "v4_pool", "vs_pool"):     # the page ids differ: compare by position
            assert torch.equal(host.layer(0)._gather(n, tokens).view(torch.uint8), layer._gather(n, tokens).view(torch.uint8)), n
        for n in ("k_mean", "k_min", "k_max"):
            if n in a:
                assert torch.equal(a[n][:, :, : tokens // 64], g[n][:, :, : tokens // 64]), n
    else:
        for n in a:
            assert torch.equal(a[n].view(torch.uint8), g[n].view(torch.uint8)), n
    _C.decode_status(DEV)


def test_device_length_append_beyond_the_capacity_stores_nothing():
    from thriftattention_b200 import _C

    torch.manual_seed(6)
    cfg = ta.AttentionConfig(selection="block_mean", top_k=2, quant_format="nvfp4")
    cache = ta.ThriftAttentionCache(config=cfg, max_cache_len=128)
    k = torch.randn(1, 2, 100, 128, device=DEV, dtype=torch.float16)
    cache.update(k, k, 0)
    layer = cache.layer(0)
    before = {n: t.clone() for n, t in _layer_buffers(layer).items()}
    length = torch.tensor([128], dtype=torch.int32, device=DEV)
    one = torch.randn(1, 2, 1, 128, device=DEV, dtype=torch.float16)
    _C.cache_append_at(one, one, layer.k_fp16, layer.v_fp16, layer.k_packed, layer.k_scale, layer.v_packed_t, layer.v_scale_t,
                       length, k_mean=layer.k_mean)
    _C.advance_length(length, 1, 128)
    torch.cuda.synchronize()
    assert int(length.item()) == 128
    for n, t in _layer_buffers(layer).items():
        assert torch.equal(t.view(torch.uint8), before[n].view(torch.uint8)), n


@pytest.mark.parametrize("paged", [False, True])
def test_ragged_batch_with_one_device_length_per_sequence(monkeypatch, paged):
    """Three sequences of different lengths in one batch, their lengths in an int32 tensor on the GPU: one graph of
    append + decode step serves them all, and every sequence gets, token by token, the bytes of the host-length calls
    made for that sequence alone."""
    from thriftattention_b200 import _C

    torch.manual_seed(9)
    b, hkv, g, d, max_len, chains, steps = 3, 2, 4, 128, 1024, 3, 70
    prompts = [30, 250, 601]
    dtype = torch.float16
    cfg = ta.AttentionConfig(selection="quest", fraction=0.2, quant_format="nvfp4", sink_blocks=1, local_blocks=2)
    # the batch cache (its Python-side length is not used) and one reference cache per sequence
    batch_cache = ta.ThriftAttentionCache(config=cfg, max_cache_len=max_len, paged=paged)
    refs = [ta.ThriftAttentionCache(config=cfg, max_cache_len=max_len, paged=paged) for _ in range(b)]
    longest = max(prompts)
    k0 = torch.randn(b, hkv, longest, d, device=DEV).to(dtype)
    v0 = torch.randn(b, hkv, longest, d, device=DEV).to(dtype)
    batch_cache.update(torch.zeros_like(k0[:, :, :1]), torch.zeros_like(v0[:, :, :1]), 0)     # allocates the layer
    layer = batch_cache.layer(0)
    layer.reserve(max_len)
    bufs = ((layer.k_pool, layer.v_pool, layer.k4_pool, layer.ks_pool, layer.v4_pool, layer.vs_pool) if paged else
            (layer.k_fp16, layer.v_fp16, layer.k_packed, layer.k_scale, layer.v_packed_t, layer.v_scale_t))
    table = layer.page_table if paged else None
    stats = dict(k_mean=layer.k_mean, k_min=layer.k_min, k_max=layer.k_max)
    # prompts: sequence i alone, through the host-length append on its own slice of the batch cache
    for i, n in enumerate(prompts):
        refs[i].update(k0[i:i + 1, :, :n], v0[i:i + 1, :, :n], 0)
        sl = {name: t[i:i + 1] for name, t in stats.items() if t is not None}
        if paged:
            _C.cache_append_paged(k0[i:i + 1, :, :n].contiguous(), v0[i:i + 1, :, :n].contiguous(), *bufs, table[i:i + 1], start=0,
                                  is_mx=False, stat_block=64, **sl)
        else:
            _C.cache_append(k0[i:i + 1, :, :n].contiguous(), v0[i:i + 1, :, :n].contiguous(), *[t[i:i + 1] for t in bufs], start=0,
                            is_mx=False, stat_block=64, **sl)
    for pages in range(1, max_len // 64 + 1):
        monkeypatch.setitem(_C._decode_step_splits, (hkv, pages), min(chains, pages))

    lengths = torch.tensor(prompts, dtype=torch.int32, device=DEV)
    q_in = torch.zeros(b, hkv, g, d, device=DEV, dtype=dtype)
    k_in = torch.zeros(b, hkv, 1, d, device=DEV, dtype=dtype)
    v_in = torch.zeros(b, hkv, 1, d, device=DEV, dtype=dtype)
    out_buf = torch.zeros(b, hkv, g, d, device=DEV, dtype=dtype)
    sel_buf = None

    def step():
        nonlocal sel_buf
        _C.cache_append_at(k_in, v_in, *bufs, lengths, offset=0, page_table=table, is_mx=False, stat_block=64, **stats)
        _, sel_buf = _C.cached_decode_step_at(q_in, *bufs, layer.k_min, layer.k_max, lengths, offset=1, max_len=max_len,
                                              fraction=0.2, sink=1, local=2, is_mx=False, splits=chains, sel_out=sel_buf,
                                              out=out_buf, page_table=table)
        _C.advance_length(lengths, 1, max_len)

    saved = {i: t.clone() for i, t in enumerate(list(bufs) + [t for t in stats.values() if t is not None])}
    step()                                                  # eager once (kernel attributes, scratch), then undo it
    torch.cuda.synchronize()
    for i, t in enumerate(list(bufs) + [t for t in stats.values() if t is not None]):
        t.view(torch.uint8).copy_(saved[i].view(torch.uint8))
    lengths.copy_(torch.tensor(prompts, dtype=torch.int32))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()

    for t in range(steps):
        q = torch.randn(b, hkv * g, 1, d, device=DEV).to(dtype)
        k1 = torch.randn(b, hkv, 1, d, device=DEV).to(dtype)
        v1 = torch.randn(b, hkv, 1, d, device=DEV).to(dtype)
        q_in.copy_(q.reshape(b, hkv, g, d)); k_in.copy_(k1); v_in.copy_(v1)
        graph.replay()
        for i in range(b):
            refs[i].update(k1[i:i + 1], v1[i:i + 1], 0)
            want = tc.cached_decode_attention(q[i:i + 1], refs[i], 0, cfg)
            assert torch.equal(out_buf[i].reshape(1, hkv * g, 1, d), want), f"sequence {i}, token {prompts[i] + t}"
    assert lengths.tolist() == [n + steps for n in prompts]
    _C.decode_status(DEV)

"""Host-side behaviour of the Transformers hook and generation cache (no GPU): registration, config
resolution, prompt padding arithmetic, routing rules and their messages, capacity policy, crop.
Scenarios follow the reference's tests/test_transformers_integration.py."""
from types import SimpleNamespace

import pytest
import torch

from thriftattention_b200.config import AttentionConfig
from thriftattention_b200.integrations import transformers as hf
from thriftattention_b200.integrations import transformers_cache as cache_mod
from thriftattention_b200.integrations.transformers_cache import (
    ThriftAttentionCache,
    ThriftAttentionCacheLayer,
    use_thriftattention_cache,
)


@pytest.fixture
def registry(monkeypatch):
    """Stand-in for transformers.AttentionInterface; records registrations."""
    seen = {"fn": {}, "mask": []}

    class Registry:
        @staticmethod
        def register(name, fn):
            seen["fn"][name] = fn

    monkeypatch.setattr(hf, "_get_attention_registry", lambda: Registry)
    monkeypatch.setattr(hf, "_register_attention_mask", lambda name=None: seen["mask"].append(name))
    return seen


def _module(name, **extra):
    return SimpleNamespace(config=SimpleNamespace(_attn_implementation=name), training=False, is_causal=True, **extra)


def _qkv(d=64, s=64, h=2):
    return tuple(torch.randn(1, h, s, d) for _ in range(3))


# ----------------------------------------------------------------------------------- registration
def test_register_custom_name_and_config(registry):
    name = hf.register_transformers_attention(hf.TransformersAttentionConfig(name="t_custom", method="fp4"))
    assert name == "t_custom"
    assert registry["fn"]["t_custom"] is hf.thriftattention_forward
    assert registry["mask"] == ["t_custom"]
    assert hf.get_registered_transformers_attention_config("t_custom").method == "fp4"
    assert hf.get_registered_transformers_attention_config("never") is None


def test_default_registration_name(registry):
    assert hf.register_transformers_attention() == "thrift_attention"
    cfg = hf.get_registered_transformers_attention_config("thrift_attention")
    assert (cfg.method, cfg.selection, cfg.fraction, cfg.block_size, cfg.quant_format) == (
        "thrift", "block_mean", 0.05, 64, "nvfp4")


def test_register_real_transformers_interface():
    transformers = pytest.importorskip("transformers")
    if not hasattr(transformers, "AttentionInterface"):
        pytest.skip("no AttentionInterface in this Transformers")
    name = hf.register_transformers_attention(hf.TransformersAttentionConfig(name="t_real_interface"))
    assert transformers.AttentionInterface._global_mapping[name] is hf.thriftattention_forward
    # registering twice is not an error
    hf.register_transformers_attention(hf.TransformersAttentionConfig(name="t_real_interface"))


@pytest.mark.parametrize("field,value,match", [
    ("name", " padded", "non-empty string"), ("name", "", "non-empty string"),
    ("method", "dense", "method must be one of"), ("selection", "random", "selection must be one of"),
    ("quant_format", "int4", "quant_format must be one of"), ("backend", "sm120", "backend must be one of"),
    ("fraction", 1.5, r"fraction must be in \[0, 1\]"), ("top_k", -1, "top_k must be non-negative"),
    ("block_size", 0, "block_size must be positive"), ("fallback", "sdpa", "fallback must be one of"),
    ("sink_blocks", -2, "sink_blocks must be non-negative"),
])
def test_config_validation(registry, field, value, match):
    with pytest.raises(ValueError, match=match):
        hf.register_transformers_attention(hf.TransformersAttentionConfig(**{"name": "t_bad", field: value}))


def test_extensions_are_admitted(registry):
    cfg = hf.TransformersAttentionConfig(name="t_ext", selection="quest", quant_format="mxfp4", block_size=128,
                                         sink_blocks=4, local_blocks=16, backend="sm100").attention_config()
    assert (cfg.selection, cfg.quant_format, cfg.block_size, cfg.sink_blocks, cfg.local_blocks) == (
        "quest", "mxfp4", 128, 4, 16)


# ------------------------------------------------------------------------------- config resolution
def test_registered_config_used_and_cpu_tensors_rejected(registry):
    hf.register_transformers_attention(hf.TransformersAttentionConfig(name="t_registered"))
    module = _module("t_registered", num_key_value_groups=1)
    before = dict(vars(module))
    with pytest.raises(RuntimeError, match="requires CUDA tensors"):
        hf.thriftattention_forward(module, *_qkv(), None, scaling=64 ** -0.5)
    assert vars(module) == before                       # the hook never writes onto the model


def test_unregistered_name_explains_registration():
    with pytest.raises(RuntimeError, match="register_transformers_attention"):
        hf.thriftattention_forward(_module("t_missing"), *_qkv(), None, scaling=64 ** -0.5)


def test_active_cache_config_wins(registry):
    hf.register_transformers_attention(hf.TransformersAttentionConfig(name="t_override", method="fp4"))
    cache = ThriftAttentionCache(config=AttentionConfig(method="thrift", top_k=7))
    with use_thriftattention_cache(cache):
        got = hf._module_config(_module("t_override"))
        assert cache_mod.get_active_thriftattention_cache() is cache
    assert (got.method, got.top_k) == ("thrift", 7)
    assert cache_mod.get_active_thriftattention_cache() is None
    assert hf._module_config(_module("t_override")).method == "fp4"


# ------------------------------------------------------------------------------ prepare generation
def test_prepare_generation_cache_pads_and_freezes_topk(registry):
    hf.register_transformers_attention(hf.TransformersAttentionConfig(name="t_cache", fraction=0.05))
    child = SimpleNamespace()

    class Model:
        config = SimpleNamespace(_attn_implementation="t_cache", max_position_embeddings=1024)

        def modules(self):
            return [self, child]

    prepared = hf.prepare_transformers_generation_cache(Model(), [1, 2, 3], max_new_tokens=5, device="cpu")
    assert prepared.input_ids.shape == (1, 64) and prepared.input_ids[0, :3].tolist() == [1, 2, 3]
    assert prepared.input_ids[0, 3:].abs().sum() == 0
    assert prepared.cache_position.tolist() == list(range(64))
    assert (prepared.prompt_length, prepared.padded_length, prepared.padding) == (3, 64, 61)
    assert prepared.past_key_values.max_cache_len == 69
    assert prepared.past_key_values.prefill_real_seq_len == 3
    assert prepared.config.top_k == 1
    assert vars(child) == {}


@pytest.mark.parametrize("prompt,block,fraction,expect_pad,expect_k", [
    (65536, 64, 0.05, 0, 26), (65536, 128, 0.10, 0, 26), (1000, 64, 0.5, 24, 4), (130, 128, 0.05, 126, 1),
])
def test_prepare_generation_cache_arithmetic(prompt, block, fraction, expect_pad, expect_k):
    from thriftattention_b200.selection import resolve_top_k

    cfg = AttentionConfig(fraction=fraction, block_size=block)
    prepared = hf.prepare_transformers_generation_cache(object(), torch.zeros(prompt, dtype=torch.long), config=cfg,
                                                        max_new_tokens=8)
    assert prepared.padding == expect_pad == (-prompt) % block
    assert prepared.config.top_k == resolve_top_k(max(prompt // block, 1), causal=True, fraction=fraction)
    if prompt == 65536 and block == 64:
        assert prepared.config.top_k == expect_k
    assert prepared.past_key_values.max_cache_len == prompt + expect_pad + 8


def test_prepare_generation_cache_keeps_explicit_topk_and_fp4():
    p = hf.prepare_transformers_generation_cache(object(), [0] * 70, config=AttentionConfig(top_k=9), pad_to_block=False)
    assert p.config.top_k == 9 and p.padding == 0 and p.input_ids.shape == (1, 70)
    p = hf.prepare_transformers_generation_cache(object(), torch.zeros(2, 70, dtype=torch.long),
                                                 config=hf.TransformersAttentionConfig(method="fp4"))
    assert p.config.top_k is None and p.input_ids.shape == (2, 128)
    with pytest.raises(ValueError, match="rank 1 or rank 2"):
        hf.prepare_transformers_generation_cache(object(), torch.zeros(1, 1, 4), config=AttentionConfig())
    with pytest.raises(RuntimeError, match="pass config= explicitly"):
        hf.prepare_transformers_generation_cache(object(), [1, 2])
    with pytest.raises(TypeError):
        hf.prepare_transformers_generation_cache(object(), [1, 2], config={"method": "fp4"})


def test_trim_padding_crops_only_when_padded():
    calls = []
    fake = SimpleNamespace(crop=lambda n: calls.append(n))
    common = dict(input_ids=torch.zeros(1, 1), cache_position=torch.zeros(1), past_key_values=fake, config=AttentionConfig())
    hf.TransformersCacheInputs(prompt_length=64, padded_length=64, padding=0, **common).trim_padding()
    hf.TransformersCacheInputs(prompt_length=3, padded_length=64, padding=61, **common).trim_padding()
    assert calls == [3]


# ------------------------------------------------------------------------------------ routing rules
def test_fast_path_output_is_sequence_major(registry, monkeypatch):
    """The hook returns [B, S, H, D] (integrations/transformers.py:200 of the reference transposes and copies;
    here the kernel epilogue writes that layout, so the hook hands the kernel's tensor through)."""
    for causal in (True, False):
        name = f"t_fast_{causal}"
        hf.register_transformers_attention(hf.TransformersAttentionConfig(name=name, causal=causal))
        seen = {}
        produced = torch.arange(1 * 64 * 2 * 64, dtype=torch.float32).reshape(1, 64, 2, 64)

        def fake_attention(q, k, v, **kwargs):
            seen["config"] = kwargs["config"]
            seen["shape"] = tuple(q.shape)
            return produced

        monkeypatch.setattr(hf, "_fast_path_rejection_reason", lambda *a, **k: None)
        monkeypatch.setattr(hf, "thrift_attention_seq_major", fake_attention)
        module = _module(name)
        module.is_causal = causal
        out, weights = hf.thriftattention_forward(module, *_qkv(), None, scaling=64 ** -0.5)
        assert weights is None and out is produced and seen["shape"] == (1, 2, 64, 64)
        assert seen["config"].causal is causal and seen["config"].selection == "block_mean"


def test_sequence_major_entry_point_shares_the_public_one(monkeypatch):
    """attention_seq_major runs the same selection + backend call as attention, with one extra flag."""
    from thriftattention_b200 import functional

    calls = []

    class Backend:
        def attention(self, q, k, v, **kwargs):
            calls.append(kwargs)
            return "out"

    class Policy:
        def select(self, q, k, **kwargs):
            return "sel"

    monkeypatch.setattr(functional, "select_backend", lambda *a, **k: Backend())
    monkeypatch.setattr(functional, "get_selection_policy", lambda name: Policy())
    q = torch.zeros(1, 2, 64, 64, dtype=torch.float16)
    assert functional.attention(q, q, q) == "out" and functional.attention_seq_major(q, q, q) == "out"
    assert "seq_major_out" not in calls[0] and calls[1]["seq_major_out"] is True
    assert calls[0]["selection"] == calls[1]["selection"] == "sel"


def test_cached_decode_output_is_a_view_in_bshd(registry, monkeypatch):
    hf.register_transformers_attention(hf.TransformersAttentionConfig(name="t_dec"))
    monkeypatch.setattr(hf, "_cached_decode_rejection_reason", lambda *a, **k: None)
    produced = torch.randn(2, 8, 1, 128)
    monkeypatch.setattr(hf, "cached_decode_attention", lambda q, cache, layer_idx, config: produced)
    cache = ThriftAttentionCache(config=AttentionConfig())
    with use_thriftattention_cache(cache):
        out, _ = hf.thriftattention_forward(_module("t_dec", layer_idx=3), torch.randn(2, 8, 1, 128), None, None, None)
    assert out.shape == (2, 1, 8, 128) and out.data_ptr() == produced.data_ptr()
    assert torch.equal(out[:, 0], produced[:, :, 0])


class _Cuda16:
    """Looks like a CUDA fp16 tensor to the routing rules; carries only a shape."""

    is_cuda = True
    dtype = torch.float16

    def __init__(self, *shape):
        self.shape = torch.Size(shape)
        self.ndim = len(shape)


def test_fast_path_rejection_reasons():
    cfg = AttentionConfig()
    q, k, v = _qkv(d=128)
    mod = _module("x")
    reason = lambda *a, **kw: hf._fast_path_rejection_reason(*a, kw)
    assert "training mode" in reason(SimpleNamespace(training=True), q, k, v, None, cfg)
    assert "attention weights" in reason(mod, q, k, v, None, cfg, output_attentions=True)
    assert "explicit attention masks" in reason(mod, q, k, v, torch.ones(1), cfg)
    assert "configured for causal attention but this call requested non-causal" in reason(mod, q, k, v, None, cfg,
                                                                                         is_causal=False)
    assert reason(mod, q, "k", v, None, cfg) is not None
    assert "shaped [batch, heads, seq, head_dim]" in reason(mod, q[0], k, v, None, cfg)
    assert "requires CUDA tensors" in reason(mod, q, k, v, None, cfg)


def test_shape_rules_on_device_like_tensors(monkeypatch):
    monkeypatch.setattr(hf, "_tensor_rejection", lambda *a, **k: None)
    cfg = AttentionConfig()
    mod = _module("x")
    T = _Cuda16
    r = lambda q, k, v, cfg=cfg, **kw: hf._fast_path_rejection_reason(mod, q, k, v, None, cfg, kw)
    assert r(T(1, 8, 128, 128), T(1, 2, 128, 128), T(1, 2, 128, 128)) is None
    assert "head_dim 64 or 128, got 96" in r(T(1, 8, 128, 96), T(1, 2, 128, 96), T(1, 2, 128, 96))
    assert r(T(1, 8, 128, 64), T(1, 2, 128, 64), T(1, 2, 128, 64)) is None
    assert "1/sqrt(head_dim)" in r(T(1, 8, 128, 128), T(1, 2, 128, 128), T(1, 2, 128, 128), scaling=0.5)
    assert r(T(1, 8, 128, 128), T(1, 2, 128, 128), T(1, 2, 128, 128), scaling=torch.tensor(128 ** -0.5)) is None
    assert "query length must be divisible by 64" in r(T(1, 8, 100, 128), T(1, 2, 128, 128), T(1, 2, 128, 128))
    assert "key/value length must be divisible by 64" in r(T(1, 8, 1, 128), T(1, 2, 100, 128), T(1, 2, 100, 128))
    long = 64 * 2049
    assert "at most 2048" in r(T(1, 8, 64, 128), T(1, 2, long, 128), T(1, 2, long, 128))
    assert r(T(1, 8, 1, 128), T(1, 2, long, 128), T(1, 2, long, 128)) is None           # decode has no such limit
    assert r(T(1, 8, 64, 128), T(1, 2, long, 128), T(1, 2, long, 128), cfg=AttentionConfig(method="fp4")) is None


def test_cached_route_rules(monkeypatch):
    monkeypatch.setattr(hf, "_tensor_rejection", lambda *a, **k: None)
    T = _Cuda16
    cfg = AttentionConfig()
    q1, q64 = T(1, 8, 1, 128), T(1, 8, 64, 128)
    k, v = T(1, 2, 64, 128), T(1, 2, 64, 128)
    dec = lambda mod, q=q1, cfg=cfg, **kw: hf._cached_decode_rejection_reason(mod, q, k, v, None, cfg, kw)
    pre = lambda mod, q=q64, **kw: hf._cached_prefill_rejection_reason(mod, q, k, v, None, cfg, kw)
    assert dec(_module("x", layer_idx=0)) == "no active ThriftAttention generation cache"
    assert pre(_module("x", layer_idx=0)) == "no active ThriftAttention generation cache"

    cache = ThriftAttentionCache(config=cfg)
    with use_thriftattention_cache(cache):
        assert "expose layer_idx" in dec(_module("x"))
        assert "integer layer_idx" in dec(_module("x", layer_idx="first"))
        assert "has not been populated" in dec(_module("x", layer_idx=0))
        cache.layer(0).seq_len = 64
        assert dec(_module("x", layer_idx=0)) is None
        assert "has not been populated" in dec(_module("x", layer_idx=1))
        assert "only supports causal" in dec(_module("x", layer_idx=0), cfg=AttentionConfig(causal=False))
        assert "query sequence length 1" in dec(_module("x", layer_idx=0), q=q64)
        assert "at most 16 Q heads" in dec(_module("x", layer_idx=0), q=T(1, 34, 1, 128))
        assert "divisible by KV heads" in dec(_module("x", layer_idx=0), q=T(1, 7, 1, 128))
        assert "64-token KV blocks" in dec(_module("x", layer_idx=0), cfg=AttentionConfig(block_size=128))
        assert "greater than 1" in pre(_module("x", layer_idx=0), q=q1)
        assert pre(_module("x", layer_idx=0)) is None
        cache.layer(0).seq_len = 128
        assert "does not match attention key length" in pre(_module("x", layer_idx=0))


def test_rejected_call_raises_with_reason(registry):
    hf.register_transformers_attention(hf.TransformersAttentionConfig(name="t_reject"))
    with pytest.raises(RuntimeError, match="fast path rejected this attention call: .*explicit attention masks"):
        hf.thriftattention_forward(_module("t_reject"), *_qkv(), torch.ones(1, 1, 64, 64))


# ------------------------------------------------------------------------------------------- cache
class _RecordingExtension:
    """Extension stand-in for CPU tests: records cache_append calls and performs only the 16-bit stores."""

    def __init__(self):
        self.appends = []

    def cache_append(self, k_new, v_new, k_hi, v_hi, k_codes, k_scales, v_codes_t, v_scales_t, *, start, k_count=None,
                     v_count=None, k_mean=None, k_min=None, k_max=None, is_mx=False, stat_block=64, keep_k=False,
                     keep_v=False):
        kc = k_new.shape[2] if k_new is not None else (k_count or 0)
        vc = v_new.shape[2] if v_new is not None else (v_count or 0)
        self.appends.append(dict(start=start, k=kc, v=vc, stats=k_mean is not None, minmax=k_min is not None,
                                 is_mx=is_mx, keep_k=keep_k, keep_v=keep_v, has_k=k_new is not None,
                                 has_v=v_new is not None))
        if k_new is not None:
            k_hi[:, :, start:start + kc] = k_new
        if v_new is not None:
            v_hi[:, :, start:start + vc] = v_new


@pytest.fixture
def ext(monkeypatch):
    fake = _RecordingExtension()
    monkeypatch.setattr(cache_mod, "get_extension", lambda: fake)
    return fake


def test_update_is_one_fused_append_and_views_are_logical(ext):
    layer = ThriftAttentionCacheLayer()
    k, v = torch.randn(2, 3, 70, 128).half(), torch.randn(2, 3, 70, 128).half()
    key, value = layer.update(k, v)
    assert len(ext.appends) == 1 and ext.appends[0] == dict(start=0, k=70, v=70, stats=True, minmax=False, is_mx=False,
                                                           keep_k=False, keep_v=False, has_k=True, has_v=True)
    assert layer.seq_len == 70 and layer.capacity == 128
    assert key.shape == (2, 3, 70, 128) and torch.equal(key, k) and torch.equal(value, v)
    assert layer.k_packed.shape == (2, 3, 128, 64) and layer.k_scale.shape == (2, 3, 128, 8)
    assert layer.k_scale.dtype == torch.float8_e4m3fn
    assert layer.v_packed_t.shape == (2, 3, 128, 64) and layer.v_scale_t.shape == (2, 3, 128, 8)
    assert layer.k_mean.shape == (2, 3, 2, 128) and layer.k_min is None
    # a decode token appends at seq_len; cache_position overrides it
    layer.update(k[:, :, :1], v[:, :, :1])
    assert ext.appends[-1]["start"] == 70 and layer.seq_len == 71
    layer.update(k[:, :, :2], v[:, :, :2], {"cache_position": torch.tensor([10, 11])})
    assert ext.appends[-1]["start"] == 10 and layer.seq_len == 71
    kp, vp, ks, vs = layer.packed_views()
    assert kp.shape[2] == 128 and ks.shape[2] == 128 and vp.shape[3] == 64 and vs.shape[3] == 8
    # zero-length updates launch nothing
    n = len(ext.appends)
    layer.update(k[:, :, :0], v[:, :, :0])
    assert len(ext.appends) == n


def test_mxfp4_quest_layer_layout(ext):
    cache = ThriftAttentionCache(config=AttentionConfig(selection="quest", quant_format="mxfp4"), max_cache_len=300)
    cache.update(torch.zeros(1, 2, 5, 128).bfloat16(), torch.zeros(1, 2, 5, 128).bfloat16(), 1)
    assert len(cache) == 2 and cache.get_seq_length(0) == 0 and cache.get_seq_length(1) == 5
    layer = cache.layers[1]
    assert layer.capacity == 384 and layer.k_scale.shape == (1, 2, 384, 4) and layer.k_scale.dtype == torch.float8_e8m0fnu
    assert layer.v_scale_t.shape == (1, 2, 128, 12) and layer.k_min.shape == layer.k_max.shape == (1, 2, 6, 128)
    assert ext.appends[0]["is_mx"] and ext.appends[0]["minmax"]


@pytest.mark.parametrize("limit,lengths,capacities", [
    (None, [1, 64, 65, 129, 300, 1000], [128, 128, 128, 256, 512, 1024]),
    (69, [64, 69], [128, 128]),
    (1000, [10, 1000], [1024, 1024]),
])
def test_capacity_policy(ext, limit, lengths, capacities):
    layer = ThriftAttentionCacheLayer(max_cache_len=limit)
    got = []
    for n in lengths:
        add = n - layer.seq_len
        layer.update(torch.ones(1, 1, add, 128).half() * n, torch.ones(1, 1, add, 128).half())
        got.append(layer.capacity)
        assert layer.key_view()[0, 0, -1, 0] == n and layer.key_view()[0, 0, 0, 0] == lengths[0]   # growth keeps old rows
    assert got == capacities
    if limit is not None:
        with pytest.raises(ValueError, match="exceeds max_cache_len"):
            layer.update(torch.ones(1, 1, limit, 128).half(), torch.ones(1, 1, limit, 128).half())


def test_update_validation(ext):
    layer = ThriftAttentionCacheLayer()
    h = lambda *s: torch.zeros(*s).half()
    with pytest.raises(ValueError, match=r"\[batch, heads, seq, head_dim\]"):
        layer.update(h(2, 4, 8), h(2, 4, 8))
    with pytest.raises(ValueError, match="identical shapes"):
        layer.update(h(1, 1, 4, 128), h(1, 1, 5, 128))
    with pytest.raises(ValueError, match="float16 or bfloat16"):
        layer.update(torch.zeros(1, 1, 4, 128), torch.zeros(1, 1, 4, 128))
    with pytest.raises(ValueError, match="same dtype"):
        layer.update(h(1, 1, 4, 128), h(1, 1, 4, 128).bfloat16())
    with pytest.raises(ValueError, match="contiguous cache_position"):
        layer.update(h(1, 1, 2, 128), h(1, 1, 2, 128), {"cache_position": torch.tensor([0, 2])})
    layer.update(h(1, 2, 4, 128), h(1, 2, 4, 128))
    with pytest.raises(ValueError, match="shape changed"):
        layer.update(h(2, 2, 4, 128), h(2, 2, 4, 128))
    with pytest.raises(ValueError, match="dtype changed"):
        layer.update(h(1, 2, 4, 128).bfloat16(), h(1, 2, 4, 128).bfloat16())
    with pytest.raises(ValueError, match="requires layer_idx"):
        ThriftAttentionCache().update(h(1, 1, 1, 128), h(1, 1, 1, 128))
    with pytest.raises(RuntimeError, match="not been initialized"):
        ThriftAttentionCacheLayer().key_view()


def test_crop_zeroes_rounded_physical_tail():
    layer = ThriftAttentionCacheLayer()
    layer.seq_len = layer.capacity = 128
    layer.k_fp16, layer.v_fp16 = torch.ones(1, 1, 128, 64), torch.ones(1, 1, 128, 64)
    layer.k_packed = layer.k_scale = layer.v_packed_t = layer.v_scale_t = torch.empty(1)
    calls = []
    layer._quantize_k_range = lambda rows, start, end: calls.append(("k", tuple(rows.shape), float(rows.abs().sum()), start, end))
    layer._quantize_v_range = lambda start, end: calls.append(("v", start, end))
    layer.crop(65)
    assert layer.seq_len == 65
    assert torch.all(layer.k_fp16[:, :, :65] == 1) and torch.all(layer.v_fp16[:, :, :65] == 1)
    assert torch.all(layer.k_fp16[:, :, 65:] == 0) and torch.all(layer.v_fp16[:, :, 65:] == 0)
    assert calls == [("k", (1, 1, 63, 64), 0.0, 65, 128), ("v", 65, 128)]
    # K is cleared to the next multiple of 64 only, V to the next multiple of 128
    layer.k_fp16.fill_(1), layer.v_fp16.fill_(1)
    layer.seq_len = 128
    calls.clear()
    layer.crop(-118)
    assert layer.seq_len == 10 and calls == [("k", (1, 1, 54, 64), 0.0, 10, 64), ("v", 10, 128)]
    assert torch.all(layer.k_fp16[:, :, 64:] == 1) and torch.all(layer.v_fp16[:, :, 10:] == 0)
    calls.clear()
    layer.crop(500)                                   # longer than the content: nothing to do
    assert layer.seq_len == 10 and calls == []


def test_crop_launches(ext):
    layer = ThriftAttentionCacheLayer()
    layer.update(torch.ones(1, 1, 128, 128).half(), torch.ones(1, 1, 128, 128).half())
    ext.appends.clear()
    layer.crop(3)
    assert ext.appends == [
        dict(start=3, k=61, v=0, stats=False, minmax=False, is_mx=False, keep_k=False, keep_v=False, has_k=True, has_v=False),
        dict(start=3, k=0, v=125, stats=False, minmax=False, is_mx=False, keep_k=False, keep_v=True, has_k=False, has_v=False)]


def test_cache_protocol(ext):
    cache = ThriftAttentionCache.from_model(SimpleNamespace(config=SimpleNamespace(max_position_embeddings=256)))
    assert cache.max_cache_len == 256 and cache.get_max_cache_shape() == 256 and not cache.is_initialized
    assert cache.get_mask_sizes(5, 0) == (5, 0) and cache.max_batch_size is None
    k = torch.randn(2, 1, 100, 128).half()
    for i in range(2):
        cache.update(k, k, i, {"cache_position": torch.arange(100)})
    assert cache.seen_tokens == 100 and cache.get_seq_length(1) == 100 and cache.get_seq_length(7) == 0
    assert cache.get_mask_sizes(1, 1) == (101, 0) and cache.max_batch_size == 2 and cache.is_initialized
    assert cache.is_sliding == [False, False] and not cache.is_compileable
    assert cache.get_usable_length(10) == 100 and cache.get_usable_length(200) == 56
    assert cache[1][0].shape == (2, 1, 100, 128) and len(cache.to_legacy_cache()) == 2
    cache.reorder_cache(torch.tensor([1, 1]))
    assert torch.equal(cache[0][0][0], k[1])
    cache.batch_repeat_interleave(2)
    assert cache.max_batch_size == 4 and cache.layers[0].k_mean.shape[0] == 4
    cache.batch_select_indices(torch.tensor([0]))
    assert cache.max_batch_size == 1
    cache.crop(40)
    assert cache.seen_tokens == 40 and cache.get_seq_length(1) == 40
    cache.reset()
    assert cache.seen_tokens == 0 and cache.get_seq_length(0) == 0
    assert cache_mod.is_thriftattention_cache(cache) and not cache_mod.is_thriftattention_cache(object())


# --------------------------------------------------------------------------- selection over the cache
def test_cached_decode_local_selection(monkeypatch):
    calls = []

    class Extension:
        @staticmethod
        def single_query_local_topk(q_grouped, selected_count, num_kv_blocks):
            calls.append((tuple(q_grouped.shape), selected_count, num_kv_blocks))
            return torch.tensor([[2, 3]], dtype=torch.int32)

    monkeypatch.setattr(cache_mod, "get_extension", lambda: Extension)
    got = cache_mod.select_cached_decode_blocks(torch.empty(1, 1, 1, 64), SimpleNamespace(seq_len=256),
                                                AttentionConfig(selection="local", top_k=2))
    assert got.tolist() == [[2, 3]] and calls == [((1, 1, 1, 64), 2, 4)]
    none = cache_mod.select_cached_decode_blocks(torch.empty(2, 3, 1, 64), SimpleNamespace(seq_len=63),
                                                 AttentionConfig(selection="local", top_k=2))
    assert none.shape == (6, 0) and none.dtype == torch.int32
    with pytest.raises(ValueError, match="unsupported cached decode selection"):
        cache_mod.select_cached_decode_blocks(torch.empty(1, 1, 1, 64), SimpleNamespace(seq_len=64),
                                              SimpleNamespace(selection="other"))


def test_cached_prefill_local_selection(monkeypatch):
    from thriftattention_b200.selection import local

    calls = []

    class Extension:
        @staticmethod
        def local_block_topk(q, num_kv_blocks, selected_count, causal, block_size):
            calls.append((tuple(q.shape), num_kv_blocks, selected_count, causal, block_size))
            return torch.tensor([[[0, 1], [1, 2]]], dtype=torch.int32)

    monkeypatch.setattr(local, "check_qkv", lambda *a, **k: None)
    monkeypatch.setattr(local, "get_extension", lambda: Extension)
    q = torch.empty(1, 1, 128, 64, dtype=torch.float16)
    k = torch.empty(1, 1, 256, 64, dtype=torch.float16)
    got = cache_mod.select_cached_prefill_blocks(q, k, SimpleNamespace(key_view=lambda: k),
                                                 AttentionConfig(selection="local", top_k=2))
    assert got.tolist() == [[[0, 1], [1, 2]]] and calls == [((1, 1, 128, 64), 4, 2, True, 64)]


def test_decode_topk_selection_counts_only_complete_blocks(monkeypatch):
    calls = []

    class Extension:
        @staticmethod
        def select_decode_blocks(q_grouped, k_a, k_b, count, num_blocks, is_bf16, sink=0, local=0, out=None):
            calls.append(dict(quest=k_b is not None, count=count, blocks=num_blocks, sink=sink, local=local,
                              out=tuple(out.shape)))
            return out

    monkeypatch.setattr(cache_mod, "get_extension", lambda: Extension)
    layer = ThriftAttentionCacheLayer(track_minmax=True)
    layer.seq_len = 64 * 10 + 17
    layer.k_mean = layer.k_min = layer.k_max = torch.zeros(2, 4, 16, 128).half()
    q = torch.zeros(2, 4, 4, 128).half()
    cache_mod.select_cached_decode_blocks(q, layer, AttentionConfig(top_k=3))
    cache_mod.select_cached_decode_blocks(q, layer, AttentionConfig(selection="quest", fraction=0.25, sink_blocks=1,
                                                                    local_blocks=2))
    cache_mod.select_cached_decode_blocks(q, layer, AttentionConfig(top_k=9, sink_blocks=4, local_blocks=4))
    assert calls == [
        dict(quest=False, count=3, blocks=10, sink=0, local=0, out=(8, 3)),
        dict(quest=True, count=2, blocks=10, sink=1, local=2, out=(8, 5)),     # round(0.25 * 10) = 2, non-causal rule
        dict(quest=False, count=9, blocks=10, sink=0, local=1, out=(8, 10)),   # forced blocks clipped to what is left
    ]
    with pytest.raises(ValueError, match="same dtype"):
        cache_mod.select_cached_decode_blocks(q.bfloat16(), layer, AttentionConfig(top_k=3))
    layer.seq_len = 40
    assert cache_mod.select_cached_decode_blocks(q, layer, AttentionConfig(top_k=3)).shape == (8, 0)


def test_query_block_means_skip_padding(monkeypatch):
    class Extension:
        @staticmethod
        def block_stats(x, block, mean=False, minmax=False):
            b, h, s, d = x.shape
            return x.reshape(b, h, s // block, block, d).float().mean(3).to(x.dtype), None, None

    monkeypatch.setattr(cache_mod, "get_extension", lambda: Extension)
    q = torch.randn(1, 2, 256, 16).half()
    full = cache_mod._query_block_means(q, 64, None)
    assert torch.equal(full, cache_mod._query_block_means(q, 64, 256)) and full.shape == (1, 2, 4, 16)
    part = cache_mod._query_block_means(q, 64, 70)
    assert torch.equal(part[:, :, 0], full[:, :, 0])
    assert torch.allclose(part[:, :, 1].float(), q[:, :, 64:70].float().mean(2), atol=1e-3)
    assert part[:, :, 2:].abs().sum() == 0
    edge = cache_mod._query_block_means(q, 64, 128)
    assert torch.equal(edge[:, :, :2], full[:, :, :2]) and edge[:, :, 2:].abs().sum() == 0


def test_cache_position_is_read_once_per_forward():
    """Every layer of a forward pass receives the same cache_position tensor object; its value is read (a device
    synchronisation on a GPU) for the first layer only.  A new tensor, or the same one changed in place, is read
    again."""
    from thriftattention_b200.integrations import transformers_cache as cache_mod

    first = torch.tensor([5])
    assert cache_mod._cache_position_start({"cache_position": first}, 0) == 5
    memo = cache_mod._POSITION_MEMO
    assert memo[0]() is first and memo[2] == 5
    second = torch.tensor([9])
    assert cache_mod._cache_position_start({"cache_position": second}, 0) == 9
    assert cache_mod._cache_position_start({"cache_position": first}, 0) == 5     # other object: read again
    first.add_(1)
    assert cache_mod._cache_position_start({"cache_position": first}, 0) == 6     # changed in place: read again
    assert cache_mod._cache_position_start({"cache_position": torch.arange(3, 7)}, 0) == 3
    with pytest.raises(ValueError, match="contiguous cache_position"):
        cache_mod._cache_position_start({"cache_position": torch.tensor([3, 5])}, 0)
    assert cache_mod._cache_position_start(None, 7) == 7 and cache_mod._cache_position_start({"cache_position": 4}, 7) == 4


def test_device_length_mode_refuses_updates_it_cannot_serve():
    """With the length kept on the GPU the Python-side lengths are stale: anything but the single-token step of the
    active cache (which the attention function appends itself) is an error, not a silent write at a wrong position."""
    cache = ThriftAttentionCache(config=AttentionConfig(), max_cache_len=128)
    with pytest.raises(RuntimeError, match="filled cache"):
        cache.enable_device_length()
    cache.layers.append(cache_mod.ThriftAttentionCacheLayer(max_cache_len=128, quant_format="nvfp4", track_minmax=False))
    cache.layers[0].seq_len = 5
    cache.device_length = torch.zeros(1, dtype=torch.int32)
    k = torch.zeros(1, 2, 3, 128, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="device-length mode"):
        cache.update(k, k, 0)                                  # three tokens
    with pytest.raises(RuntimeError, match="device-length mode"):
        cache.update(k[:, :, :1], k[:, :, :1], 0)              # one token, but the cache is not the active one
    with cache_mod.use_thriftattention_cache(cache):
        got_k, got_v = cache.update(k[:, :, :1], k[:, :, :1], 0)
    assert got_k.data_ptr() == k.data_ptr() and cache.layers[0].seq_len == 5     # handed on, nothing stored

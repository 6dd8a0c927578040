"""Python-layer conformance with the reference's API: orchestration in ``attention``, argument
order across the operator boundary, configuration defaults and error behaviour.  These mirror
the reference's mock-based unit tests (tests/test_functional.py, tests/test_selection.py)."""
from types import SimpleNamespace
from typing import get_args

import pytest
import torch

import thriftattention_b200 as ta
from thriftattention_b200.config import AttentionConfig, SelectionMethod


class FakeQuantFormat:
    def __init__(self, name="nvfp4"):
        self.name = name

    def quantize_qkv(self, *a, **k):
        return "qp", "kp", "vp", "qs", "ks", "vs"

    def quantize_single_query_qkv(self, *a, **k):
        return "qp", "kp", "vp", "qs", "ks", "vs"


def test_config_defaults_match_reference():
    c = AttentionConfig()
    assert (c.method, c.causal, c.selection, c.fraction, c.top_k, c.block_size, c.quant_format, c.backend,
            c.implementation, c.fallback) == ("thrift", True, "block_mean", 0.05, None, 64, "nvfp4", "auto", "auto", "error")
    assert (c.sink_blocks, c.local_blocks) == (0, 0)
    assert "local" in get_args(SelectionMethod)
    with pytest.raises(Exception):
        c.method = "fp4"  # frozen


def test_public_surface():
    for name in ("AttentionConfig", "attention", "QuantFormat", "get_quant_format", "SelectionConfig",
                 "get_selection_policy", "resolve_top_k"):
        assert hasattr(ta, name)
    assert ta.get_selection_policy("quest").name == "quest"
    assert ta.get_selection_policy("local").name == "local"
    assert ta.get_selection_policy("block_mean").name == "block_mean"
    with pytest.raises(NotImplementedError):
        ta.get_selection_policy("nope")
    assert ta.get_quant_format("nvfp4").name == "nvfp4" and ta.get_quant_format("mxfp4").name == "mxfp4"
    with pytest.raises(NotImplementedError):
        ta.get_quant_format("int4")


def test_attention_orchestrates_fp4_without_selection(monkeypatch):
    from thriftattention_b200 import functional

    calls = []
    q = k = v = torch.empty(1, 1, 64, 64)
    config = AttentionConfig(method="fp4", causal=False)
    fmt = FakeQuantFormat()

    class Backend:
        def attention(self, *args, **kwargs):
            calls.append((args, kwargs))
            return "out"

    def fail(name):
        raise AssertionError("selection policy must not be requested for method='fp4'")

    monkeypatch.setattr(functional, "get_quant_format", lambda name: fmt)
    monkeypatch.setattr(functional, "get_selection_policy", fail)
    monkeypatch.setattr(functional, "select_backend", lambda cfg, qf, *, head_dim, device=None: Backend())
    assert functional.attention(q, k, v, config=config) == "out"
    assert calls == [((q, k, v), {"selection": None, "quant_format": fmt, "config": config, "is_bf16": False})]


def test_attention_builds_selection_for_thrift(monkeypatch):
    from thriftattention_b200 import functional

    calls = []
    q, k, v = (torch.empty(1, 1, 64, 64, dtype=torch.bfloat16) for _ in range(3))
    config = AttentionConfig(method="thrift", causal=False, selection="block_mean", fraction=0.25, top_k=3, block_size=64)
    fmt = FakeQuantFormat()

    class Policy:
        def select(self, q_arg, k_arg, *, config, causal, is_bf16):
            calls.append(("select", q_arg, k_arg, config, causal, is_bf16))
            return "selected"

    class Backend:
        def attention(self, *args, **kwargs):
            calls.append(("backend", args, kwargs))
            return "out"

    monkeypatch.setattr(functional, "get_quant_format", lambda name: fmt)
    monkeypatch.setattr(functional, "get_selection_policy", lambda name: Policy())
    monkeypatch.setattr(functional, "select_backend", lambda cfg, qf, *, head_dim, device=None: Backend())
    assert functional.attention(q, k, v, config=config) == "out"
    _, q_arg, k_arg, sel_cfg, causal, is_bf16 = calls[0]
    assert q_arg is q and k_arg is k
    assert (sel_cfg.name, sel_cfg.fraction, sel_cfg.top_k, sel_cfg.block_size) == ("block_mean", 0.25, 3, 64)
    assert causal is False and is_bf16 is True
    assert calls[1] == ("backend", (q, k, v), {"selection": "selected", "quant_format": fmt, "config": config, "is_bf16": True})


@pytest.mark.parametrize("method,causal,fmt,expected", [
    ("fp4", True, "nvfp4", "fp4_attention_causal_nvfp4_packed"),
    ("fp4", False, "mxfp4", "fp4_attention_noncausal_mxfp4_packed"),
    ("thrift", True, "nvfp4", "thrift_attention_causal_nvfp4_packed"),
    ("thrift", False, "mxfp4", "thrift_attention_noncausal_mxfp4_packed"),
])
def test_backend_tiled_dispatch_and_argument_order(monkeypatch, method, causal, fmt, expected):
    """The operator boundary keeps the reference's positional order
    (q_hi, k_hi, v_hi, selection, *packed, is_bf16) — tests/test_functional.py:174-271 there."""
    from thriftattention_b200.backends import sm100

    seen = {}

    def make(name):
        def fn(*args):
            seen["name"], seen["args"] = name, args
            return "out"
        return fn

    ext = SimpleNamespace(**{n: make(n) for n in (
        "fp4_attention_causal_nvfp4_packed", "fp4_attention_noncausal_nvfp4_packed", "fp4_attention_causal_mxfp4_packed",
        "fp4_attention_noncausal_mxfp4_packed", "thrift_attention_causal_nvfp4_packed",
        "thrift_attention_noncausal_nvfp4_packed", "thrift_attention_causal_mxfp4_packed",
        "thrift_attention_noncausal_mxfp4_packed")})
    monkeypatch.setattr(sm100, "get_extension", lambda: ext)
    monkeypatch.setattr(sm100, "check_qkv", lambda *a: None)
    q, k, v = torch.empty(1, 2, 128, 64), torch.empty(1, 1, 128, 64), torch.empty(1, 1, 128, 64)
    cfg = AttentionConfig(method=method, causal=causal, quant_format=fmt)
    out = sm100.SM100_BACKEND.attention(q, k, v, selection="sel", quant_format=FakeQuantFormat(fmt), config=cfg, is_bf16=False)
    assert out == "out" and seen["name"] == expected
    if method == "fp4":
        assert seen["args"] == ("qp", "kp", "vp", "qs", "ks", "vs", False)
    else:
        assert seen["args"][3:] == ("sel", "qp", "kp", "vp", "qs", "ks", "vs", False)
        assert all(a.shape == b.shape for a, b in zip(seen["args"][:3], (q, k, v)))


def test_backend_single_query_groups_heads(monkeypatch):
    from thriftattention_b200.backends import sm100

    seen = {}

    def fn(*args):
        seen["args"] = args
        return torch.zeros(2, 2, 4, 64)

    ext = SimpleNamespace(thrift_attention_single_query_nvfp4_packed=fn)
    monkeypatch.setattr(sm100, "get_extension", lambda: ext)
    monkeypatch.setattr(sm100, "check_qkv", lambda *a: None)
    q, k, v = torch.randn(2, 8, 1, 64), torch.randn(2, 2, 128, 64), torch.randn(2, 2, 128, 64)
    out = sm100.SM100_BACKEND.attention(q, k, v, selection="sel", quant_format=FakeQuantFormat(), config=AttentionConfig(),
                                        is_bf16=False)
    assert out.shape == (2, 8, 1, 64)
    q_grouped = seen["args"][0]
    assert q_grouped.shape == (2, 2, 4, 64) and torch.equal(q_grouped, q.reshape(2, 2, 4, 64))
    assert seen["args"][3:] == ("sel", "qp", "kp", "vp", "qs", "ks", "vs", False)


def test_backend_rejections():
    from thriftattention_b200.backends import sm100
    from thriftattention_b200.backends.registry import select_backend
    from thriftattention_b200.backends.single_query import _group_single_query, _use_single_query

    fmt = FakeQuantFormat()
    with pytest.raises(ValueError, match="head_dim"):
        select_backend(AttentionConfig(), fmt, head_dim=96)
    with pytest.raises(NotImplementedError):
        select_backend(AttentionConfig(backend="sm120"), fmt, head_dim=64)
    assert select_backend(AttentionConfig(), fmt, head_dim=128).name == "sm100"
    q = torch.empty(1, 34, 1, 64)
    with pytest.raises(NotImplementedError, match="at most 16"):
        _group_single_query(q, 2)
    with pytest.raises(ValueError):
        _use_single_query(torch.empty(1, 1, 4, 64), "single_query")
    with pytest.raises(ValueError, match="CUDA"):
        sm100.SM100_BACKEND.attention(torch.empty(1, 1, 64, 64, dtype=torch.float16), torch.empty(1, 1, 64, 64, dtype=torch.float16),
                                      torch.empty(1, 1, 64, 64, dtype=torch.float16), selection=None, quant_format=fmt,
                                      config=AttentionConfig(method="fp4"), is_bf16=False)


def test_checks_messages():
    from thriftattention_b200 import _checks

    with pytest.raises(ValueError, match="must be a CUDA tensor"):
        _checks.require_cuda_half("q", torch.empty(1, 1, 1, 64, dtype=torch.float16))
    with pytest.raises(ValueError, match="divisible by 64"):
        _checks.require_block_aligned("k", 100, 64)
    with pytest.raises(ValueError, match="head_dim must be 64 or 128"):
        _checks.require_supported_head_dim(96)


def test_selection_policies_route_by_query_length(monkeypatch):
    from thriftattention_b200.selection import SelectionConfig, block_mean, local, quest

    calls = []
    for mod, pair, key in ((block_mean, "select_block_pairs", "select_key_blocks"),
                           (quest, "select_quest_block_pairs", "select_quest_key_blocks"),
                           (local, "select_local_block_pairs", "select_local_key_blocks")):
        monkeypatch.setattr(mod, pair, lambda *a, _n=pair, **k: calls.append((_n, k)) or "pairs")
        monkeypatch.setattr(mod, key, lambda *a, _n=key, **k: calls.append((_n, k)) or "keys")
    for name in ("block_mean", "quest", "local"):
        pol = ta.get_selection_policy(name)
        cfg = SelectionConfig(name=name, top_k=2, fraction=None, block_size=64)
        assert pol.select(torch.empty(1, 1, 64, 64), torch.empty(1, 1, 64, 64), config=cfg, causal=True, is_bf16=False) == "pairs"
        assert pol.select(torch.empty(1, 1, 1, 64), torch.empty(1, 1, 64, 64), config=cfg, causal=True, is_bf16=False) == "keys"
        with pytest.raises(ValueError, match="does not match"):
            pol.select(torch.empty(1, 1, 1, 64), torch.empty(1, 1, 64, 64), config=SelectionConfig(name="quest" if name != "quest" else "local"),
                       causal=True, is_bf16=False)
    assert [c[0] for c in calls] == ["select_block_pairs", "select_key_blocks", "select_quest_block_pairs",
                                     "select_quest_key_blocks", "select_local_block_pairs", "select_local_key_blocks"]
    assert calls[0][1]["causal"] is True and "causal" not in calls[1][1]


def test_attention_host_argument_errors():
    """The host-side entry point validates shapes before it touches CUDA."""
    import thriftattention_b200 as ta

    q = torch.zeros(1, 4, 64, 128, dtype=torch.float16)
    k = torch.zeros(1, 3, 64, 128, dtype=torch.float16)
    with pytest.raises(ValueError, match="multiple of the number of KV heads"):
        ta.attention_host(q, k, k)
    with pytest.raises(ValueError, match="expects q"):
        ta.attention_host(q, k, k[:, :2])
    with pytest.raises(ValueError, match="kv_heads_per_chunk"):
        ta.attention_host(q, k[:, :2], k[:, :2], kv_heads_per_chunk=0)

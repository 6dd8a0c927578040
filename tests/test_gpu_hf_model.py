"""End to end through Hugging Face Transformers on the GPU: a small random-init Llama (head_dim 128,
grouped-query attention) loaded with the registered attention name runs a padded prefill and a few decode
steps over a ThriftAttentionCache.  The SAME weights are run a second time with an attention function that
calls the CPU oracle (block-mean selection + mixed FP4/16-bit attention on the same K/V), and the logits
of the two runs are compared."""
import pytest
import torch

import oracle
from thriftattention_b200 import AttentionConfig
from thriftattention_b200.integrations import (
    TransformersAttentionConfig,
    prepare_transformers_generation_cache,
    register_transformers_attention,
)
from thriftattention_b200.integrations import transformers as hf
from thriftattention_b200.selection import resolve_top_k

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
transformers = pytest.importorskip("transformers")

_ORACLE_STATE = {}


def _oracle_forward(module, query, key, value, attention_mask, **kwargs):
    """Attention function with the reference semantics, computed by the CPU oracle."""
    cfg = _ORACLE_STATE["config"]
    real = _ORACLE_STATE["real_q_len"]
    assert attention_mask is None
    q, k, v = query.cpu(), key.cpu(), value.cpu()
    b, hq, sq, d = q.shape
    hkv, n = k.shape[1], k.shape[2]
    if sq > 1:
        qm, = oracle.block_stats(q, 64, ("mean",))
        if real is not None and real < sq:
            full, tail = divmod(real, 64)
            if tail:
                qm[:, :, full] = (q[:, :, full * 64: full * 64 + tail].float().sum(2) / tail).to(qm.dtype)
                qm[:, :, full + 1:] = 0
            else:
                qm[:, :, full:] = 0
        mean, = oracle.block_stats(k, 64, ("mean",))
        count = resolve_top_k(n // 64, causal=True, top_k=cfg.top_k, fraction=cfg.fraction)
        sel = oracle.select_prefill(qm, mean, k=count, causal=True)
        out = oracle.prefill_attention(q, k, v, sel, fmt="nvfp4", block=64, causal=True)
        return out.transpose(1, 2).contiguous().to(query.device), None
    pad = max(64, -(-n // 64) * 64)
    kp = torch.zeros(b, hkv, pad, d, dtype=k.dtype)
    vp = torch.zeros(b, hkv, pad, d, dtype=k.dtype)
    kp[:, :, :n], vp[:, :, :n] = k, v
    complete = n // 64
    count = resolve_top_k(complete, causal=False, top_k=cfg.top_k, fraction=cfg.fraction)
    qg = q.reshape(b, hkv, hq // hkv, d)
    mean, = oracle.block_stats(kp, 64, ("mean",))
    sel = oracle.select_decode(qg, mean, k=count, num_kv_blocks=complete) if count else None
    splits = _ORACLE_STATE["pick_splits"](b * hkv, pad // 64)
    out = oracle.decode_attention(qg, kp, vp, sel, fmt="nvfp4", splits=min(splits, pad // 64))
    return out.reshape(b, 1, hq, d).to(query.device), None


def _tiny_llama(name):
    cfg = transformers.LlamaConfig(vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                                   max_position_embeddings=4096)
    cfg._attn_implementation = name
    torch.manual_seed(0)
    return transformers.LlamaForCausalLM(cfg).half().eval().to(DEV)


def _hook_against_oracle(model_factory, hook_name, fraction, vocab, prompt_len, new_tokens, padding, layers, paged=False):
    from thriftattention_b200._extension import get_extension

    name = register_transformers_attention(TransformersAttentionConfig(name=hook_name, fraction=fraction))
    transformers.AttentionInterface.register("thrift_oracle_test", _oracle_forward)
    try:
        from transformers import AttentionMaskInterface
        from transformers.masking_utils import sdpa_mask

        AttentionMaskInterface.register("thrift_oracle_test", sdpa_mask)
    except ImportError:
        pass
    model = model_factory(name)
    ids = torch.randint(0, vocab, (1, prompt_len), generator=torch.Generator().manual_seed(1)).to(DEV)

    # ---------------- run A: the registered sm_100a path over a ThriftAttentionCache
    prep = prepare_transformers_generation_cache(model, ids, max_new_tokens=new_tokens, paged=paged)
    assert prep.past_key_values.paged == paged
    assert (prep.padding, prep.padded_length) == (padding, prompt_len + padding)
    count = resolve_top_k(prompt_len // 64, causal=True, fraction=fraction)
    assert prep.config.top_k == count
    logits_a, tokens = [], []
    with prep.activate(), torch.no_grad():
        out = model(input_ids=prep.input_ids, past_key_values=prep.past_key_values, cache_position=prep.cache_position,
                    use_cache=True)
        prep.trim_padding()
        assert prep.past_key_values.get_seq_length() == prompt_len
        logits_a.append(out.logits[:, prompt_len - 1].float().cpu())
        for step in range(new_tokens):
            tokens.append(int(logits_a[-1].argmax()))
            pos = prompt_len + step
            out = model(input_ids=torch.tensor([[tokens[-1]]], device=DEV), past_key_values=prep.past_key_values,
                        cache_position=torch.tensor([pos], device=DEV), use_cache=True)
            logits_a.append(out.logits[:, -1].float().cpu())
        assert prep.past_key_values.get_seq_length() == prompt_len + new_tokens
        assert len(prep.past_key_values) == layers

    # ---------------- run B: same weights, attention computed by the CPU oracle over a plain dynamic cache
    _ORACLE_STATE.update(config=prep.config, real_q_len=prompt_len, pick_splits=get_extension().decode_pick_splits)
    model.config._attn_implementation = "thrift_oracle_test"
    cache_b = transformers.DynamicCache(config=model.config)
    logits_b = []
    with torch.no_grad():
        out = model(input_ids=prep.input_ids, past_key_values=cache_b, cache_position=prep.cache_position, use_cache=True)
        cache_b.crop(prompt_len)
        logits_b.append(out.logits[:, prompt_len - 1].float().cpu())
        _ORACLE_STATE["real_q_len"] = None
        for step in range(new_tokens):
            pos = prompt_len + step
            out = model(input_ids=torch.tensor([[tokens[step]]], device=DEV), past_key_values=cache_b,
                        cache_position=torch.tensor([pos], device=DEV), use_cache=True)
            logits_b.append(out.logits[:, -1].float().cpu())

    for a, b in zip(logits_a, logits_b):
        scale = b.abs().max().item()
        assert (a - b).abs().max().item() <= 0.02 * scale + 1e-3, ((a - b).abs().max().item(), scale)
        assert torch.nn.functional.cosine_similarity(a, b).item() > 0.9995


def test_llama_prefill_and_decode_through_the_hook():
    _hook_against_oracle(_tiny_llama, "thrift_hf_test", 0.25, 512, 300, 3, 20, 2)


def test_llama_prefill_and_decode_through_the_hook_over_a_paged_cache():
    """The same run with the cache in page pools: prompt padding cropped inside a page, decode through the page table."""
    _hook_against_oracle(_tiny_llama, "thrift_hf_test_paged", 0.25, 512, 300, 3, 20, 2, paged=True)


def _llama3_8b_shaped(name):
    """Two decoder layers with the Llama-3-8B shape: d_model 4096, 32 q / 8 kv heads x 128, SwiGLU 14336,
    RoPE theta 5e5, vocab 128256, fp16, random init."""
    cfg = transformers.LlamaConfig(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=2,
                                   num_attention_heads=32, num_key_value_heads=8, head_dim=128, rope_theta=500000.0,
                                   max_position_embeddings=8192, tie_word_embeddings=False)
    cfg._attn_implementation = name
    torch.manual_seed(0)
    with torch.device(DEV):
        return transformers.LlamaForCausalLM(cfg).half().eval()


def test_llama3_8b_shaped_layers_through_the_hook():
    """The Llama-3-8B layer shape, a 4096-token prompt (no padding) and three decode steps, NVFP4 with the top 10 %
    of the key blocks in fp16: logits against the same weights with the CPU oracle as the attention function."""
    _hook_against_oracle(_llama3_8b_shaped, "thrift_hf_8b_shape", 0.10, 128256, 4096, 3, 0, 2)


def test_hook_rejects_what_the_kernels_cannot_serve():
    name = register_transformers_attention(TransformersAttentionConfig(name="thrift_hf_reject"))
    module = type("M", (), {})()
    module.config = type("C", (), {"_attn_implementation": name})()
    module.training = False
    module.is_causal = True
    q = torch.randn(1, 4, 100, 128, device=DEV).half()
    with pytest.raises(RuntimeError, match="query length must be divisible by 64"):
        hf.thriftattention_forward(module, q, q[:, :2], q[:, :2], None)
    q = torch.randn(1, 4, 128, 128, device=DEV).half()
    with pytest.raises(RuntimeError, match="1/sqrt"):
        hf.thriftattention_forward(module, q, q[:, :2], q[:, :2], None, scaling=1.0)
    out, weights = hf.thriftattention_forward(module, q, q[:, :2].contiguous(), q[:, :2].contiguous(), None,
                                              scaling=128 ** -0.5)
    assert out.shape == (1, 128, 4, 128) and weights is None and torch.isfinite(out).all()




@pytest.mark.parametrize("paged", [False, True])
def test_whole_model_decode_step_replays_from_one_cuda_graph(monkeypatch, paged):
    """Device-length mode of the cache: ONE CUDA graph holds a single-token forward pass of the whole model (embedding,
    every layer's projections, cache append and attention through the registered function, head, arg-max fed back as
    the next input) and is replayed per token.  The logits of every step equal, bit for bit, those of the eager loop
    over a second cache (Python-side lengths) that runs the attention kernel with the same chain count."""
    from thriftattention_b200 import _C

    name = register_transformers_attention(TransformersAttentionConfig(name="thrift_graph_test", fraction=0.25))
    model = _tiny_llama(name)
    prompt_len, new_tokens, chains = 300, 100, 2
    ids = torch.randint(0, 512, (1, prompt_len), generator=torch.Generator().manual_seed(3)).to(DEV)
    hkv = model.config.num_key_value_heads
    for pages in range(1, 16):
        monkeypatch.setitem(_C._decode_step_splits, (hkv, pages), min(chains, pages))

    def prefill():
        prep = prepare_transformers_generation_cache(model, ids, max_new_tokens=new_tokens + 8, paged=paged)
        with prep.activate():
            out = model(input_ids=prep.input_ids, past_key_values=prep.past_key_values, cache_position=prep.cache_position,
                        use_cache=True, logits_to_keep=1)
            prep.trim_padding()
        return prep, out.logits[:, -1].argmax(-1, keepdim=True)

    with torch.no_grad():
        # eager loop, lengths in Python
        prep, tok = prefill()
        want = []
        with prep.activate():
            for step in range(new_tokens):
                pos = torch.tensor([prompt_len + step], device=DEV)
                out = model(input_ids=tok, past_key_values=prep.past_key_values, cache_position=pos,
                            position_ids=pos.view(1, 1), use_cache=True)
                want.append(out.logits[0, -1].clone())
                tok = out.logits[:, -1].argmax(-1, keepdim=True)

        # graph loop, length on the GPU
        prep, tok = prefill()
        cache = prep.past_key_values
        cache.enable_device_length(splits=chains)
        static_tok = tok.clone()
        logits_buf = torch.zeros(512, device=DEV, dtype=torch.float16)

        def step():
            pos = cache.device_positions()
            out = model(input_ids=static_tok, past_key_values=cache, cache_position=pos, position_ids=pos.view(1, 1),
                        use_cache=True)
            logits_buf.copy_(out.logits[0, -1])
            static_tok.copy_(out.logits[:, -1].argmax(-1, keepdim=True))
            cache.advance_device_length()

        got = []
        with prep.activate():
            step()                                   # eager, in device-length mode: libraries warm, first token
            got.append(logits_buf.clone())
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            for _ in range(new_tokens - 1):
                graph.replay()
                got.append(logits_buf.clone())
        assert cache.disable_device_length() == prompt_len + new_tokens
    for i, (a, b) in enumerate(zip(want, got)):
        assert torch.equal(a, b), f"decode step {i}"
    _C.decode_status(torch.device(DEV))

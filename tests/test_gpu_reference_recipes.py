"""The reference's own CUDA acceptance recipes, run through the drop-in operator module at head_dim 64:
cosine similarity above 0.95 against fp32 SDPA for pure-FP4 and for mixed attention with every block selected,
decode and tiled, NVFP4 and MXFP4, fp16 and bf16, contexts from 4096 to 131072 tokens
(tests/test_cuda_bf16_correctness.py:42-122 and tests/test_cuda_mxfp4_correctness.py:42-125 of the reference:
q, k, v = randn * 0.25, seeds 0 / 1 / 3, 4 q / 2 kv heads for decode, 2 q / 1 kv head for the tiled kernels)."""
import pytest
import torch
import torch.nn.functional as F

from thriftattention_b200._extension import get_extension

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
CONTEXTS = (4096, 8192, 32768, 131072)
DTYPES = (torch.float16, torch.bfloat16)


def _cos(a, b):
    return F.cosine_similarity(a.float().flatten(), b.float().flatten(), dim=0).item()


def _inputs(seed, dtype, q_heads, kv_heads, q_len, kv_len, d=64):
    torch.manual_seed(seed)
    mk = lambda h, s: (torch.randn(1, h, s, d, device=DEV, dtype=dtype) * 0.25).contiguous()
    return mk(q_heads, q_len), mk(kv_heads, kv_len), mk(kv_heads, kv_len)


def _pack(ext, fmt, q, k, v, bf16, permute_k):
    q4, qs = getattr(ext, f"{fmt}_quantize")(q, bf16)
    k4, ks = getattr(ext, f"{fmt}_quantize_permuted" if permute_k else f"{fmt}_quantize")(k, bf16)
    v4, vs = getattr(ext, f"{fmt}_quantize_transposed")(v, bf16)
    return q4, k4, v4, qs, ks, vs


@pytest.mark.parametrize("fmt,seed", [("nvfp4", 0), ("mxfp4", 3)])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kv_len", CONTEXTS)
def test_single_query_recipe(fmt, seed, dtype, kv_len):
    ext = get_extension()
    bf16 = dtype == torch.bfloat16
    q, k, v = _inputs(seed, dtype, 4, 2, 1, kv_len)
    qg = q.reshape(1, 2, 2, 64).contiguous()
    packed = _pack(ext, fmt, qg, k, v, bf16, permute_k=False)
    fp4 = getattr(ext, f"fp4_attention_single_query_{fmt}_packed")(*packed, bf16).reshape(1, 4, 1, 64)
    blocks = kv_len // 64
    k_mean = k.reshape(1, 2, blocks, 64, 64).float().mean(dim=3).to(dtype).contiguous()
    selected = ext.single_query_key_mean_topk(qg, k_mean, blocks, blocks, bf16)        # every block, ranked
    assert selected.shape == (2, blocks) and sorted(selected[0].tolist()) == list(range(blocks))
    mixed = getattr(ext, f"thrift_attention_single_query_{fmt}_packed")(qg, k, v, selected, *packed, bf16).reshape(1, 4, 1, 64)
    ref = F.scaled_dot_product_attention(q.float(), k.float().repeat_interleave(2, 1), v.float().repeat_interleave(2, 1))
    assert _cos(fp4, ref) > 0.95
    assert _cos(mixed, ref) > 0.95
    # with every page in 16 bits the mixed result is far closer than the FP4 one
    assert _cos(mixed, ref) > 0.999


@pytest.mark.parametrize("fmt,seed", [("nvfp4", 1), ("mxfp4", 3)])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kv_len", CONTEXTS)
def test_tiled_recipe(fmt, seed, dtype, kv_len):
    ext = get_extension()
    bf16 = dtype == torch.bfloat16
    q, k, v = _inputs(seed, dtype, 2, 1, kv_len, kv_len)
    packed = _pack(ext, fmt, q, k, v, bf16, permute_k=True)
    fp4 = getattr(ext, f"fp4_attention_causal_{fmt}_packed")(*packed, bf16)
    blocks = kv_len // 64
    selected = torch.arange(blocks, device=DEV, dtype=torch.int32).view(1, 1, blocks).expand(2, blocks, blocks).contiguous()
    mixed = getattr(ext, f"thrift_attention_causal_{fmt}_packed")(q, k, v, selected, *packed, bf16)
    # fp32 SDPA of a 131072 x 131072 problem is done in row chunks to bound its memory
    kf, vf = k.float().repeat_interleave(2, 1), v.float().repeat_interleave(2, 1)
    step = 8192
    cos_fp4 = cos_mixed = 0.0
    dot = [0.0, 0.0]
    nrm = [0.0, 0.0, 0.0]
    for r0 in range(0, kv_len, step):
        r1 = min(r0 + step, kv_len)
        mask = torch.ones(r1 - r0, r1, device=DEV, dtype=torch.bool).tril(diagonal=r0)
        ref = F.scaled_dot_product_attention(q[:, :, r0:r1].float(), kf[:, :, :r1], vf[:, :, :r1], attn_mask=mask)
        for idx, out in enumerate((fp4, mixed)):
            dot[idx] += (out[:, :, r0:r1].float() * ref).sum().item()
        nrm[0] += fp4[:, :, r0:r1].float().square().sum().item()
        nrm[1] += mixed[:, :, r0:r1].float().square().sum().item()
        nrm[2] += ref.square().sum().item()
    cos_fp4 = dot[0] / (nrm[0] * nrm[2]) ** 0.5
    cos_mixed = dot[1] / (nrm[1] * nrm[2]) ** 0.5
    assert cos_fp4 > 0.95 and cos_mixed > 0.95
    assert cos_mixed > 0.999


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_mean_topk_recipe(dtype):
    """Three key blocks along one channel: the ranking is exact (tests/test_cuda_bf16_correctness.py:125-139)."""
    ext = get_extension()
    q_mean = torch.zeros(1, 1, 1, 64, device=DEV, dtype=dtype)
    q_mean[..., 0] = 1.0
    k_mean = torch.zeros(1, 1, 8, 64, device=DEV, dtype=dtype)
    k_mean[0, 0, :, 0] = torch.arange(8, device=DEV, dtype=dtype)
    got = ext.block_mean_topk(q_mean, k_mean, 3, False, dtype == torch.bfloat16)
    assert got.cpu().tolist() == [[[7, 6, 5]]]

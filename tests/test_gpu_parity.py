"""GPU parity tests (B200): every CUDA entry point against the CPU oracle on identical seeded
inputs, through the C ABI.  Bit-exact for codes, scales, statistics and indices; attention within
max-abs 2e-3 / mean-abs 2e-4 for fp16 outputs (one bf16 ulp, 2^-7 relative, for bf16 outputs)."""
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

FP16_MAX_ABS, MEAN_ABS = 2e-3, 2e-4


def _tol(dtype, ref):
    if dtype == torch.bfloat16:
        return max(FP16_MAX_ABS, 2.0 ** -7 * float(ref.float().abs().max()))
    return FP16_MAX_ABS


def _ext():
    from thriftattention_b200._extension import get_extension

    return get_extension()


def _u8(t):
    return t.view(torch.uint8)


# ------------------------------------------------------------------------------------ quantisers
LAYOUTS = [("plain", "quantize"), ("permuted", "quantize_permuted"), ("transposed", "quantize_transposed"),
           ("transposed_permuted", "quantize_transposed_permuted")]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
@pytest.mark.parametrize("layout,op", LAYOUTS)
@pytest.mark.parametrize("shape", [(2, 3, 200, 128), (1, 2, 256, 64), (1, 1, 64, 128)])
def test_quantiser_bit_exact(cuda_device, dtype, fmt, layout, op, shape):
    torch.manual_seed(0)
    x = torch.randn(*shape)
    x[0, 0, :5] = 0.0                       # all-zero groups -> scale 0, codes 0
    x[0, -1, 7] *= 1000.0                   # saturates the scale range
    x[0, -1, 9] *= 1e-4
    x[0, 0, 11, ::2] = -0.0
    x = x.to(dtype)
    codes_ref, scale_ref = oracle.quantize(x, fmt, layout)
    codes, scale = getattr(_ext(), f"{fmt}_{op}")(x.to(cuda_device), dtype == torch.bfloat16)
    assert codes.shape == codes_ref.shape and scale.shape == scale_ref.shape
    assert scale.dtype == (torch.float8_e8m0fnu if fmt == "mxfp4" else torch.float8_e4m3fn)
    assert torch.equal(codes.cpu(), codes_ref)
    assert torch.equal(_u8(scale).cpu(), _u8(scale_ref))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
@pytest.mark.parametrize("k_permuted", [True, False])
@pytest.mark.parametrize("hq,hkv,sq,skv,d", [(4, 2, 200, 200, 128), (2, 2, 64, 320, 64), (8, 1, 1, 1000, 128)])
def test_one_launch_qkv_quantiser_bit_exact(cuda_device, dtype, fmt, k_permuted, hq, hkv, sq, skv, d):
    """The fused launch against the oracle, tensor by tensor (ragged lengths, GQA, a single query row)."""
    from thriftattention_b200 import _C

    g = torch.Generator().manual_seed(3)
    q = torch.randn(2, hq, sq, d, generator=g).to(dtype)
    k = torch.randn(2, hkv, skv, d, generator=g).to(dtype)
    v = torch.randn(2, hkv, skv, d, generator=g).to(dtype)
    k[0, 0, :3] = 0.0
    v[1, -1, 5] *= 1000.0
    got = _C.quantize_qkv(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), is_mx=fmt == "mxfp4",
                          is_bf16=dtype == torch.bfloat16, k_permuted=k_permuted)
    want = [oracle.quantize(q, fmt, "plain"), oracle.quantize(k, fmt, "permuted" if k_permuted else "plain"),
            oracle.quantize(v, fmt, "transposed")]
    for i, (codes_ref, scale_ref) in enumerate(want):
        assert torch.equal(got[i].cpu(), codes_ref), f"codes of tensor {i}"
        assert torch.equal(_u8(got[3 + i]).cpu(), _u8(scale_ref)), f"scales of tensor {i}"


def test_quantiser_e2m1_ties_and_saturation(cuda_device):
    # values that sit exactly on e2m1 rounding ties once divided by a power-of-two scale
    base = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0])
    x = base.repeat(1, 1, 64, 8).reshape(1, 1, 64, 128).half()
    for fmt in ("nvfp4", "mxfp4"):
        c_ref, s_ref = oracle.quantize(x, fmt, "plain")
        c, s = getattr(_ext(), f"{fmt}_quantize")(x.to(cuda_device), False)
        assert torch.equal(c.cpu(), c_ref) and torch.equal(_u8(s).cpu(), _u8(s_ref))


def test_quantiser_idempotent_at_scale(cuda_device):
    """Size-independent property on a large tensor: quantising the dequantised tensor returns the same codes."""
    torch.manual_seed(1)
    x = torch.randn(1, 8, 32768, 128, device=cuda_device, dtype=torch.float16)
    ext = _ext()
    codes, scale = ext.nvfp4_quantize(x, False)
    lut = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], device=cuda_device)
    lo, hi = lut[(codes & 15).long()], lut[(codes >> 4).long()]
    deq = torch.stack([lo, hi], -1).reshape(x.shape) * scale.float().repeat_interleave(16, dim=-1)
    codes2, scale2 = ext.nvfp4_quantize(deq.half(), False)
    assert torch.equal(_u8(scale2), _u8(scale))
    same = (codes2 == codes) | ((codes2 & 0x77) == (codes & 0x77))  # the sign of a zero code may differ
    assert bool(same.all())
    err = (deq - x.float()).abs().amax() / x.float().abs().amax()
    assert float(err) < 0.2


# ------------------------------------------------------------------------------------ statistics + selection
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("block", [64, 128])
def test_block_stats_and_prefill_selection_bit_exact(cuda_device, dtype, block):
    torch.manual_seed(2)
    q = torch.randn(1, 8, 2048, 128).to(dtype)
    k = torch.randn(1, 2, 2048, 128).to(dtype)
    ext = _ext()
    qm, = oracle.block_stats(q, block, ("mean",))
    km, kmin, kmax = oracle.block_stats(k, block, ("mean", "min", "max"))
    gqm, _, _ = ext.block_stats(q.to(cuda_device), block, mean=True)
    gkm, gkmin, gkmax = ext.block_stats(k.to(cuda_device), block, mean=True, minmax=True)
    for a, b in ((gqm, qm), (gkm, km), (gkmin, kmin), (gkmax, kmax)):
        assert torch.equal(a.cpu(), b)
    nk = 2048 // block
    bf = dtype == torch.bfloat16
    for causal in (True, False):
        for top_k, sink, local in ((3, 0, 0), (5, 1, 2), (nk, 0, 0)):
            ref = oracle.select_prefill(qm, kmin, kmax, k=top_k, causal=causal, sink=sink, local=local)
            got = ext.select_prefill_blocks(gqm, gkmin, gkmax, top_k, causal, bf, sink, local)
            assert torch.equal(got.cpu(), ref)
            ref = oracle.select_prefill(qm, km, None, k=top_k, causal=causal, sink=sink, local=local)
            got = ext.select_prefill_blocks(gqm, gkm, None, top_k, causal, bf, sink, local)
            assert torch.equal(got.cpu(), ref)
    # reference-named operators, K statistics expanded per Q head as the reference passes them
    exp = lambda t: t.repeat_interleave(4, dim=1).contiguous()
    got = ext.quest_block_topk(gqm, exp(gkmin), exp(gkmax), 4, True, bf)
    assert torch.equal(got.cpu(), oracle.select_prefill(qm, kmin, kmax, k=4, causal=True))
    got = ext.block_mean_topk(gqm, exp(gkm), 4, True, bf)
    assert torch.equal(got.cpu(), oracle.select_prefill(qm, km, None, k=4, causal=True))
    sel = oracle.select_prefill(qm, kmin, kmax, k=5, causal=True)
    assert torch.equal(ext.pack_topk_mask(sel.to(cuda_device), nk).cpu(), oracle.pack_mask(sel, nk))


def test_prefill_selection_with_ties(cuda_device):
    """Exact score ties take the reference's tie-break (smallest bit-reversal of idx mod 32, then idx div 32):
    a few ties inside the candidate set (duplicated key blocks), and everything tied (zero queries, as the
    padded rows of a prompt are), which exceeds the candidate cap and takes the arg-max rounds."""
    torch.manual_seed(23)
    ext = _ext()
    nq = nk = 640
    qm = torch.randn(1, 2, nq, 128).half()
    km = torch.randn(1, 1, nk, 128).half()
    km[:, :, 100:140] = km[:, :, 300:340]                    # 40 exact duplicates
    km[:, :, 500:520] = km[:, :, 20:21]                      # a block repeated 20 times
    qm[:, :, 600:] = 0                                       # rows whose scores are all zero
    qm[:, 1, 10] = 0
    for k, causal in ((20, True), (64, False), (300, True)):
        ref = oracle.select_prefill(qm, km, None, k=k, causal=causal)
        got = ext.select_prefill_blocks(qm.to(cuda_device), km.to(cuda_device), None, k, causal, False)
        assert torch.equal(got.cpu(), ref)
        lo, hi = km - 0.5, km + 0.5
        ref = oracle.select_prefill(qm, lo, hi, k=k, causal=causal, sink=1, local=1)
        got = ext.select_prefill_blocks(qm.to(cuda_device), lo.to(cuda_device), hi.to(cuda_device), k, causal, False, 1, 1)
        assert torch.equal(got.cpu(), ref)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_decode_selection_bit_exact(cuda_device, dtype):
    torch.manual_seed(3)
    ext = _ext()
    bf = dtype == torch.bfloat16
    qg = torch.randn(2, 2, 4, 128).to(dtype)
    k = torch.randn(2, 2, 8192, 128).to(dtype)
    km, kmin, kmax = oracle.block_stats(k, 64, ("mean", "min", "max"))
    dq, dkm, dkmin, dkmax = (t.to(cuda_device) for t in (qg, km, kmin, kmax))
    for top_k, sink, local, nk in ((6, 0, 0, 60), (6, 2, 3, 128), (13, 0, 0, 128), (40, 4, 16, 128)):
        ref = oracle.select_decode(qg, kmin, kmax, k=top_k, num_kv_blocks=nk, sink=sink, local=local)
        got = ext.select_decode_blocks(dq, dkmin, dkmax, top_k, nk, bf, sink, local)
        assert torch.equal(got.cpu(), ref)
        ref = oracle.select_decode(qg, km, None, k=top_k, num_kv_blocks=nk, sink=sink, local=local)
        got = ext.select_decode_blocks(dq, dkm, None, top_k, nk, bf, sink, local)
        assert torch.equal(got.cpu(), ref)
    assert torch.equal(ext.single_query_quest_topk(dq, dkmin, dkmax, 5, 100, bf).cpu(),
                       oracle.select_decode(qg, kmin, kmax, k=5, num_kv_blocks=100))
    assert torch.equal(ext.single_query_key_mean_topk(dq, dkm, 5, 100, bf).cpu(),
                       oracle.select_decode(qg, km, None, k=5, num_kv_blocks=100))
    topk = torch.empty(4, 5, dtype=torch.int32, device=cuda_device)
    ws_s = torch.empty(4, 2, 5, device=cuda_device)
    ws_i = torch.empty(4, 2, 5, dtype=torch.int32, device=cuda_device)
    done = torch.zeros(4, dtype=torch.int32, device=cuda_device)
    ext.single_query_key_mean_topk_into(dq, dkm, topk, ws_s, ws_i, done, 100, bf)
    assert torch.equal(topk.cpu(), oracle.select_decode(qg, km, None, k=5, num_kv_blocks=100))


def _stats(nk, dtype, seed, hkv=2):
    g = torch.Generator().manual_seed(seed)
    km = torch.randn(1, hkv, nk, 128, generator=g)
    ch = torch.randperm(128, generator=g)[:4]
    km[..., ch] *= 10.0                                       # key outlier channels
    half = torch.rand(1, hkv, nk, 128, generator=g) * 0.5
    return km.to(dtype), (km - half).to(dtype), (km + half).to(dtype), g


def _check_decode_selection(ext, dev, qg, km, kmin, kmax, k, nk, sink, local, bf):
    """Two-pass kernel path == oracle == the kernel's exact path.  A query group above 8 heads always takes the
    exact path; repeating heads does not change the maximum over the group, so the same selection must come out."""
    reps = {1: 9, 2: 5, 4: 3, 8: 2}[qg.size(2)]
    q_wide = qg.repeat(1, 1, reps, 1)
    dq, dq_wide = qg.to(dev), q_wide.to(dev)
    for a, b in ((kmin, kmax), (km, None)):
        ref = oracle.select_decode(qg, a, b, k=k, num_kv_blocks=nk, sink=sink, local=local)
        da, db = a.to(dev), None if b is None else b.to(dev)
        got = ext.select_decode_blocks(dq, da, db, k, nk, bf, sink, local)
        assert torch.equal(got.cpu(), ref), f"two-pass selection differs from the oracle (quest={b is not None})"
        exact = ext.select_decode_blocks(dq_wide, da, db, k, nk, bf, sink, local)
        assert torch.equal(exact.cpu(), ref), f"exact selection differs from the oracle (quest={b is not None})"


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("group", [1, 4, 8])
@pytest.mark.parametrize("nk", [256, 1024, 2048])
def test_decode_selection_two_pass_bit_exact(cuda_device, dtype, group, nk):
    """The long-context selection path (approximate tensor-core pass, exact re-scoring of the candidates) that the
    2048-page decode configurations run: index- and order-equal to the oracle (shared/block_selection.cu:339-441)
    on eight seeds, with the 10 % + 4 sink + 16 local and the fixed-53 configurations."""
    ext = _ext()
    bf = dtype == torch.bfloat16
    for seed in range(8):
        km, kmin, kmax, g = _stats(nk, dtype, 100 + seed)
        qg = torch.randn(1, 2, group, 128, generator=g).to(dtype)
        k10 = oracle.resolve_top_k(nk, causal=False, fraction=0.1)
        _check_decode_selection(ext, cuda_device, qg, km, kmin, kmax, k10, nk, 4, 16, bf)
        _check_decode_selection(ext, cuda_device, qg, km, kmin, kmax, min(53, nk // 4), nk, 0, 0, bf)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_decode_selection_two_pass_adversarial(cuda_device, dtype):
    """Rows built to sit on the pruning bound of the two-pass path: exact ties that straddle the k-th place,
    all-zero queries (every page ties), one huge outlier channel (a wide error bound) and more tied candidates
    than the exact re-scoring holds (falls back to scoring every page)."""
    ext = _ext()
    bf = dtype == torch.bfloat16
    nk, k = 2048, 205
    km, kmin, kmax, g = _stats(nk, dtype, 7)
    qg = torch.randn(1, 2, 4, 128, generator=g).to(dtype)

    def run(qq, a_mean, a_min, a_max, kk=k, sink=4, local=16):
        _check_decode_selection(ext, cuda_device, qq, a_mean, a_min, a_max, kk, nk, sink, local, bf)

    # (1) duplicated pages around the k-th place: find the oracle's ranking, then copy the page at rank k-1 over
    #     40 pages spread over the sequence, so that exact ties straddle the cut
    for a_min, a_max in ((kmin, kmax), (km, km)):
        ref = oracle.select_decode(qg, a_min, a_max, k=k, num_kv_blocks=nk)
        for h in range(2):
            pivot = int(ref[h, k - 1])
            idx = torch.arange(37, nk - 20, 50)
            for t in (km, kmin, kmax):
                t[0, h, idx] = t[0, h, pivot].clone()
    run(qg, km, kmin, kmax)
    run(qg, km, kmin, kmax, kk=53, sink=0, local=0)
    # (2) all-zero query: every score is +0, every page ties, the candidate set overflows
    run(torch.zeros_like(qg), km, kmin, kmax)
    # (3) one huge channel in q and in the statistics
    q_big = qg.clone()
    q_big[..., 5] = 200.0
    k_big, kmin_big, kmax_big = km.clone(), kmin.clone(), kmax.clone()
    for t in (k_big, kmin_big, kmax_big):
        t[..., 5] *= 100.0
    run(q_big, k_big, kmin_big, kmax_big)
    # (4) 700 identical pages that all rank first: more candidates than the exact pass holds
    k_dup, kmin_dup, kmax_dup = km.clone(), kmin.clone(), kmax.clone()
    ref = oracle.select_decode(qg, kmin, kmax, k=1, num_kv_blocks=nk)
    for h in range(2):
        top = int(ref[h, 0])
        idx = torch.randperm(nk, generator=g)[:700]
        for t in (k_dup, kmin_dup, kmax_dup):
            t[0, h, idx] = t[0, h, top].clone()
    run(qg, k_dup, kmin_dup, kmax_dup)
    # (5) negative zero and sign mixtures in q
    q_sign = qg.clone()
    q_sign[..., ::3] = -0.0
    run(q_sign, km, kmin, kmax)


def test_reference_known_answers_on_gpu(cuda_device):
    """The reference tests' small known answers (tests/test_selection.py:37-129,
    tests/test_cuda_bf16_correctness.py:125-139), embedded in head_dim 64."""
    ext = _ext()

    def pad(t):
        out = torch.zeros(*t.shape[:-1], 64, dtype=t.dtype)
        out[..., : t.shape[-1]] = t
        return out.to(cuda_device)

    q = pad(torch.tensor([[[[1.0, -1.0], [1.0, -1.0], [-1.0, 1.0], [-1.0, 1.0]]]], dtype=torch.float16))
    k = pad(torch.tensor([[[[2.0, -4.0], [1.0, -3.0], [-3.0, 5.0], [-2.0, 6.0]]]], dtype=torch.float16))
    qm, _, _ = ext.block_stats(q, 2, mean=True)
    _, lo, hi = ext.block_stats(k, 2, minmax=True)
    assert ext.quest_block_topk(qm, lo, hi, 2, True, False).tolist() == [[[0, -1], [1, 0]]]
    q = pad(torch.tensor([[[[1.0, -2.0]]]], dtype=torch.float16)).reshape(1, 1, 1, 64)
    k = pad(torch.tensor([[[[4.0, -3.0], [2.0, -1.0], [1.0, -1.0], [0.0, 0.0], [3.0, 2.0], [3.0, 1.0]]]], dtype=torch.float16))
    _, lo, hi = ext.block_stats(k, 2, minmax=True)
    assert ext.single_query_quest_topk(q, lo, hi, 1, 3, False).tolist() == [[0]]
    q = torch.zeros(1, 1, 1, 64, dtype=torch.float16, device=cuda_device)
    q[..., 0] = 1.0
    km = torch.zeros(1, 1, 8, 64, dtype=torch.float16, device=cuda_device)
    km[0, 0, :, 0] = torch.arange(8, dtype=torch.float16)
    assert ext.single_query_key_mean_topk(q, km, 3, 8, False).tolist() == [[7, 6, 5]]


def test_local_windows_on_gpu(cuda_device):
    ext = _ext()
    for flat, nq, nk, k, causal in ((2, 5, 5, 3, True), (2, 5, 5, 3, False), (6, 4, 7, 5, True), (1, 6, 3, 3, True), (1, 8, 8, 8, False)):
        q = torch.empty(1, flat, nq * 64, 64, dtype=torch.float16, device=cuda_device)
        assert torch.equal(ext.local_block_topk(q, nk, k, causal, 64).cpu(), oracle.local_prefill(flat, nq, nk, k, causal))
    qg = torch.empty(1, 3, 2, 64, dtype=torch.float16, device=cuda_device)
    assert ext.single_query_local_topk(qg, 3, 7).tolist() == [[4, 5, 6]] * 3


# ------------------------------------------------------------------------------------ prefill attention
def _prefill_case(dev, dtype, fmt, block, S, hq, hkv, frac, causal, kperm, seed=0, outlier=False, sq=None, d=128):
    torch.manual_seed(seed)
    sq = S if sq is None else sq
    q = torch.randn(1, hq, sq, d)
    k = torch.randn(1, hkv, S, d)
    v = torch.randn(1, hkv, S, d)
    if outlier:
        k[:, :, :, torch.randperm(d)[:4]] *= 10
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    bf, mx = dtype == torch.bfloat16, fmt == "mxfp4"
    ext = _ext()
    nk = S // block
    top_k = oracle.resolve_top_k(nk, causal=causal, fraction=frac) if frac > 0 else 0
    sel = None
    if top_k:
        qm, = oracle.block_stats(q, block, ("mean",))
        kmin, kmax = oracle.block_stats(k, block, ("min", "max"))
        sel = oracle.select_prefill(qm, kmin, kmax, k=top_k, causal=causal)
    ref = oracle.prefill_attention(q, k, v, sel, fmt=fmt, block=block, causal=causal)
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    q4, qs = getattr(ext, f"{fmt}_quantize")(qd, bf)
    k4, ks = getattr(ext, f"{fmt}_quantize_permuted" if kperm else f"{fmt}_quantize")(kd, bf)
    v4, vs = getattr(ext, f"{fmt}_quantize_transposed")(vd, bf)
    out = ext.prefill_attention(qd, kd, vd, sel.to(dev) if sel is not None else None, q4, k4, v4, qs, ks, vs,
                                causal=causal, is_mx=mx, is_bf16=bf, block_size=block, k_permuted=kperm, check_status=True)
    err = (out.float().cpu() - ref.float()).abs()
    assert not torch.isnan(out).any()
    assert err.max().item() <= _tol(dtype, ref), f"max abs {err.max().item()}"
    assert err.mean().item() <= MEAN_ABS
    return out, ref, (q, k, v)


PREFILL_CASES = [
    (torch.float16, "nvfp4", 128, 256, 1, 1, 0.0, True, False),
    (torch.float16, "nvfp4", 128, 256, 1, 1, 0.5, True, False),
    (torch.float16, "nvfp4", 128, 1024, 2, 1, 0.1, True, True),
    (torch.float16, "nvfp4", 64, 1024, 2, 1, 0.1, True, True),
    (torch.float16, "nvfp4", 64, 1024, 2, 1, 0.1, False, True),
    (torch.float16, "nvfp4", 64, 1024, 2, 1, 1.0, True, True),     # every block selected: pure 16-bit pass
    (torch.bfloat16, "nvfp4", 64, 1024, 2, 2, 0.25, True, True),
    (torch.float16, "mxfp4", 64, 1024, 4, 2, 0.1, True, True),
    (torch.bfloat16, "mxfp4", 128, 1024, 4, 2, 0.1, True, False),
    (torch.float16, "nvfp4", 64, 2048, 8, 8, 0.1, True, True),     # configuration 1 shape (8 q = 8 kv heads, 2048)
    (torch.float16, "nvfp4", 128, 4096, 8, 2, 0.1, True, True),    # several work items per CTA
    (torch.float16, "nvfp4", 64, 1088, 1, 1, 0.1, True, True),     # q_len not a multiple of the 128-row tile
]


@pytest.mark.parametrize("dtype,fmt,block,S,hq,hkv,frac,causal,kperm", PREFILL_CASES)
def test_prefill_attention_matches_oracle(cuda_device, dtype, fmt, block, S, hq, hkv, frac, causal, kperm):
    out, ref, (q, k, v) = _prefill_case(cuda_device, dtype, fmt, block, S, hq, hkv, frac, causal, kperm, outlier=(S >= 2048))
    # the reference's own bar: cosine similarity > 0.95 against fp32 SDPA (tests/test_cuda_bf16_correctness.py:84-85)
    if frac >= 0.1:
        g = hq // hkv
        sd = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float().repeat_interleave(g, 1),
                                                              v.float().repeat_interleave(g, 1), is_causal=causal)
        cos = torch.nn.functional.cosine_similarity(out.float().cpu().flatten(), sd.flatten(), dim=0)
        assert float(cos) > 0.95


@pytest.mark.parametrize("dtype,fmt,block,S,hq,hkv,frac,causal,kperm", [
    (torch.float16, "nvfp4", 64, 1024, 2, 1, 0.1, True, True),
    (torch.float16, "nvfp4", 64, 1024, 2, 1, 0.0, True, False),
    (torch.bfloat16, "nvfp4", 128, 1024, 4, 2, 0.25, True, False),
    (torch.float16, "mxfp4", 64, 1024, 4, 2, 0.1, True, True),
    (torch.bfloat16, "mxfp4", 64, 512, 2, 2, 0.5, False, False),
    (torch.float16, "nvfp4", 64, 4096, 4, 1, 0.1, True, True),
])
def test_prefill_attention_head_dim_64(cuda_device, dtype, fmt, block, S, hq, hkv, frac, causal, kperm):
    """The reference's own CUDA tests run at head_dim 64 (tests/test_cuda_bf16_correctness.py:42-122)."""
    _prefill_case(cuda_device, dtype, fmt, block, S, hq, hkv, frac, causal, kperm, d=64)


def _seeded_prefill_configs(n):
    rng = torch.Generator().manual_seed(2024)
    pick = lambda seq: seq[int(torch.randint(0, len(seq), (1,), generator=rng))]
    out = []
    for _ in range(n):
        hkv = pick((1, 2, 3))
        out.append((pick((torch.float16, torch.bfloat16)), pick(("nvfp4", "mxfp4")), pick((64, 128)),
                    128 * int(torch.randint(1, 11, (1,), generator=rng)), hkv * pick((1, 2, 4)), hkv,
                    pick((0.0, 0.1, 0.3, 1.0)), pick((True, False)), pick((True, False)), pick((64, 128))))
    return out


@pytest.mark.parametrize("idx,cfg", list(enumerate(_seeded_prefill_configs(16))))
def test_prefill_seeded_random_shapes(cuda_device, idx, cfg):
    """Sixteen configurations drawn from a fixed seed (dtype, format, block size, 128..1280 tokens, head counts,
    selected fraction, causal, K layout, head_dim), each against the oracle."""
    dtype, fmt, block, S, hq, hkv, frac, causal, kperm, d = cfg
    _prefill_case(cuda_device, dtype, fmt, block, S, hq, hkv, frac, causal, kperm, seed=100 + idx, outlier=idx % 2 == 0, d=d)


def test_prefill_noncausal_rectangular(cuda_device):
    _prefill_case(cuda_device, torch.float16, "nvfp4", 64, 1024, 2, 1, 0.1, False, True, sq=256)


def test_prefill_is_deterministic_and_reference_named_ops_agree(cuda_device):
    torch.manual_seed(4)
    ext = _ext()
    q = torch.randn(1, 4, 1024, 128, device=cuda_device).half()
    k = torch.randn(1, 2, 1024, 128, device=cuda_device).half()
    v = torch.randn(1, 2, 1024, 128, device=cuda_device).half()
    qm, _, _ = ext.block_stats(q, 64, mean=True)
    km, _, _ = ext.block_stats(k, 64, mean=True)
    sel = ext.block_mean_topk(qm, km, 3, True, False)
    packed = (ext.nvfp4_quantize(q)[0], ext.nvfp4_quantize_permuted(k)[0], ext.nvfp4_quantize_transposed(v)[0],
              ext.nvfp4_quantize(q)[1], ext.nvfp4_quantize_permuted(k)[1], ext.nvfp4_quantize_transposed(v)[1])
    a = ext.thrift_attention_causal_nvfp4_packed(q, k, v, sel, *packed, False)
    b = ext.thrift_attention_causal_nvfp4_packed(q, k, v, sel, *packed, False)
    assert torch.equal(a, b)
    empty = sel[:, :, :0].contiguous()
    c = ext.thrift_attention_causal_nvfp4_packed(q, k, v, empty, *packed, False)
    d = ext.fp4_attention_causal_nvfp4_packed(*packed, False)
    assert torch.equal(c, d)  # topk_count == 0 falls back to pure FP4 (bindings.cpp:525-528 of the reference)


def test_prefill_sequence_major_output(cuda_device):
    """out_seq_major writes [B, Sq, Hq, D] from the kernel epilogue: bit-identical to the transposed default."""
    import thriftattention_b200 as ta
    from thriftattention_b200.functional import attention_seq_major

    torch.manual_seed(8)
    ext = _ext()
    for d, b, hq, hkv, S in ((128, 2, 4, 2, 512), (64, 1, 6, 3, 320)):
        q = torch.randn(b, hq, S, d, device=cuda_device).half()
        k = torch.randn(b, hkv, S, d, device=cuda_device).half()
        v = torch.randn(b, hkv, S, d, device=cuda_device).half()
        qm, _, _ = ext.block_stats(q, 64, mean=True)
        km, _, _ = ext.block_stats(k, 64, mean=True)
        sel = ext.block_mean_topk(qm, km, 2, True, False)
        q4, qs = ext.nvfp4_quantize(q)
        k4, ks = ext.nvfp4_quantize_permuted(k)
        v4, vs = ext.nvfp4_quantize_transposed(v)
        for args in ((q, k, v, sel), (None, None, None, None)):
            kw = dict(causal=True, is_mx=False, block_size=64, k_permuted=True)
            plain = ext.prefill_attention(*args, q4, k4, v4, qs, ks, vs, **kw)
            major = ext.prefill_attention(*args, q4, k4, v4, qs, ks, vs, seq_major_out=True, **kw)
            assert major.shape == (b, S, hq, d) and major.is_contiguous()
            assert torch.equal(major, plain.transpose(1, 2))
        cfg = ta.AttentionConfig(fraction=0.25)
        assert torch.equal(attention_seq_major(q, k, v, config=cfg), ta.attention(q, k, v, config=cfg).transpose(1, 2))
    # one query token: the sequence-major result is a view of the grouped decode output
    q1 = torch.randn(2, 4, 1, 128, device=cuda_device).half()
    kk = torch.randn(2, 2, 256, 128, device=cuda_device).half()
    cfg = ta.AttentionConfig(fraction=0.5, causal=False)
    assert torch.equal(attention_seq_major(q1, kk, kk, config=cfg), ta.attention(q1, kk, kk, config=cfg).transpose(1, 2))


def test_attention_host_pipelines_head_groups(cuda_device):
    """Host tensors in, host tensor out, one KV-head group at a time on three streams: the result equals the
    device-resident call bit for bit, for every chunking."""
    import thriftattention_b200 as ta

    torch.manual_seed(14)
    q = torch.randn(2, 8, 512, 128).half().pin_memory()
    k = torch.randn(2, 4, 512, 128).half().pin_memory()
    v = torch.randn(2, 4, 512, 128).half().pin_memory()
    cfg = ta.AttentionConfig(selection="quest", fraction=0.25)
    want = ta.attention(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), config=cfg).cpu()
    for per_chunk in (1, 3, 4):
        got = ta.attention_host(q, k, v, config=cfg, device=cuda_device, kv_heads_per_chunk=per_chunk)
        torch.cuda.synchronize(cuda_device)
        assert got.is_pinned() and torch.equal(got, want)
    got = ta.attention_host(q, k, v, config=cfg, device=cuda_device, q_heads_per_chunk=1)   # one query head at a time
    torch.cuda.synchronize(cuda_device)
    assert torch.equal(got, want)
    with pytest.raises(ValueError, match="q_heads_per_chunk"):
        ta.attention_host(q, k, v, config=cfg, device=cuda_device, kv_heads_per_chunk=2, q_heads_per_chunk=1)
    out = torch.zeros_like(want).pin_memory()
    assert ta.attention_host(q, k, v, config=cfg, device=cuda_device, out=out) is out
    torch.cuda.synchronize(cuda_device)
    assert torch.equal(out, want)
    with pytest.raises(ValueError, match="host tensors"):
        ta.attention_host(q.to(cuda_device), k, v, config=cfg)


def test_public_attention_api(cuda_device):
    import thriftattention_b200 as ta

    torch.manual_seed(5)
    q = torch.randn(1, 4, 512, 128).half()
    k = torch.randn(1, 2, 512, 128).half()
    v = torch.randn(1, 2, 512, 128).half()
    for selection in ("block_mean", "quest", "local"):
        cfg = ta.AttentionConfig(selection=selection, top_k=2, block_size=64)
        out = ta.attention(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), config=cfg)
        if selection == "local":
            sel = oracle.local_prefill(4, 8, 8, 2, True)
        else:
            qm, = oracle.block_stats(q, 64, ("mean",))
            km, kmin, kmax = oracle.block_stats(k, 64, ("mean", "min", "max"))
            sel = oracle.select_prefill(qm, kmin, kmax, k=2, causal=True) if selection == "quest" else \
                oracle.select_prefill(qm, km, None, k=2, causal=True)
        ref = oracle.prefill_attention(q, k, v, sel, fmt="nvfp4", block=64, causal=True)
        err = (out.float().cpu() - ref.float()).abs()
        assert err.max().item() <= FP16_MAX_ABS and err.mean().item() <= MEAN_ABS
    out = ta.attention(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device),
                       config=ta.AttentionConfig(method="fp4", quant_format="mxfp4"))
    ref = oracle.prefill_attention(q, k, v, None, fmt="mxfp4", block=64, causal=True)
    assert (out.float().cpu() - ref.float()).abs().max().item() <= FP16_MAX_ABS
    with pytest.raises(ValueError, match="divisible"):
        ta.attention(q[:, :, :100].to(cuda_device), k.to(cuda_device), v.to(cuda_device))
    with pytest.raises(ValueError, match="CUDA"):
        ta.attention(q, k, v)


@pytest.mark.parametrize("S,top_k_expected", [(32768, 13), (131072, 53)])
def test_prefill_long_context_slice_matches_oracle(cuda_device, S, top_k_expected):
    """Configuration-2 shape (32q/8kv, 32768 tokens) and the benchmark's own (131072 tokens): 128-token blocks,
    top-10%, outlier keys.  The whole problem runs on the GPU, the oracle recomputes one q head's selection and
    slices of its rows."""
    import thriftattention_b200 as ta

    block = 128
    g = torch.Generator(device=cuda_device).manual_seed(0)
    q = torch.randn(1, 32, S, 128, device=cuda_device, dtype=torch.float16, generator=g)
    k = torch.randn(1, 8, S, 128, device=cuda_device, dtype=torch.float16, generator=g)
    v = torch.randn(1, 8, S, 128, device=cuda_device, dtype=torch.float16, generator=g)
    k[:, :, :, torch.tensor([3, 40, 77, 101], device=cuda_device)] *= 10
    cfg = ta.AttentionConfig(selection="quest", fraction=0.10, block_size=block, quant_format="nvfp4")
    out = ta.attention(q, k, v, config=cfg)
    top_k = oracle.resolve_top_k(S // block, causal=True, fraction=0.10)
    assert top_k == top_k_expected
    for head in (5, 30):
        qh, kh, vh = q[:, head:head + 1].cpu(), k[:, head // 4:head // 4 + 1].cpu(), v[:, head // 4:head // 4 + 1].cpu()
        qm, = oracle.block_stats(qh, block, ("mean",))
        kmin, kmax = oracle.block_stats(kh, block, ("min", "max"))
        sel = oracle.select_prefill(qm, kmin, kmax, k=top_k, causal=True)
        for lo in (0, S // 2, S - 256):
            ref = oracle.prefill_attention(qh, kh, vh, sel, fmt="nvfp4", block=block, causal=True, rows=(lo, lo + 256))
            err = (out[0, head, lo:lo + 256].float().cpu() - ref[0, 0, lo:lo + 256].float()).abs()
            assert err.max().item() <= FP16_MAX_ABS and err.mean().item() <= MEAN_ABS


@pytest.mark.parametrize("fmt,dtype,d,block,hq,hkv", [("mxfp4", torch.bfloat16, 128, 128, 32, 8), ("nvfp4", torch.float16, 64, 64, 8, 8)])
def test_prefill_long_context_slices_other_formats(cuda_device, fmt, dtype, d, block, hq, hkv):
    """32,768 tokens in the other format / type / head size / block size combinations: bf16 + MXFP4 with 128-token
    blocks (the long-context configuration's shape), and head_dim 64 with 64-token blocks and no query grouping (the
    reference's acceptance shape).  Oracle rows at the start, middle and end of one head."""
    import thriftattention_b200 as ta

    S = 32768
    g = torch.Generator(device=cuda_device).manual_seed(2)
    q = torch.randn(1, hq, S, d, device=cuda_device, dtype=torch.float32, generator=g).to(dtype)
    k = torch.randn(1, hkv, S, d, device=cuda_device, dtype=torch.float32, generator=g).to(dtype)
    v = torch.randn(1, hkv, S, d, device=cuda_device, dtype=torch.float32, generator=g).to(dtype)
    k[:, :, :, torch.tensor([1, 17, 33, 60], device=cuda_device)] *= 10
    cfg = ta.AttentionConfig(selection="quest", fraction=0.05, block_size=block, quant_format=fmt)
    out = ta.attention(q, k, v, config=cfg)
    top_k = oracle.resolve_top_k(S // block, causal=True, fraction=0.05)
    head = hq - 3
    grp = hq // hkv
    qh, kh, vh = q[:, head:head + 1].cpu(), k[:, head // grp:head // grp + 1].cpu(), v[:, head // grp:head // grp + 1].cpu()
    qm, = oracle.block_stats(qh, block, ("mean",))
    kmin, kmax = oracle.block_stats(kh, block, ("min", "max"))
    sel = oracle.select_prefill(qm, kmin, kmax, k=top_k, causal=True)
    for lo in (0, S // 2, S - 256):
        ref = oracle.prefill_attention(qh, kh, vh, sel, fmt=fmt, block=block, causal=True, rows=(lo, lo + 256))
        err = (out[0, head, lo:lo + 256].float().cpu() - ref[0, 0, lo:lo + 256].float()).abs()
        assert err.max().item() <= _tol(dtype, ref[0, 0, lo:lo + 256]) and err.mean().item() <= MEAN_ABS


def test_prefill_at_benchmark_size_scales_exactly_with_v(cuda_device):
    """Size-independent property at the benchmark's size (32q/8kv x 131072): V enters the result linearly and its
    block scales are floating point, so doubling V (a power of two: every scale byte moves by one exponent step,
    every code stays) must double the output values - exactly, except where an fp16 subnormal gets rounded."""
    import thriftattention_b200 as ta

    S = 131072
    g = torch.Generator(device=cuda_device).manual_seed(7)
    q = torch.randn(1, 32, S, 128, device=cuda_device, dtype=torch.float16, generator=g)
    k = torch.randn(1, 8, S, 128, device=cuda_device, dtype=torch.float16, generator=g)
    v = torch.randn(1, 8, S, 128, device=cuda_device, dtype=torch.float16, generator=g)
    cfg = ta.AttentionConfig(selection="quest", fraction=0.10, block_size=128, quant_format="nvfp4")
    out1 = ta.attention(q, k, v, config=cfg)
    out2 = ta.attention(q, k, v * 2, config=cfg)
    assert torch.isfinite(out1).all()
    # The only roundings that do not commute with the doubling are those of fp16 SUBNORMALS: the state rounded
    # between the two phases (and the output itself) where a value lies below 2^-14.  Such an element may move by one
    # subnormal step (2^-24, doubled: 2^-23), which in turn may flip the final rounding of its output by one ulp.
    diff = (out1.float() * 2 - out2.float()).abs()
    assert bool((diff <= 2.0 ** -22 + 2.0 ** -10 * out2.float().abs()).all())
    assert float((diff > 0).float().mean()) < 0.01


# ------------------------------------------------------------------------------------ decode attention
DECODE_CASES = [
    (torch.float16, "nvfp4", 1, 1, 4, 256, 0, 1, 128),
    (torch.float16, "nvfp4", 1, 1, 4, 256, 1, 1, 128),
    (torch.float16, "nvfp4", 2, 2, 8, 4096, 6, 5, 128),
    (torch.float16, "nvfp4", 1, 2, 1, 1024, 2, 3, 128),
    (torch.bfloat16, "nvfp4", 2, 2, 4, 1024, 3, 2, 128),
    (torch.float16, "mxfp4", 2, 2, 4, 1024, 3, 2, 128),
    (torch.bfloat16, "mxfp4", 2, 2, 4, 2048, 5, 4, 128),
    (torch.float16, "nvfp4", 2, 8, 4, 8192, 13, 7, 128),
    (torch.float16, "nvfp4", 1, 2, 16, 2048, 4, 2, 128),       # the largest query group
    (torch.bfloat16, "mxfp4", 1, 1, 12, 1024, 16, 1, 128),     # every page selected: 16-bit pages only
    (torch.float16, "nvfp4", 2, 2, 4, 1024, 3, 2, 64),         # head_dim 64
    (torch.bfloat16, "nvfp4", 1, 2, 8, 2048, 0, 3, 64),
    (torch.float16, "mxfp4", 2, 1, 4, 1024, 2, 2, 64),
    (torch.bfloat16, "mxfp4", 1, 2, 2, 512, 8, 1, 64),
]


def _seeded_decode_configs(n):
    rng = torch.Generator().manual_seed(4048)
    pick = lambda seq: seq[int(torch.randint(0, len(seq), (1,), generator=rng))]
    out = []
    for _ in range(n):
        pages = int(torch.randint(1, 40, (1,), generator=rng))
        out.append((pick((torch.float16, torch.bfloat16)), pick(("nvfp4", "mxfp4")), pick((1, 2, 3)), pick((1, 2)),
                    pick((1, 2, 3, 4, 5, 8, 12, 16)), pages * 64, min(pages, pick((0, 1, 3, 7, 40))),
                    min(pages, pick((1, 2, 3, 5))), pick((64, 128))))
    return out


@pytest.mark.parametrize("idx,cfg", list(enumerate(_seeded_decode_configs(16))))
def test_decode_seeded_random_shapes(cuda_device, idx, cfg):
    """Sixteen configurations drawn from a fixed seed (1..39 pages, any group size up to 16, ragged split counts,
    none / some / all pages selected), each against the oracle through the same check as the listed cases."""
    test_decode_attention_matches_oracle(cuda_device, *cfg)


def _to_page_pools(table, n_pool, k4, ks, v4, vs, k_hi, v_hi):
    """Scatters contiguous cache tensors into page pools addressed by ``table`` [B, pages] (64-token pages)."""
    B, hkv, S = k4.shape[0], k4.shape[1], k4.shape[2]
    pages = S // 64
    flat = table.reshape(-1).long()

    def rows(t):       # [B, hkv, S, X] -> pool [n_pool, hkv, 64, X]
        pool = torch.zeros(n_pool, hkv, 64, t.shape[-1], dtype=t.dtype, device=t.device)
        pool[flat] = t.reshape(B, hkv, pages, 64, -1).permute(0, 2, 1, 3, 4).reshape(B * pages, hkv, 64, -1)
        return pool

    def cols(t, per_page):   # [B, hkv, D, >= pages * per_page] -> pool [n_pool, hkv, D, per_page]
        D = t.shape[2]
        pool = torch.zeros(n_pool, hkv, D, per_page, dtype=t.dtype, device=t.device)
        pool[flat] = (t[..., :pages * per_page].reshape(B, hkv, D, pages, per_page).permute(0, 3, 1, 2, 4)
                      .reshape(B * pages, hkv, D, per_page))
        return pool

    group = k4.shape[-1] * 2 // ks.shape[-1]                     # elements per scale: D / scales per row
    return rows(k4), rows(ks), cols(v4, 32), cols(vs, 64 // group), rows(k_hi), rows(v_hi)


@pytest.mark.parametrize("dtype,fmt,B,hkv,G,S,top_k,splits,d", [
    (torch.float16, "nvfp4", 3, 2, 4, 2048, 5, 4, 128),
    (torch.bfloat16, "mxfp4", 2, 2, 8, 1024, 3, 0, 128),
    (torch.float16, "mxfp4", 2, 3, 2, 1024, 0, 2, 64),
    (torch.bfloat16, "nvfp4", 1, 2, 4, 4096, 64, 8, 64),
])
def test_paged_decode_equals_contiguous(cuda_device, dtype, fmt, B, hkv, G, S, top_k, splits, d):
    """Page pools behind a seeded random page table give bit-identical results to the contiguous cache (and so
    inherit its parity with the oracle): the table only changes where a page is fetched from."""
    torch.manual_seed(12)
    ext = _ext()
    bf, mx = dtype == torch.bfloat16, fmt == "mxfp4"
    q = torch.randn(B, hkv, G, d, device=cuda_device).to(dtype)
    k = torch.randn(B, hkv, S, d, device=cuda_device).to(dtype)
    v = torch.randn(B, hkv, S, d, device=cuda_device).to(dtype)
    pages = S // 64
    sel = None
    if top_k:
        _, kmin, kmax = ext.block_stats(k, 64, minmax=True)
        sel = ext.single_query_quest_topk(q, kmin, kmax, top_k, pages, bf)
    q4, qs = getattr(ext, f"{fmt}_quantize")(q, bf)
    k4, ks = getattr(ext, f"{fmt}_quantize")(k, bf)
    v4, vs = getattr(ext, f"{fmt}_quantize_transposed")(v, bf)
    want, wo, wml = ext.decode_attention(q, k, v, sel, q4, k4, v4, qs, ks, vs, is_mx=mx, is_bf16=bf, num_splits=splits,
                                         return_partials=True)
    n_pool = B * pages + 7                                    # a few unused pages in the pool
    table = torch.randperm(n_pool, device=cuda_device)[:B * pages].to(torch.int32).reshape(B, pages)
    pk4, pks, pv4, pvs, pk, pv = _to_page_pools(table, n_pool, _u8(k4), _u8(ks), _u8(v4), _u8(vs), k, v)
    got, go, gml = ext.decode_attention(q, pk, pv, sel, q4, pk4, pv4, qs, pks, pvs, is_mx=mx, is_bf16=bf,
                                        num_splits=splits, kv_len=S, page_table=table, return_partials=True)
    assert torch.equal(got, want) and torch.equal(go, wo) and torch.equal(gml, wml)
    ext.decode_status(cuda_device)


def test_paged_decode_skips_page_table_entries_outside_the_pool(cuda_device):
    """A negative or too-large page-table entry is never turned into an address: the kernel leaves the page out,
    the call reports it through the status word, and the next call with a sound table is unaffected."""
    torch.manual_seed(14)
    ext = _ext()
    B, hkv, G, S, d = 2, 2, 4, 2048, 128
    pages = S // 64
    q = torch.randn(B, hkv, G, d, device=cuda_device).half()
    k = torch.randn(B, hkv, S, d, device=cuda_device).half()
    v = torch.randn(B, hkv, S, d, device=cuda_device).half()
    _, kmin, kmax = ext.block_stats(k, 64, minmax=True)
    sel = ext.single_query_quest_topk(q, kmin, kmax, 4, pages, False)
    q4, qs = ext.nvfp4_quantize(q)
    k4, ks = ext.nvfp4_quantize(k)
    v4, vs = ext.nvfp4_quantize_transposed(v)
    want = ext.decode_attention(q, k, v, sel, q4, k4, v4, qs, ks, vs, is_mx=False, num_splits=4)
    n_pool = B * pages
    table = torch.randperm(n_pool, device=cuda_device).to(torch.int32).reshape(B, pages)
    pk4, pks, pv4, pvs, pk, pv = _to_page_pools(table, n_pool, _u8(k4), _u8(ks), _u8(v4), _u8(vs), k, v)
    bad = table.clone()
    bad[0, 3] = -7
    bad[1, 20] = n_pool
    bad[1, int(sel[2, 0])] = 1 << 30                          # a selected (16-bit) page as well
    with pytest.raises(RuntimeError, match="page-table"):
        ext.decode_attention(q, pk, pv, sel, q4, pk4, pv4, qs, pks, pvs, is_mx=False, num_splits=4, kv_len=S,
                             page_table=bad, check_status=True)
    got = ext.decode_attention(q, pk, pv, sel, q4, pk4, pv4, qs, pks, pvs, is_mx=False, num_splits=4, kv_len=S,
                               page_table=table, check_status=True)
    assert torch.equal(got, want)


def test_paged_decode_at_the_128k_shape_matches_oracle(cuda_device):
    """The long-context decode configuration at its stated size per sequence: 131072 cached tokens behind a seeded
    random page table, 8 KV heads x 4 query heads, Quest top-10 % (205 of 2048 pages) + 4 sink + 16 local pages in
    16 bits, the rest NVFP4, the chain count the library picks.  Two sequences run on the GPU; four (sequence, KV
    head) rows are compared with the oracle, selection index-equal and attention within the fp16 tolerance."""
    torch.manual_seed(31)
    ext = _ext()
    B, hkv, G, S, d = 2, 8, 4, 131072, 128
    pages = S // 64
    gen = torch.Generator(device=cuda_device).manual_seed(31)
    q = torch.randn(B, hkv, G, d, device=cuda_device, generator=gen).half()
    k = torch.randn(B, hkv, S, d, device=cuda_device, generator=gen).half()
    v = torch.randn(B, hkv, S, d, device=cuda_device, generator=gen).half()
    k[..., torch.randperm(d, device=cuda_device, generator=gen)[:4]] *= 10.0
    top_k = oracle.resolve_top_k(pages, causal=False, fraction=0.1)
    assert top_k == 205
    _, kmin, kmax = ext.block_stats(k, 64, minmax=True)
    sel = ext.select_decode_blocks(q, kmin, kmax, top_k, pages, False, sink=4, local=16)
    q4, qs = ext.nvfp4_quantize(q)
    k4, ks = ext.nvfp4_quantize(k)
    v4, vs = ext.nvfp4_quantize_transposed(v)
    n_pool = B * pages + 5
    table = torch.randperm(n_pool, device=cuda_device, generator=gen)[:B * pages].to(torch.int32).reshape(B, pages)
    pk4, pks, pv4, pvs, pk, pv = _to_page_pools(table, n_pool, _u8(k4), _u8(ks), _u8(v4), _u8(vs), k, v)
    splits = ext.decode_pick_splits(B * hkv, pages)
    out = ext.decode_attention(q, pk, pv, sel, q4, pk4, pv4, qs, pks, pvs, is_mx=False, num_splits=splits, kv_len=S,
                               page_table=table)
    ext.decode_status(cuda_device)
    rows = [(0, 0), (0, 5), (1, 2), (1, 7)]
    bi = torch.tensor([r[0] for r in rows])
    hi = torch.tensor([r[1] for r in rows])
    qo = q.cpu()[bi, hi].unsqueeze(0)                     # [1, 4, G, d]: the four rows as four KV heads of one sequence
    ko = k.cpu()[bi, hi].unsqueeze(0)
    vo = v.cpu()[bi, hi].unsqueeze(0)
    lo, hi_ = oracle.block_stats(ko, 64, ("min", "max"))
    sel_ref = oracle.select_decode(qo, lo, hi_, k=top_k, num_kv_blocks=pages, sink=4, local=16)
    flat = [b * hkv + h for b, h in rows]
    assert torch.equal(sel.cpu()[flat], sel_ref)
    ref = oracle.decode_attention(qo, ko, vo, sel_ref, fmt="nvfp4", splits=splits)
    got = out.cpu()[bi, hi].unsqueeze(0)
    err = (got.float() - ref.float()).abs()
    assert err.max().item() <= FP16_MAX_ABS and err.mean().item() <= MEAN_ABS


@pytest.mark.parametrize("ties", [False, True])
@pytest.mark.parametrize("world,pages,top_k,sink,local,quest", [(2, 64, 6, 1, 2, True), (4, 256, 25, 4, 16, True),
                                                               (8, 2048, 205, 4, 16, True), (3, 100, 10, 0, 0, False),
                                                               (4, 64, 64, 2, 3, True), (5, 700, 33, 1, 1, False)])
def test_sharded_selection_merge_equals_single_gpu(cuda_device, world, pages, top_k, sink, local, quest, ties):
    """The shards of a KV sequence each rank their own pages; the merge kernel over the gathered candidate buffers
    reproduces the single-GPU selection exactly (same picks in the same order, same forced pages) - also when page
    counts do not divide evenly, when a shard comes out empty, and (``ties``) when every page has the same score, so
    that the tie-break alone decides both the shards' own cuts and the merge.  All shards are emulated in one
    process here; the NCCL exchange itself is covered by the two-GPU test."""
    from thriftattention_b200 import distributed as tad

    torch.manual_seed(21)
    ext = _ext()
    B, hkv, G, d = 2, 2, 4, 128
    rows = B * hkv
    q = torch.randn(B, hkv, G, d, device=cuda_device).half()
    if quest:
        lo = torch.randn(B, hkv, pages, d, device=cuda_device).half()
        hi = lo + torch.rand(B, hkv, pages, d, device=cuda_device).half()
    else:
        lo, hi = torch.randn(B, hkv, pages, d, device=cuda_device).half(), None
    if ties:
        lo = lo[:, :, :1].expand(-1, -1, pages, -1).contiguous()
        hi = None if hi is None else hi[:, :, :1].expand(-1, -1, pages, -1).contiguous()
    k_eff = min(top_k, pages - min(sink, pages) - min(local, pages - min(sink, pages)))
    want = ext.select_decode_blocks(q, lo, hi, k_eff, pages, False, sink=sink, local=local)
    shards = tad.plan_page_shards(pages, world)
    n_sink = min(sink, pages)
    local_lo = max(pages - local, n_sink)
    biggest = max(s.num_pages for s in shards)
    send = min(n_sink, biggest) + min(pages - local_lo, biggest) + min(k_eff, biggest)
    gathered = torch.empty(world, 2, rows, send, dtype=torch.int32, device=cuda_device)
    for s in shards:
        my_sink = max(0, min(n_sink, s.page_end) - s.page_begin)
        my_local = max(0, s.page_end - max(local_lo, s.page_begin))
        cand = min(k_eff, max(s.num_pages - my_sink - my_local, 0))
        sl = slice(s.page_begin, s.page_end)
        assert s.page_begin % 32 == 0 or s.num_pages == 0
        if s.num_pages == 0:
            gathered[s.rank, 0].fill_(-1)
            gathered[s.rank, 1].view(torch.float32).fill_(-torch.finfo(torch.float32).max)
            continue
        ext.select_decode_blocks(q, lo[:, :, sl].contiguous(), None if hi is None else hi[:, :, sl].contiguous(), cand,
                                 s.num_pages, False, sink=my_sink, local=my_local, out=gathered[s.rank, 0],
                                 return_scores=True, scores_out=gathered[s.rank, 1].view(torch.float32), row_width=send)
    picks = torch.full((rows, top_k), -1, dtype=torch.int64, device=cuda_device)
    forced = [[] for _ in range(rows)]
    for s in shards:
        mine = ext.merge_page_candidates(gathered, rank=s.rank, total_pages=pages, top_k=top_k, sink=sink, local=local)
        assert mine.shape == (rows, sink + local + top_k)
        t = mine[:, sink + local:].long()
        assert not ((t >= 0) & (picks >= 0)).any()              # every pick belongs to exactly one shard
        picks = torch.where(t >= 0, t + s.page_begin, picks)
        assert ((t < s.num_pages)).all()
        for r in range(rows):
            forced[r] += [int(x) + s.page_begin for x in mine[r, : sink + local].tolist() if x >= 0]
    n_forced = n_sink + (pages - local_lo)
    assert torch.equal(picks[:, :k_eff].cpu(), want[:, n_forced:n_forced + k_eff].long().cpu())
    assert (picks[:, k_eff:] == -1).all()
    for r in range(rows):
        assert sorted(forced[r]) == sorted(want[r, :n_forced].tolist())


def test_decode_step_replays_from_a_cuda_graph(cuda_device):
    """Quantise q + page selection + paged attention + merge allocate nothing behind torch's back and never
    synchronise, so one decode step can be captured once and replayed on new queries."""
    torch.manual_seed(13)
    ext = _ext()
    B, hkv, G, S, d, top_k = 2, 2, 4, 4096, 128, 6
    pages = S // 64
    k = torch.randn(B, hkv, S, d, device=cuda_device).half()
    v = torch.randn(B, hkv, S, d, device=cuda_device).half()
    _, kmin, kmax = ext.block_stats(k, 64, minmax=True)
    k4, ks = ext.nvfp4_quantize(k)
    v4, vs = ext.nvfp4_quantize_transposed(v)
    table = torch.randperm(B * pages, device=cuda_device).to(torch.int32).reshape(B, pages)
    pools = _to_page_pools(table, B * pages, _u8(k4), _u8(ks), _u8(v4), _u8(vs), k, v)
    pk4, pks, pv4, pvs, pk, pv = pools
    q_static = torch.randn(B, hkv, G, d, device=cuda_device).half()

    def step():
        q4, qs = ext.nvfp4_quantize(q_static)
        sel = ext.select_decode_blocks(q_static, kmin, kmax, top_k, pages, False, sink=1, local=2)
        return ext.decode_attention(q_static, pk, pv, sel, q4, pk4, pv4, qs, pks, pvs, is_mx=False, kv_len=S,
                                    page_table=table, allow_padded_selection=True)

    side = torch.cuda.Stream(device=cuda_device)
    side.wait_stream(torch.cuda.current_stream(cuda_device))
    with torch.cuda.stream(side):
        for _ in range(2):
            step()
    torch.cuda.current_stream(cuda_device).wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out_static = step()
    for seed in (1, 2):
        q_static.copy_(torch.randn(B, hkv, G, d, device=cuda_device, generator=torch.Generator(cuda_device).manual_seed(seed)).half())
        graph.replay()
        replayed = out_static.clone()
        assert torch.equal(replayed, step())
    ext.decode_status(cuda_device)


@pytest.mark.parametrize("dtype,fmt,B,hkv,G,S,top_k,splits,d", DECODE_CASES)
def test_decode_attention_matches_oracle(cuda_device, dtype, fmt, B, hkv, G, S, top_k, splits, d):
    torch.manual_seed(6)
    ext = _ext()
    bf, mx = dtype == torch.bfloat16, fmt == "mxfp4"
    q = torch.randn(B, hkv, G, d).to(dtype)
    k = torch.randn(B, hkv, S, d).to(dtype)
    v = torch.randn(B, hkv, S, d).to(dtype)
    sel = None
    if top_k:
        kmin, kmax = oracle.block_stats(k, 64, ("min", "max"))
        sel = oracle.select_decode(q, kmin, kmax, k=top_k, num_kv_blocks=S // 64)
    ref, ref_o, ref_ml = oracle.decode_attention(q, k, v, sel, fmt=fmt, splits=splits, return_partials=True)
    qd, kd, vd = q.to(cuda_device), k.to(cuda_device), v.to(cuda_device)
    q4, qs = getattr(ext, f"{fmt}_quantize")(qd, bf)
    k4, ks = getattr(ext, f"{fmt}_quantize")(kd, bf)
    v4, vs = getattr(ext, f"{fmt}_quantize_transposed")(vd, bf)
    out, po, pml = ext.decode_attention(qd, kd, vd, sel.to(cuda_device) if sel is not None else None, q4, k4, v4, qs, ks, vs,
                                        is_mx=mx, is_bf16=bf, num_splits=splits, return_partials=True)
    err = (out.float().cpu() - ref.float()).abs()
    assert err.max().item() <= _tol(dtype, ref) and err.mean().item() <= MEAN_ABS
    assert (pml.cpu() - ref_ml).abs().max().item() < 1e-3
    merged = ext.merge_decode_partials(po.unsqueeze(0).contiguous(), pml.unsqueeze(0).contiguous(), is_mx=mx, is_bf16=bf)
    assert torch.equal(merged.view_as(out), out)
    # two half-sequence "shards" merged with the shard-merge entry point reproduce a 2-chain run
    if splits == 2:
        o2 = po.permute(1, 0, 2, 3).unsqueeze(2).contiguous()
        m2 = pml.permute(1, 0, 2, 3).unsqueeze(2).contiguous()
        assert torch.equal(ext.merge_decode_partials(o2, m2, is_mx=mx, is_bf16=bf).view_as(out), out)


def test_decode_through_public_api_and_reference_named_ops(cuda_device):
    import thriftattention_b200 as ta

    torch.manual_seed(7)
    ext = _ext()
    q = torch.randn(2, 8, 1, 128).half()
    k = torch.randn(2, 2, 2048, 128).half()
    v = torch.randn(2, 2, 2048, 128).half()
    out = ta.attention(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device),
                       config=ta.AttentionConfig(selection="quest", top_k=4))
    qg = q.reshape(2, 2, 4, 128)
    kmin, kmax = oracle.block_stats(k, 64, ("min", "max"))
    sel = oracle.select_decode(qg, kmin, kmax, k=4, num_kv_blocks=32)
    splits = ext.decode_pick_splits(4, 32)
    ref = oracle.decode_attention(qg, k, v, sel, fmt="nvfp4", splits=splits).reshape(2, 8, 1, 128)
    err = (out.float().cpu() - ref.float()).abs()
    assert err.max().item() <= FP16_MAX_ABS and err.mean().item() <= MEAN_ABS
    out4 = ta.attention(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), config=ta.AttentionConfig(method="fp4"))
    ref4 = oracle.decode_attention(qg, k, v, None, fmt="nvfp4", splits=splits).reshape(2, 8, 1, 128)
    assert (out4.float().cpu() - ref4.float()).abs().max().item() <= FP16_MAX_ABS


def test_bounded_waits_give_up_cleanly(cuda_device):
    """Every device-side wait is bounded.  With the producers switched off (they copy nothing, so nothing
    asynchronous is in flight) and a budget of 200k cycles the consumers' waits run out: the kernels drain, free
    their tensor memory and report TA100_ERR_DEVICE_TIMEOUT through the status calls; the next normal launch gives
    the result it gave before."""
    torch.manual_seed(15)
    ext = _ext()
    q = torch.randn(1, 4, 512, 128, device=cuda_device).half()
    k = torch.randn(1, 2, 512, 128, device=cuda_device).half()
    v = torch.randn(1, 2, 512, 128, device=cuda_device).half()
    q4, qs = ext.nvfp4_quantize(q)
    k4, ks = ext.nvfp4_quantize_permuted(k)
    v4, vs = ext.nvfp4_quantize_transposed(v)
    prefill = lambda: ext.prefill_attention(None, None, None, None, q4, k4, v4, qs, ks, vs, causal=True, is_mx=False,
                                            check_status=True)
    want_p = prefill()
    qd = torch.randn(1, 2, 4, 128, device=cuda_device).half()
    qd4, qds = ext.nvfp4_quantize(qd)
    kd4, kds = ext.nvfp4_quantize(k)
    decode = lambda: ext.decode_attention(None, None, None, None, qd4, kd4, v4, qds, kds, vs, is_mx=False, num_splits=2,
                                          check_status=True)
    want_d = decode()
    try:
        ext.debug_set_wait(200_000, skip_loads=True)
        with pytest.raises(RuntimeError, match="timed out"):
            prefill()
        with pytest.raises(RuntimeError, match="timed out"):
            decode()
    finally:
        ext.debug_set_wait(0, skip_loads=False)
    assert torch.equal(prefill(), want_p)
    assert torch.equal(decode(), want_d)


def test_argument_errors_raise(cuda_device):
    ext = _ext()
    x = torch.randn(1, 1, 64, 96, device=cuda_device).half()
    with pytest.raises(RuntimeError, match="head_dim"):
        ext.nvfp4_quantize(x, False)
    with pytest.raises(RuntimeError, match="contiguous"):
        ext.nvfp4_quantize(torch.randn(1, 1, 256, 128, device=cuda_device).half()[:, :, ::2], False)
    qm = torch.randn(1, 1, 4, 64, device=cuda_device).half()
    with pytest.raises(RuntimeError, match="topk_count"):
        ext.block_mean_topk(qm, qm, 9, True, False)

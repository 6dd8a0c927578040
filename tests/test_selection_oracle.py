"""The oracle's selection against the reference's golden numbers: resolve_top_k table, the
reference tests' small known answers, local-window closed forms, and fixtures produced by the
reference's own PyTorch selection code (tests/golden/make_golden.py)."""
import pytest
import torch

import oracle
from thriftattention_b200.selection import resolve_top_k


def _pad(t, d=64):
    """Embed a [..., n] tensor into head_dim d by zero padding (the known answers use head_dim 2)."""
    out = torch.zeros(*t.shape[:-1], d, dtype=t.dtype)
    out[..., : t.shape[-1]] = t
    return out


def test_resolve_top_k_reference_goldens():
    # tests/test_selection.py:11-34 of the reference
    assert resolve_top_k(8, top_k=99) == 8
    assert [resolve_top_k(2048, fraction=f) for f in (0.05, 0.10, 0.25)] == [52, 105, 274]
    assert [resolve_top_k(2048, causal=False, fraction=f) for f in (0.05, 0.10, 0.25)] == [102, 205, 512]
    with pytest.raises(ValueError, match="top_k"):
        resolve_top_k(8, top_k=-1)
    with pytest.raises(ValueError, match="fraction"):
        resolve_top_k(8, fraction=1.5)


def test_resolve_top_k_matches_reference_table(golden):
    for n, causal, top_k, fraction, expected in golden["top_k"]:
        assert resolve_top_k(n, causal=causal, top_k=top_k, fraction=fraction) == expected
        assert oracle.resolve_top_k(n, causal=causal, top_k=top_k, fraction=fraction) == expected


def test_block_stats_match_reference_pytorch(golden):
    for case in golden["stats"]:
        mean, lo, hi = oracle.block_stats(case["x"], case["block"], ("mean", "min", "max"))
        assert torch.equal(lo, case["min"]) and torch.equal(hi, case["max"])
        # means: fp32 accumulation order differs from torch's; after rounding to 16 bits they agree
        assert torch.equal(mean, case["mean"])


def test_known_answer_block_mean_gqa():
    # tests/test_selection.py:37-59
    q = torch.tensor([[[[10.0, 0.0]], [[0.0, 1.0]], [[1.0, 0.0]], [[0.0, 10.0]]]], dtype=torch.float16)
    k = torch.tensor([[[[1.0, 0.0], [1.0, 0.0], [0.0, 1.0], [0.0, 1.0]],
                       [[0.0, 1.0], [0.0, 1.0], [1.0, 0.0], [1.0, 0.0]]]], dtype=torch.float16)
    qg = _pad(q).reshape(1, 2, 2, 64)
    km, = oracle.block_stats(_pad(k), 2, ("mean",))
    assert oracle.select_decode(qg, km, None, k=1, num_kv_blocks=2).tolist() == [[0], [0]]


def test_known_answer_quest_decode():
    # tests/test_selection.py:75-100
    q = torch.tensor([[[[1.0, -2.0]]]], dtype=torch.float16)
    k = torch.tensor([[[[4.0, -3.0], [2.0, -1.0], [1.0, -1.0], [0.0, 0.0], [3.0, 2.0], [3.0, 1.0]]]], dtype=torch.float16)
    lo, hi = oracle.block_stats(_pad(k), 2, ("min", "max"))
    assert oracle.select_decode(_pad(q).reshape(1, 1, 1, 64), lo, hi, k=1, num_kv_blocks=3).tolist() == [[0]]


def test_known_answer_quest_prefill_causal_padding():
    # tests/test_selection.py:103-129
    q = torch.tensor([[[[1.0, -1.0], [1.0, -1.0], [-1.0, 1.0], [-1.0, 1.0]]]], dtype=torch.float16)
    k = torch.tensor([[[[2.0, -4.0], [1.0, -3.0], [-3.0, 5.0], [-2.0, 6.0]]]], dtype=torch.float16)
    qm, = oracle.block_stats(_pad(q), 2, ("mean",))
    lo, hi = oracle.block_stats(_pad(k), 2, ("min", "max"))
    assert oracle.select_prefill(qm, lo, hi, k=2, causal=True).tolist() == [[[0, -1], [1, 0]]]


def test_known_answer_exact_rank_order():
    # tests/test_cuda_bf16_correctness.py:125-139 of the reference: scores rise with the block index
    q = torch.zeros(1, 1, 1, 64, dtype=torch.float16)
    q[..., 0] = 1.0
    k_mean = torch.zeros(1, 1, 8, 64, dtype=torch.float16)
    k_mean[0, 0, :, 0] = torch.arange(8, dtype=torch.float16)
    assert oracle.select_decode(q, k_mean, None, k=3, num_kv_blocks=8).tolist() == [[7, 6, 5]]


def _expected_local(flat, nq, nk, k, causal):
    rows = []
    for qb in range(nq):
        if causal:
            end = min(qb, nk - 1)
            valid = min(end + 1, k)
            start = max(0, end - k + 1)
            rows.append([start + r if r < valid else -1 for r in range(k)])
        else:
            center = min(qb, nk - 1)
            start = min(max(center - k // 2, 0), max(nk - k, 0))
            rows.append([start + r for r in range(k)])
    return torch.tensor(rows, dtype=torch.int32).reshape(nq, k).unsqueeze(0).expand(flat, -1, -1).contiguous()


LOCAL_CASES = [(1, 2, 5, 5, 3, True), (1, 2, 5, 5, 3, False), (2, 3, 4, 7, 5, True), (2, 3, 4, 7, 5, False),
               (1, 1, 6, 3, 3, True), (1, 1, 6, 3, 2, False), (1, 2, 1, 1, 1, True), (1, 2, 3, 4, 0, True),
               (1, 1, 8, 8, 8, True), (1, 1, 8, 8, 8, False)]


@pytest.mark.parametrize("batch,heads,nq,nk,k,causal", LOCAL_CASES)
def test_local_windows_closed_form(batch, heads, nq, nk, k, causal):
    # closed forms of tests/test_cuda_local_selection.py:9-49
    got = oracle.local_prefill(batch * heads, nq, nk, k, causal)
    assert torch.equal(got, _expected_local(batch * heads, nq, nk, k, causal).reshape(batch * heads, nq, k))


def test_local_decode_window():
    assert oracle.local_decode(3, 7, 3).tolist() == [[4, 5, 6]] * 3


def test_quest_and_mean_selection_match_reference_pytorch(golden):
    for case in golden["quest_prefill"]:
        q, k, blk = case["q"], case["k"], case["block"]
        qm, = oracle.block_stats(q, blk, ("mean",))
        lo, hi = oracle.block_stats(k, blk, ("min", "max"))
        got = oracle.select_prefill(qm, lo, hi, k=case["top_k"], causal=case["causal"])
        assert torch.equal(got, case["sel"])
    for case in golden["quest_decode"]:
        q, k, blk = case["q"], case["k"], case["block"]
        b, hq, _, d = q.shape
        hkv = k.shape[1]
        lo, hi = oracle.block_stats(k, blk, ("min", "max"))
        got = oracle.select_decode(q.reshape(b, hkv, hq // hkv, d), lo, hi, k=case["top_k"], num_kv_blocks=k.shape[2] // blk)
        assert torch.equal(got, case["sel"])
    for case in golden["mean_decode"]:
        q, k, blk = case["q"], case["k"], case["block"]
        b, hq, _, d = q.shape
        hkv = k.shape[1]
        km, = oracle.block_stats(k, blk, ("mean",))
        got = oracle.select_decode(q.reshape(b, hkv, hq // hkv, d), km, None, k=case["top_k"], num_kv_blocks=k.shape[2] // blk)
        assert torch.equal(got, case["sel"])


def test_sink_and_local_forcing_extension():
    torch.manual_seed(5)
    q = torch.randn(1, 2, 16 * 8, 64).half()
    k = torch.randn(1, 1, 16 * 8, 64).half()
    qm, = oracle.block_stats(q, 8, ("mean",))
    lo, hi = oracle.block_stats(k, 8, ("min", "max"))
    base = oracle.select_prefill(qm, lo, hi, k=3, causal=True)
    ext = oracle.select_prefill(qm, lo, hi, k=3, causal=True, sink=1, local=2)
    assert ext.shape[-1] == 6 and base.shape[-1] == 3
    for h in range(2):
        for qb in range(16):
            row = [v for v in ext[h, qb].tolist() if v >= 0]
            assert len(set(row)) == len(row)
            assert 0 in row and qb in row and max(row) <= qb
            if qb >= 1:
                assert qb - 1 in row
            assert len(row) == min(qb + 1, 6)
    # with no forcing the extension reduces to the reference behaviour
    assert torch.equal(oracle.select_prefill(qm, lo, hi, k=3, causal=True, sink=0, local=0), base)


def test_pack_mask():
    sel = torch.tensor([[[0, 65, -1], [3, 2, 1]]], dtype=torch.int32)
    mask = oracle.pack_mask(sel, 128)
    assert mask.shape == (1, 2, 2)
    assert mask[0, 0].tolist() == [1, 2] and mask[0, 1].tolist() == [14, 0]

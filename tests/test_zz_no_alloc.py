"""The allocation-free decode entry point (ta100_decode_attention_static).

Some callers of this library cannot allocate device memory while serving: a process that handed
all free HBM to its own pool at start-up, or a decode loop that cannot tolerate the device-wide
synchronisation of cudaMalloc.  For them the split-KV scratch is a fixed array inside the library.
This test drives that entry point through the C ABI twice in a row, with different inputs, and
checks each result against the regular entry point (whose scratch the caller provides): the two must
agree bit for bit, since only the location of the scratch differs — the second call also shows that
stale scratch contents from the first do not leak into the result.  The first result is also compared
with the CPU oracle, within the attention tolerance of the other GPU tests.
It sits last in collection order so that a failure here cannot hide any other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

TOL_MAX_ABS, TOL_MEAN_ABS = 2e-3, 2e-4  # the attention tolerance used throughout the GPU tests


def _inputs(dev, seed, batch, hkv, group, seq, top_k):
    from thriftattention_b200 import _C

    g = torch.Generator(device=dev).manual_seed(seed)
    q = torch.randn(batch, hkv, group, 128, device=dev, dtype=torch.float16, generator=g)
    k = torch.randn(batch, hkv, seq, 128, device=dev, dtype=torch.float16, generator=g)
    v = torch.randn(batch, hkv, seq, 128, device=dev, dtype=torch.float16, generator=g)
    q4, qs = _C.nvfp4_quantize(q)
    k4, ks = _C.nvfp4_quantize(k)
    v4, vs = _C.nvfp4_quantize_transposed(v)
    _, kmin, kmax = _C.block_stats(k, 64, minmax=True)
    sel = _C.single_query_quest_topk(q, kmin, kmax, top_k, seq // 64, False)
    return q, k, v, sel, q4, k4, v4, qs, ks, vs


def test_static_scratch_entry_matches_regular_entry_twice(cuda_device):
    from thriftattention_b200 import _C, _lib

    lib = _lib.load()
    assert lib.ta100_decode_static_scratch_bytes() == 16 << 20
    stream = ctypes.c_void_p(torch.cuda.current_stream(cuda_device).cuda_stream)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    for seed, (batch, hkv, group, seq, top_k, splits) in enumerate([(2, 2, 4, 4096, 6, 5), (1, 4, 8, 2048, 3, 4)]):
        q, k, v, sel, q4, k4, v4, qs, ks, vs = _inputs(cuda_device, seed, batch, hkv, group, seq, top_k)
        expected = _C.decode_attention(q, k, v, sel, q4, k4, v4, qs, ks, vs, is_mx=False, is_bf16=False, num_splits=splits)
        out = torch.full((batch, hkv, group, 128), float("nan"), device=cuda_device, dtype=torch.float16)
        rc = lib.ta100_decode_attention_static(ptr(q), ptr(k), ptr(v), ptr(sel), sel.size(1), ptr(q4), ptr(k4), ptr(v4),
                                               ptr(qs), ptr(ks), ptr(vs), None, 0, 0, ptr(out), batch, hkv, group, seq, seq,
                                               128, 0, 0, splits, stream)
        assert rc == 0, lib.ta100_status_string(rc)
        torch.cuda.synchronize()
        assert not torch.isnan(out).any()
        assert torch.equal(out, expected)
        if seed == 0:
            import oracle

            ref = oracle.decode_attention(q.cpu(), k.cpu(), v.cpu(), sel.cpu(), fmt="nvfp4", splits=splits)
            err = (out.float().cpu() - ref.float()).abs()
            assert err.max().item() <= TOL_MAX_ABS and err.mean().item() <= TOL_MEAN_ABS
        # the Python wrapper goes through the same entry point
        out2 = torch.empty_like(out)
        _C.decode_attention_noalloc(q, k, v, sel, q4, k4, v4, qs, ks, vs, out2, is_mx=False, num_splits=splits)
        assert torch.equal(out2, out)


def test_static_scratch_entry_rejects_oversized_problems(cuda_device):
    from thriftattention_b200 import _lib

    lib = _lib.load()
    one = torch.zeros(16, device=cuda_device)
    p = ctypes.c_void_p(one.data_ptr())
    # 512 (sequence, head) pairs x 64 chains x 8 rows x 130 floats = 136 MB of partials: beyond the 16 MiB array
    rc = lib.ta100_decode_attention_static(None, None, None, None, 0, p, p, p, p, p, p, None, 0, 0, p, 64, 8, 8, 131072,
                                           131072,
                                           128, 0, 0, 64, None)
    assert rc == -9
    assert b"16 MiB" in lib.ta100_status_string(rc)

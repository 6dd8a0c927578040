"""The C-ABI library loads on a machine without a GPU and exports every symbol that
include/thrift_sm100.h declares.  No compute calls here."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "thrift_sm100.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ta100_\w+)\s*\(", text)))


def test_header_symbols_are_exported():
    from thriftattention_b200 import _lib

    lib = _lib.load()
    names = _declared_symbols()
    assert len(names) >= 15
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert set(_lib.SIGNATURES) == set(names)


def test_version_and_status_strings():
    from thriftattention_b200 import _lib

    lib = _lib.load()
    assert lib.ta100_version() >= 100
    assert lib.ta100_status_string(0) == b"ok"
    for code in range(-8, 0):
        assert lib.ta100_status_string(code) not in (b"ok", b"unknown status")


def test_argument_errors_are_reported_without_a_gpu():
    from thriftattention_b200 import _lib

    lib = _lib.load()
    # null pointers / bad head_dim are rejected before any CUDA call
    assert lib.ta100_quantize(None, None, None, 1, 64, 128, 0, 0, 0, None) == -1
    buf = ctypes.create_string_buffer(256)
    p = ctypes.cast(buf, ctypes.c_void_p)
    assert lib.ta100_quantize(p, p, p, 1, 64, 96, 0, 0, 0, None) == -3
    assert lib.ta100_block_stats(p, None, None, None, 1, 100, 128, 64, 0, None) == -2
    assert lib.ta100_prefill_workspace_bytes(1, 32, 8, 131072, 131072, 128, 0) > 0
    assert lib.ta100_decode_workspace_bytes(256, 4, 128, 16) == 256 * 16 * 4 * 130 * 4
    # the entries that read the sequence length from device memory insist on that pointer (and its alignment)
    assert lib.ta100_advance_length(None, 1, 1, 128, None) == -1
    assert lib.ta100_cache_append_at(p, p, p, p, p, p, p, p, None, None, None, None, 0, 0, 1, 1, 1, 128, None, 1, 0, 1, 1, 128, 64,
                                     0, 0, 0, None) == -1
    odd = ctypes.c_void_p(p.value + 2)
    assert lib.ta100_cache_append_at(p, p, p, p, p, p, p, p, None, None, None, None, 0, 0, 1, 1, 1, 128, odd, 1, 0, 1, 1, 128, 64,
                                     0, 0, 0, None) == -4
    assert lib.ta100_cache_append_at(p, p, p, p, p, p, p, p, None, None, None, None, 0, 0, 2, 1, 1, 128, p, 3, 0, 1, 1, 128, 64,
                                     0, 0, 0, None) == -2      # three lengths for a batch of two
    assert lib.ta100_cached_decode_step_at(p, p, p, p, p, p, p, p, p, None, 0, 0, p, None, p, 4, p, p, p, 1, 1, 4, None, 1, 1, 128,
                                           128, 2, 1, 0.0, 0, 0, 128, 0, 0, 1, None) == -1
    assert lib.ta100_cached_decode_step_at(p, p, p, p, p, p, p, p, p, None, 0, 0, p, None, p, 4, p, p, p, 1, 1, 4, p, 1, 1, 100,
                                           128, 2, 1, 0.0, 0, 0, 128, 0, 0, 1, None) == -2      # max_len not in whole pages


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    import pytest

    from thriftattention_b200 import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "_LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(ImportError, match="not built"):
        _lib.load()


def test_device_side_block_counts_follow_the_python_rule():
    """The counts the device-length decode step derives from the length (restated for the host in
    ta100_decode_step_counts) equal what cached_decode_attention computes in Python - resolve_top_k with its
    round-half-to-even, then local and sink blocks as far as there is room - for every length and a spread of
    fractions, ties included."""
    from thriftattention_b200 import _lib
    from thriftattention_b200.selection import resolve_top_k

    lib = _lib.load()
    out = (ctypes.c_int * 4)()
    cases = [(None, f, s, l) for f in (0.0, 0.05, 0.1, 0.25, 0.3, 0.5, 0.75, 1.0) for s, l in ((0, 0), (1, 1), (4, 16))]
    cases += [(k, None, s, l) for k in (0, 1, 7, 300) for s, l in ((0, 0), (2, 3))]
    for top_k, fraction, sink_cfg, local_cfg in cases:
        for blocks in list(range(0, 70)) + [255, 256, 257, 1023, 2047, 2048]:
            for extra in (0, 63):
                assert lib.ta100_decode_step_counts(blocks * 64 + extra, -1 if top_k is None else top_k,
                                                    0.05 if fraction is None else fraction, sink_cfg, local_cfg, out) == 0
                k = resolve_top_k(blocks, causal=False, top_k=top_k, fraction=fraction)
                local = max(0, min(local_cfg, blocks - k))
                sink = max(0, min(sink_cfg, blocks - k - local))
                if k == 0:
                    sink = local = 0
                assert list(out) == [blocks, k, sink, local], (top_k, fraction, sink_cfg, local_cfg, blocks)

"""CPU oracle (test infrastructure only).

Python front end over ``thrift_oracle.c``: a plain-C restatement of the
reference's quantiser, selection and attention arithmetic.  Only ``tests/``,
``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may import
this package; the product package never does.

All tensor arguments are CPU ``torch`` tensors (fp16 / bf16 / uint8 / int32);
results are returned as CPU tensors of the same dtypes the CUDA path produces.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np
import torch

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_build" / "libthrift_oracle.so"
_lib = None


def build(force: bool = False) -> Path:
    """Compile the C oracle with gcc (idempotent)."""
    src = _HERE / "thrift_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        _LIB_PATH.parent.mkdir(exist_ok=True)
        subprocess.run(
            ["gcc", "-O2", "-fopenmp", "-fPIC", "-ffp-contract=off", "-shared", "-o", str(_LIB_PATH), str(src), "-lm"],
            check=True,
        )
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(str(build()))
        _lib.ora_half_to_float.restype = ctypes.c_float
        _lib.ora_half_to_float.argtypes = [ctypes.c_uint16]
        _lib.ora_from_e4m3.restype = ctypes.c_float
        _lib.ora_from_e4m3.argtypes = [ctypes.c_uint8]
        _lib.ora_from_e8m0.restype = ctypes.c_float
        _lib.ora_from_e8m0.argtypes = [ctypes.c_uint8]
        _lib.ora_from_e2m1.restype = ctypes.c_float
        _lib.ora_from_e2m1.argtypes = [ctypes.c_uint8]
        for name in ("ora_to_e2m1", "ora_to_e4m3", "ora_to_e8m0"):
            fn = getattr(_lib, name)
            fn.restype = ctypes.c_uint8
            fn.argtypes = [ctypes.c_float]
        _lib.ora_float_to_half.restype = ctypes.c_uint16
        _lib.ora_float_to_half.argtypes = [ctypes.c_float]
        _lib.ora_float_to_bf16.restype = ctypes.c_uint16
        _lib.ora_float_to_bf16.argtypes = [ctypes.c_float]
        _lib.ora_merge_partials.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                            ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_void_p]
    return _lib


def _p(t):
    if t is None:
        return None
    if isinstance(t, torch.Tensor):
        assert t.device.type == "cpu" and t.is_contiguous()
        return ctypes.c_void_p(t.data_ptr())
    assert isinstance(t, np.ndarray) and t.flags["C_CONTIGUOUS"]
    return ctypes.c_void_p(t.ctypes.data)


def _is_bf16(x: torch.Tensor) -> int:
    assert x.dtype in (torch.float16, torch.bfloat16)
    return int(x.dtype == torch.bfloat16)


def _scale_dtype(fmt: str):
    return torch.float8_e8m0fnu if fmt == "mxfp4" else torch.float8_e4m3fn


def _group(fmt: str) -> int:
    return 32 if fmt == "mxfp4" else 16


# --------------------------------------------------------------------------- scalar codecs
def to_e2m1(x: float) -> int:
    return lib().ora_to_e2m1(ctypes.c_float(x))


def to_e4m3(x: float) -> int:
    return lib().ora_to_e4m3(ctypes.c_float(x))


def to_e8m0(x: float) -> int:
    return lib().ora_to_e8m0(ctypes.c_float(x))


def from_e4m3(b: int) -> float:
    return lib().ora_from_e4m3(ctypes.c_uint8(b))


def from_e8m0(b: int) -> float:
    return lib().ora_from_e8m0(ctypes.c_uint8(b))


def from_e2m1(b: int) -> float:
    return lib().ora_from_e2m1(ctypes.c_uint8(b))


def perm32(x: int) -> int:
    return lib().ora_perm32(ctypes.c_int(x))


# --------------------------------------------------------------------------- quantisers
def quantize(x: torch.Tensor, fmt: str = "nvfp4", layout: str = "plain"):
    """x: [B, H, S, D] fp16/bf16 -> (codes uint8, scales fp8) in the reference's layouts.

    layout: "plain" | "permuted" | "transposed" | "transposed_permuted".
    """
    x = x.contiguous()
    b, h, s, d = x.shape
    g = _group(fmt)
    is_mx = int(fmt == "mxfp4")
    permuted = int("permuted" in layout)
    if layout.startswith("transposed"):
        p = (s + 127) // 128 * 128
        codes = torch.empty(b, h, d, p // 2, dtype=torch.uint8)
        scales = torch.empty(b, h, d, p // g, dtype=torch.uint8)
        lib().ora_quantize_transposed(_p(x), b * h, s, d, is_mx, _is_bf16(x), permuted, _p(codes), _p(scales))
    else:
        codes = torch.empty(b, h, s, d // 2, dtype=torch.uint8)
        scales = torch.empty(b, h, s, d // g, dtype=torch.uint8)
        lib().ora_quantize_rows(_p(x), b * h, s, d, is_mx, _is_bf16(x), permuted, _p(codes), _p(scales))
    return codes, scales.view(_scale_dtype(fmt))


# --------------------------------------------------------------------------- statistics / selection
def block_stats(x: torch.Tensor, block: int, want=("mean", "min", "max")):
    x = x.contiguous()
    b, h, s, d = x.shape
    nb = s // block
    outs = {}
    for name in ("mean", "min", "max"):
        outs[name] = torch.empty(b, h, nb, d, dtype=x.dtype) if name in want else None
    lib().ora_block_stats(_p(x), b * h, s, d, block, _is_bf16(x), _p(outs["mean"]), _p(outs["min"]), _p(outs["max"]))
    return tuple(outs[n] for n in want)


def select_prefill(q_mean, k_a, k_b=None, *, k: int, causal: bool = True, sink: int = 0, local: int = 0):
    """q_mean [B,Hq,nq,D]; k_a (+k_b) [B,Hkv,nk,D] un-expanded. Quest when k_b is given (k_a=min, k_b=max)."""
    q_mean = q_mean.contiguous()
    k_a = k_a.contiguous()
    b, hq, nq, d = q_mean.shape
    hkv, nk = k_a.shape[1], k_a.shape[2]
    width = sink + local + k
    out = torch.empty(b * hq, nq, width, dtype=torch.int32)
    if width == 0:
        return out
    kb = k_b.contiguous() if k_b is not None else None
    lib().ora_select_prefill(_p(q_mean), _p(k_a), _p(kb), b * hq, hq // hkv, nq, nk, d, k, int(causal),
                             int(k_b is not None), _is_bf16(q_mean), sink, local, _p(out))
    return out


def select_decode(q_grouped, k_a, k_b=None, *, k: int, num_kv_blocks: int, sink: int = 0, local: int = 0):
    """q_grouped [B,Hkv,G,D]; k_a (+k_b) [B,Hkv,cap_blocks,D]."""
    q_grouped = q_grouped.contiguous()
    k_a = k_a.contiguous()
    b, hkv, g, d = q_grouped.shape
    width = sink + local + k
    out = torch.empty(b * hkv, width, dtype=torch.int32)
    if width == 0:
        return out
    kb = k_b.contiguous() if k_b is not None else None
    lib().ora_select_decode(_p(q_grouped), _p(k_a), _p(kb), b * hkv, g, num_kv_blocks, k_a.shape[2], d, k,
                            int(k_b is not None), _is_bf16(q_grouped), sink, local, _p(out))
    return out


def local_prefill(flat_heads: int, nq: int, nk: int, k: int, causal: bool = True):
    out = torch.empty(flat_heads, nq, k, dtype=torch.int32)
    if k:
        lib().ora_local_prefill(flat_heads, nq, nk, k, int(causal), _p(out))
    return out


def local_decode(flat_heads: int, nk: int, k: int):
    out = torch.empty(flat_heads, k, dtype=torch.int32)
    if k:
        lib().ora_local_decode(flat_heads, nk, k, _p(out))
    return out


def pack_mask(sel: torch.Tensor, nk: int):
    sel = sel.contiguous()
    k = sel.shape[-1]
    rows = sel.numel() // max(k, 1) if k else int(np.prod(sel.shape[:-1]))
    words = (nk + 63) // 64
    mask = torch.zeros(*sel.shape[:-1], words, dtype=torch.int64)
    if k:
        lib().ora_pack_mask(_p(sel), rows, k, nk, words, _p(mask))
    return mask


# --------------------------------------------------------------------------- attention
def prefill_attention(q, k, v, sel, *, fmt="nvfp4", block=64, causal=True, round_partial=True,
                      rows=None, packed=None):
    """Mixed prefill attention. q [B,Hq,Sq,D], k/v [B,Hkv,Skv,D]; sel [B*Hq, Sq/block, W] or None.

    ``packed`` may supply (q4, k4, v4t, qs, ks, vst) in *plain* (logical) K order; otherwise the
    oracle quantises q, k, v itself.  ``rows=(lo, hi)`` restricts the query rows that are computed.
    """
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    b, hq, sq, d = q.shape
    hkv, skv = k.shape[1], k.shape[2]
    if packed is None:
        q4, qs = quantize(q, fmt, "plain")
        k4, ks = quantize(k, fmt, "plain")
        v4t, vst = quantize(v, fmt, "transposed")
    else:
        q4, k4, v4t, qs, ks, vst = [t.contiguous() for t in packed]
    out = torch.zeros_like(q)
    lo, hi = rows if rows is not None else (0, sq)
    width = 0 if sel is None else sel.shape[-1]
    sel_c = sel.contiguous() if sel is not None else None
    for bi in range(b):
        s_b = sel_c[bi * hq:(bi + 1) * hq].contiguous() if sel_c is not None else None
        lib().ora_prefill_attention(
            _p(q[bi]), _p(k[bi]), _p(v[bi]), _p(q4[bi]), _p(qs[bi].view(torch.uint8)), _p(k4[bi]),
            _p(ks[bi].view(torch.uint8)), _p(v4t[bi]), _p(vst[bi].view(torch.uint8)), _p(s_b), width, hq, hkv, sq,
            skv, skv, d, block, int(causal), int(fmt == "mxfp4"), _is_bf16(q), int(round_partial), lo, hi,
            _p(out[bi]))
    return out


def decode_attention(q_grouped, k, v, sel, *, fmt="nvfp4", splits=1, packed=None, return_partials=False):
    """q_grouped [B,Hkv,G,D]; k/v [B,Hkv,S,D]; sel [B*Hkv, W] 64-token page ids or None."""
    q_grouped, k, v = q_grouped.contiguous(), k.contiguous(), v.contiguous()
    b, hkv, g, d = q_grouped.shape
    s = k.shape[2]
    if packed is None:
        q4, qs = quantize(q_grouped, fmt, "plain")
        k4, ks = quantize(k, fmt, "plain")
        v4t, vst = quantize(v, fmt, "transposed")
    else:
        q4, k4, v4t, qs, ks, vst = [t.contiguous() for t in packed]
    out = torch.zeros_like(q_grouped)
    width = 0 if sel is None else sel.shape[-1]
    npages = (s + 63) // 64
    splits = max(1, min(splits, npages))
    part_o = torch.zeros(b * hkv, splits, g, d, dtype=torch.float32) if return_partials else None
    part_ml = torch.zeros(b * hkv, splits, g, 2, dtype=torch.float32) if return_partials else None
    lib().ora_decode_attention(
        _p(q_grouped), _p(k), _p(v), _p(q4), _p(qs.view(torch.uint8)), _p(k4), _p(ks.view(torch.uint8)), _p(v4t),
        _p(vst.view(torch.uint8)), _p(sel.contiguous() if sel is not None else None), width, b * hkv, g, s,
        k4.shape[2], d, int(fmt == "mxfp4"), _is_bf16(q_grouped), splits, _p(out), _p(part_o), _p(part_ml))
    if return_partials:
        return out, part_o, part_ml
    return out


def merge_partials(part_o, part_ml, *, fmt="nvfp4", out_dtype=torch.float16):
    """part_o [shards, rows, D] fp32, part_ml [shards, rows, 2] -> [rows, D]."""
    part_o, part_ml = part_o.contiguous(), part_ml.contiguous()
    shards, rows, d = part_o.shape
    out = torch.empty(rows, d, dtype=out_dtype)
    c = 6.0 if fmt == "mxfp4" else 2688.0
    lib().ora_merge_partials(_p(part_o), _p(part_ml), shards, rows, d, ctypes.c_float(c),
                             int(out_dtype == torch.bfloat16), _p(out))
    return out


def resolve_top_k(num_blocks: int, *, causal: bool = True, top_k=None, fraction=None) -> int:
    """Top-k count rule, restated from selection/block_mean.py:12-41 of the reference."""
    import math

    if top_k is not None:
        if top_k < 0:
            raise ValueError("top_k must be non-negative")
        return min(top_k, num_blocks)
    f = 0.05 if fraction is None else fraction
    if not 0.0 <= f <= 1.0:
        raise ValueError("fraction must be in [0, 1]")
    if num_blocks <= 0 or f <= 0.0:
        return 0
    if f >= 1.0:
        return num_blocks
    if not causal:
        return max(1, min(num_blocks, round(f * num_blocks)))
    bb = -(2 * num_blocks + 1)
    cc = f * num_blocks * (num_blocks + 1)
    disc = bb * bb - 4.0 * cc
    if disc < 0.0:
        return num_blocks
    return max(1, min(num_blocks, round((-bb - math.sqrt(disc)) / 2.0)))

"""Loader for ``libthrift_sm100.so`` — the C-ABI CUDA library behind this package.

The library is built in-tree by ``thriftattention_b200/csrc/build.py`` (nvcc, sm_100a).
There is no fallback: if the shared object is missing or a symbol cannot be
resolved, importing the extension raises ``ImportError``.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "libthrift_sm100.so"
_lib: ctypes.CDLL | None = None

_c_int, _c_ll, _c_vp, _c_sz = ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_size_t

# name -> (restype, argtypes); mirrors include/thrift_sm100.h
SIGNATURES = {
    "ta100_version": (_c_int, []),
    "ta100_status_string": (ctypes.c_char_p, [_c_int]),
    "ta100_quantize": (_c_int, [_c_vp, _c_vp, _c_vp, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_vp]),
    "ta100_quantize_qkv": (_c_int, [_c_vp] * 9 + [_c_ll, _c_int, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_vp]),
    "ta100_block_stats": (_c_int, [_c_vp, _c_vp, _c_vp, _c_vp, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_vp]),
    "ta100_cache_append": (_c_int, [_c_vp] * 11 + [_c_ll] + [_c_int] * 9 + [_c_vp]),
    "ta100_cache_append_paged": (_c_int, [_c_vp] * 12 + [_c_int] * 13 + [_c_vp]),
    "ta100_cache_append_at": (_c_int, [_c_vp] * 12 + [_c_int] * 6 + [_c_vp] + [_c_int] * 9 + [_c_vp]),
    "ta100_decode_step_counts": (_c_int, [_c_int, _c_int, ctypes.c_double, _c_int, _c_int, ctypes.POINTER(_c_int)]),
    "ta100_advance_length": (_c_int, [_c_vp, _c_int, _c_int, _c_int, _c_vp]),
    "ta100_cached_decode_step_at": (_c_int, [_c_vp] * 10 + [_c_int] * 2 + [_c_vp] * 3 + [_c_int] + [_c_vp] * 3 + [_c_int] * 3
                                    + [_c_vp] + [_c_int] * 6 + [ctypes.c_double] + [_c_int] * 6 + [_c_vp]),
    "ta100_peer_exchange_create": (_c_int, [_c_int, _c_ll, ctypes.POINTER(_c_vp), ctypes.c_char_p]),
    "ta100_peer_exchange_open": (_c_int, [ctypes.c_char_p, ctypes.POINTER(_c_vp)]),
    "ta100_peer_exchange_close": (_c_int, [_c_vp]),
    "ta100_peer_exchange_destroy": (_c_int, [_c_vp]),
    "ta100_peer_all_gather": (_c_int, [_c_vp, _c_vp, _c_ll, _c_ll, _c_int, _c_int, ctypes.POINTER(_c_vp), _c_vp]),
    "ta100_peer_exchange_status": (_c_int, [_c_vp, _c_int, _c_ll, _c_vp]),
    "ta100_select_prefill": (_c_int, [_c_vp, _c_vp, _c_vp, _c_vp] + [_c_int] * 11 + [_c_vp]),
    "ta100_select_decode": (_c_int, [_c_vp, _c_vp, _c_vp, _c_vp, _c_vp] + [_c_int] * 11 + [_c_vp]),
    "ta100_local_block_topk": (_c_int, [_c_vp, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_vp]),
    "ta100_single_query_local_topk": (_c_int, [_c_vp, _c_ll, _c_int, _c_int, _c_vp]),
    "ta100_pack_topk_mask": (_c_int, [_c_vp, _c_vp, _c_ll, _c_int, _c_int, _c_int, _c_vp]),
    "ta100_merge_page_candidates": (_c_int, [_c_vp, _c_vp] + [_c_int] * 8 + [_c_vp]),
    "ta100_reduce_partials": (_c_int, [_c_vp] * 4 + [_c_ll] + [_c_int] * 3 + [_c_vp]),
    "ta100_cached_decode_step": (_c_int, [_c_vp] * 15 + [_c_int] * 14 + [_c_vp]),
    "ta100_cached_decode_step_paged": (_c_int, [_c_vp] * 10 + [_c_int] * 2 + [_c_vp] * 6 + [_c_int] * 13 + [_c_vp]),
    "ta100_prefill_workspace_bytes": (_c_sz, [_c_int] * 7),
    "ta100_prefill_attention": (_c_int, [_c_vp] * 4 + [_c_int, _c_int] + [_c_vp] * 8 + [_c_sz] + [_c_int] * 14 + [_c_vp]),
    "ta100_prefill_status": (_c_int, [_c_vp] + [_c_int] * 7 + [_c_vp]),
    "ta100_decode_pick_splits": (_c_int, [_c_int, _c_int]),
    "ta100_decode_workspace_bytes": (_c_sz, [_c_int] * 4),
    "ta100_decode_attention": (_c_int, [_c_vp] * 4 + [_c_int] + [_c_vp] * 7 + [_c_int] * 2 + [_c_vp] * 3 + [_c_int] * 10
                               + [_c_vp]),
    "ta100_decode_status": (_c_int, [_c_vp]),
    "ta100_debug_set_wait": (_c_int, [_c_ll, _c_int]),
    "ta100_merge_partials": (_c_int, [_c_vp, _c_vp, _c_vp, _c_int, _c_ll, _c_ll, _c_ll] + [_c_int] * 5 + [_c_vp]),
    "ta100_decode_static_scratch_bytes": (_c_sz, []),
    "ta100_decode_attention_static": (_c_int, [_c_vp] * 4 + [_c_int] + [_c_vp] * 7 + [_c_int] * 2 + [_c_vp] + [_c_int] * 9
                                      + [_c_vp]),
}


def library_path() -> Path:
    return _LIB_PATH


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise ImportError(
            f"{_LIB_PATH.name} is not built. Run `python -m thriftattention_b200.csrc.build` "
            "(needs nvcc with sm_100a support) from the repository root."
        )
    try:
        lib = ctypes.CDLL(str(_LIB_PATH))
    except OSError as exc:  # pragma: no cover - depends on the host
        raise ImportError(f"could not load {_LIB_PATH}: {exc}") from exc
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name, None)
        if fn is None:
            raise ImportError(f"{_LIB_PATH.name} does not export {name}")
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(status: int, what: str) -> None:
    """Raise ``RuntimeError`` for a non-zero status returned by the library."""
    if status != 0:
        msg = load().ta100_status_string(status).decode()
        raise RuntimeError(f"{what} failed: {msg} (status {status})")

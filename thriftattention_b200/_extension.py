"""Access to the operator module (the counterpart of the reference's ``thriftattention._C``).

The reference imports a pybind11 extension lazily (src/thriftattention/_extension.py:7-15);
here the operators are ``thriftattention_b200._C``, a thin ctypes layer over the in-tree
``libthrift_sm100.so``.  There is no CPU or eager fallback: a missing library is an error.
"""
from __future__ import annotations

from importlib import import_module
from types import ModuleType


def get_extension() -> ModuleType:
    try:
        return import_module("thriftattention_b200._C")
    except ImportError as exc:
        raise ImportError(
            "The thriftattention_b200 CUDA library is not built. Run "
            "`python -m thriftattention_b200.csrc.build` on a machine with nvcc (sm_100a)."
        ) from exc

"""B200-native (sm_100a) selective mixed-precision attention.

Public surface of the reference package (src/thriftattention/__init__.py): ``attention``,
``AttentionConfig``, ``ThriftAttentionCache``, the quantisation formats and the selection
policies.  Importing this package touches no CUDA state; the CUDA library is loaded when
the first operator is called.
"""
from .config import AttentionConfig
from .functional import attention
from .offload import attention_host
from .quant import QuantFormat, get_quant_format
from .selection import SelectionConfig, get_selection_policy, resolve_top_k

__all__ = [
    "AttentionConfig",
    "attention",
    "attention_host",
    "ThriftAttentionCache",
    "QuantFormat",
    "get_quant_format",
    "SelectionConfig",
    "get_selection_policy",
    "resolve_top_k",
]


def __getattr__(name):
    # the cache pulls in the integration layer; resolve it on first use
    if name == "ThriftAttentionCache":
        from .integrations.transformers_cache import ThriftAttentionCache

        return ThriftAttentionCache
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")

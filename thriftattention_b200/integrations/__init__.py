"""Optional framework integrations (Hugging Face Transformers)."""
from .transformers import (
    TransformersAttentionConfig,
    TransformersCacheInputs,
    get_registered_transformers_attention_config,
    prepare_transformers_generation_cache,
    register_transformers_attention,
)

__all__ = [
    "TransformersAttentionConfig",
    "TransformersCacheInputs",
    "get_registered_transformers_attention_config",
    "prepare_transformers_generation_cache",
    "register_transformers_attention",
]

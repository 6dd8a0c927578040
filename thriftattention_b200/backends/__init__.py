from .base import AttentionBackend
from .registry import select_backend

__all__ = ["AttentionBackend", "select_backend"]

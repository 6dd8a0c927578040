"""KV-block selection policies (registry of the reference's src/thriftattention/selection/__init__.py)."""
from __future__ import annotations

from thriftattention_b200.config import SelectionMethod

from .base import SelectionConfig, SelectionPolicy
from .block_mean import BlockMeanSelectionPolicy, block_means, select_block_pairs, select_key_blocks
from .counts import resolve_top_k
from .local import LocalSelectionPolicy, select_local_block_pairs, select_local_key_blocks
from .quest import QuestSelectionPolicy, block_minmax, select_quest_block_pairs, select_quest_key_blocks

_POLICIES: dict[str, SelectionPolicy] = {
    policy.name: policy for policy in (BlockMeanSelectionPolicy(), LocalSelectionPolicy(), QuestSelectionPolicy())
}


def get_selection_policy(name: SelectionMethod) -> SelectionPolicy:
    policy = _POLICIES.get(name)
    if policy is None:
        raise NotImplementedError(f"selection policy {name!r} is not implemented")
    return policy


__all__ = [
    "SelectionConfig", "SelectionPolicy", "BlockMeanSelectionPolicy", "LocalSelectionPolicy",
    "QuestSelectionPolicy", "block_minmax", "block_means", "get_selection_policy", "resolve_top_k",
    "select_block_pairs", "select_key_blocks", "select_local_block_pairs", "select_local_key_blocks",
    "select_quest_block_pairs", "select_quest_key_blocks",
]

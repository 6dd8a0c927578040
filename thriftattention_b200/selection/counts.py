"""How many KV blocks a selection keeps.

Restates ``resolve_top_k`` of the reference (src/thriftattention/selection/block_mean.py:12-41):
an explicit ``top_k`` is clamped to the block count; otherwise ``fraction`` of the blocks for
non-causal attention, and for causal attention the count k whose kept area
k(2n + 1 - k)/2 is ``fraction`` of the causal triangle n(n + 1)/2.
"""
from __future__ import annotations

import math


def resolve_top_k(num_blocks: int, *, causal: bool = True, top_k: int | None = None,
                  fraction: float | None = None) -> int:
    if top_k is not None:
        if top_k < 0:
            raise ValueError("top_k must be non-negative")
        return min(top_k, num_blocks)
    share = 0.05 if fraction is None else fraction
    if not 0.0 <= share <= 1.0:
        raise ValueError("fraction must be in [0, 1]")
    if num_blocks <= 0 or share <= 0.0:
        return 0
    if share >= 1.0:
        return num_blocks
    if not causal:
        return max(1, min(num_blocks, round(share * num_blocks)))
    # smaller root of k^2 - (2n+1) k + share * n (n+1) = 0
    lin = 2 * num_blocks + 1
    disc = lin * lin - 4.0 * share * num_blocks * (num_blocks + 1)
    if disc < 0.0:
        return num_blocks
    return max(1, min(num_blocks, round((lin - math.sqrt(disc)) / 2.0)))

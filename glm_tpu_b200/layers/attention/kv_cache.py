"""Cache addressing: which GPU owns a position and where it sits in that GPU's slice.

The cache is either replicated (every GPU holds every row) or striped by position: pages of ``stripe * world`` positions, stripe ``s``
of a page on GPU ``s``.  Rows are written by ``qkv_a_post`` (only by the owner, only for active lanes); reads are bounded by the
lane's position, so stale rows are never visible.  Invalid positions are clamped and recorded in the status word, never dereferenced.
Parity: reference ``glm_tpu/layers/attention/kv_cache.py:31-426`` (block write validation, canonicalize, owner subset, gathers).
"""

from __future__ import annotations

import torch


def owner(position, stripe: int, world: int):
    return (position // stripe) % world


def local_row(position, stripe: int, world: int):
    return (position // (stripe * world)) * stripe + position % stripe


def owned_count(context_length: int, stripe: int, world: int, rank: int) -> int:
    page = stripe * world
    return (context_length // page) * stripe + min(max(context_length % page - rank * stripe, 0), stripe)


def owner_subset(positions: torch.Tensor, stripe: int, world: int, rank: int) -> torch.Tensor:
    """Local rows of the (ascending, ``-1`` padded) ``positions`` that this GPU holds, in the same order."""
    valid = positions >= 0
    mine = valid & (owner(positions.clamp(min=0), stripe, world) == rank)
    return local_row(positions[mine], stripe, world)

"""The parallel layout of one 8-GPU box.

One process drives one GPU.  Between blocks the hidden state is *replicated* on every GPU (a decode row is
12 KB, so replication is free and removes every reduction over a split hidden dimension).  Within a block:

* attention heads (q_b, kv_b, o_proj) are split over the GPUs (``heads_local = heads / world``);
* the dense MLP and the shared expert are split by intermediate columns;
* routed experts, one of two splits (``expert_split``):
  ``"whole"``: expert-parallel, expert ``e`` lives whole on GPU ``e // experts_local``.  A decode token's eight routes then land
  on the GPUs unevenly (the busiest GPU of eight streams ~2.6 experts where the average is one) and every GPU waits for the
  busiest at the all-reduce that follows.
  ``"sliced"``: every GPU holds a ``1/world`` slice of the intermediate columns of EVERY expert (the same cut as the shared expert
  and the dense MLP).  Each GPU then streams exactly ``top_k / world`` experts' worth of bytes per token whatever the routing,
  and the partial sums ride the all-reduce that the whole-expert split needs anyway; the hidden state is replicated, so neither
  split dispatches tokens.  Resident bytes are identical;
* the KV and index caches are striped by position (``config/cache.py``);
* lm_head is split by vocabulary rows; the embedding, router, q_a/kv_a and indexer tables are replicated.

The reference's fixed TPU mesh ``expert=8 x feature=4`` (``glm_tpu/config/parallel.py:9-10``,
``glm_tpu/distributed/mesh.py:31-57``) maps to: ``expert`` axis -> the ``world`` GPUs; ``feature`` axis ->
gone (hidden is replicated).
"""

from __future__ import annotations

import os
from dataclasses import dataclass

from glm_tpu_b200.config.model import ModelGeometry
from glm_tpu_b200.exceptions import PlanValidationError

RANK_AXIS = "gpu"


def default_expert_split(geometry, world: int) -> str:
    """``GLM_B200_EXPERT_SPLIT`` if set; else column-sliced experts wherever the slices fall on FP8 block boundaries (a decode
    token's routed bytes are then the same on every GPU whatever the routing), whole experts otherwise."""
    chosen = os.environ.get("GLM_B200_EXPERT_SPLIT", "").strip().lower()
    if chosen in ("whole", "sliced"):
        return chosen
    if world > 1 and geometry.num_routed_experts and geometry.moe_intermediate_size % world == 0:
        cols, (bn, bk) = geometry.moe_intermediate_size // world, geometry.fp8_block_shape
        if cols % bn == 0 and cols % bk == 0 and cols % 64 == 0:
            return "sliced"
    return "whole"


@dataclass(frozen=True)
class ParallelLayout:
    geometry: ModelGeometry
    world: int = 1
    rank: int = 0
    expert_split: str = "whole"

    def __post_init__(self) -> None:
        g = self.geometry
        if self.expert_split not in ("whole", "sliced"):
            raise PlanValidationError("expert_split is 'whole' or 'sliced'")
        if self.expert_split == "sliced" and g.num_routed_experts:
            cols, block = g.moe_intermediate_size // max(self.world, 1), g.fp8_block_shape
            if g.moe_intermediate_size % self.world or cols % block[0] or cols % block[1]:
                raise PlanValidationError(f"sliced experts need moe_intermediate_size / world = {cols} to be a multiple of the FP8 block {block}")
        if not 0 <= self.rank < self.world:
            raise PlanValidationError("rank must lie in [0, world)")
        for name, value in (
            ("attention_heads", g.attention_heads),
            ("num_routed_experts", g.num_routed_experts),
            ("dense_intermediate_size", g.dense_intermediate_size),
            ("moe_intermediate_size", g.moe_intermediate_size),
            ("vocab_size", g.vocab_size),
        ):
            if value % self.world:
                raise PlanValidationError(f"{name}={value} is not divisible by world={self.world}")

    @property
    def heads_local(self) -> int:
        return self.geometry.attention_heads // self.world

    @property
    def head_range(self) -> range:
        return range(self.rank * self.heads_local, (self.rank + 1) * self.heads_local)

    @property
    def experts_local(self) -> int:
        return self.geometry.num_routed_experts // self.world

    @property
    def expert_range(self) -> range:
        return range(self.rank * self.experts_local, (self.rank + 1) * self.experts_local)

    @property
    def sliced(self) -> bool:
        return self.expert_split == "sliced"

    @property
    def experts_resident(self) -> int:
        """How many experts this GPU holds a part of: all of them when sliced, its own when whole."""
        return self.geometry.num_routed_experts if self.sliced else self.experts_local

    @property
    def expert_base(self) -> int:
        """Global id of the first expert this GPU holds."""
        return 0 if self.sliced else self.rank * self.experts_local

    @property
    def moe_cols_local(self) -> int:
        """Intermediate columns of a routed expert that this GPU holds."""
        return self.geometry.moe_intermediate_size // self.world if self.sliced else self.geometry.moe_intermediate_size

    @property
    def moe_col_range(self) -> range:
        c = self.moe_cols_local
        return range(self.rank * c, (self.rank + 1) * c) if self.sliced else range(0, c)

    @property
    def dense_cols_local(self) -> int:
        return self.geometry.dense_intermediate_size // self.world

    @property
    def shared_cols_local(self) -> int:
        return self.geometry.moe_intermediate_size * self.geometry.num_shared_experts // self.world

    @property
    def vocab_local(self) -> int:
        return self.geometry.vocab_size // self.world

    def expert_owner(self, expert: int) -> int:
        return expert // self.experts_local

    def layout_summary(self) -> dict:
        """Which tensor is split how, and which exchange follows it (the mesh contract every rank must agree on)."""
        w = self.world
        return {
            "world": w,
            "hidden_state": "replicated",
            "embedding": "replicated",
            "q_a|kv_a|indexer_k|indexer_weights": "replicated (one fused projection)",
            "q_b,kv_b,o_proj": f"by attention head: {self.heads_local} of {self.geometry.attention_heads} per GPU; o_proj partials all-reduced",
            "indexer_q": "replicated",
            "dense_mlp": f"by column: {self.dense_cols_local} per GPU; down partials all-reduced",
            "shared_expert": f"by column: {self.shared_cols_local} per GPU; summed with the routed partials in one all-reduce",
            "routed_experts": (
                f"sliced by column: {self.moe_cols_local} of {self.geometry.moe_intermediate_size} columns of every expert per GPU (FP8 resident); partial route sums all-reduced"
                if self.sliced
                else f"whole experts: {self.experts_local} of {self.geometry.num_routed_experts} per GPU (FP8 resident); route sums all-reduced"
            ),
            "router": "replicated",
            "lm_head": f"by vocabulary row: {self.vocab_local} per GPU; packed (logit, id) candidates exchanged",
            "kv_cache,index_cache": "replicated, or striped by position in 64-row stripes (runner choice)",
            "reductions": "fp32 partial sums in rank order, one bf16 rounding",
        }

    @property
    def layout_hash(self) -> str:
        """SHA-256 of the canonical summary + geometry hash: workers compare it before they exchange anything."""
        import hashlib

        from glm_tpu_b200.utils.json_utils import canonical_hash_bytes

        return hashlib.sha256(canonical_hash_bytes({"layout": self.layout_summary(), "geometry": self.geometry.geometry_hash})).hexdigest()

    def describe(self) -> dict:
        return {
            "world": self.world,
            "rank": self.rank,
            "hidden": "replicated",
            "heads_local": self.heads_local,
            "experts_local": self.experts_local,
            "expert_split": self.expert_split,
            "moe_cols_local": self.moe_cols_local,
            "dense_cols_local": self.dense_cols_local,
            "shared_cols_local": self.shared_cols_local,
            "vocab_local": self.vocab_local,
            "kv_cache": "position-striped",
        }

"""The parallel layout of one 8-GPU box.

One process drives one GPU.  Between blocks the hidden state is *replicated* on every GPU (a decode row is
12 KB, so replication is free and removes every reduction over a split hidden dimension).  Within a block:

* attention heads (q_b, kv_b, o_proj) are split over the GPUs (``heads_local = heads / world``);
* the dense MLP and the shared expert are split by intermediate columns;
* routed experts are expert-parallel: expert ``e`` lives on GPU ``e // experts_local``;
* the KV and index caches are striped by position (``config/cache.py``);
* lm_head is split by vocabulary rows; the embedding, router, q_a/kv_a and indexer tables are replicated.

The reference's fixed TPU mesh ``expert=8 x feature=4`` (``glm_tpu/config/parallel.py:9-10``,
``glm_tpu/distributed/mesh.py:31-57``) maps to: ``expert`` axis -> the ``world`` GPUs; ``feature`` axis ->
gone (hidden is replicated).
"""

from __future__ import annotations

from dataclasses import dataclass

from glm_tpu_b200.config.model import ModelGeometry
from glm_tpu_b200.exceptions import PlanValidationError

RANK_AXIS = "gpu"


@dataclass(frozen=True)
class ParallelLayout:
    geometry: ModelGeometry
    world: int = 1
    rank: int = 0

    def __post_init__(self) -> None:
        g = self.geometry
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
            "routed_experts": f"whole experts: {self.experts_local} of {self.geometry.num_routed_experts} per GPU (FP8 resident); route sums all-reduced",
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
            "dense_cols_local": self.dense_cols_local,
            "shared_cols_local": self.shared_cols_local,
            "vocab_local": self.vocab_local,
            "kv_cache": "position-striped",
        }

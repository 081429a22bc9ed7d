"""Cache configuration and the numerical contracts of attention, the DSA indexer and the MoE.

The KV cache holds one row per position and layer: ``[latent (kv_lora_rank) | rotated RoPE key]`` in
bf16 (no padding column: a 1152-byte row is already 16-byte aligned for vector and TMA access).  The
index cache holds one bf16 key of ``index_head_dim`` per position for every *full* indexer layer.

Both caches are striped by position over the ``world`` GPUs of the box: positions are cut into stripes
of ``stripe`` rows, stripe ``s`` belongs to GPU ``s % world``, and a GPU stores its stripes back to back.
A page is ``stripe * world`` positions, so with 8 GPUs and 64-row stripes the layout is the 512-position
page of the reference (``glm_tpu/config/cache.py:67-95``, owner ``(pos % 512) // 64``).

Parity: reference ``glm_tpu/config/cache.py:21-64`` (MLA contract), ``:98-143`` (DSA contract),
``:221-367`` (``CacheConfig``).
"""

from __future__ import annotations

from dataclasses import dataclass, field

from glm_tpu_b200.config.model import ModelGeometry
from glm_tpu_b200.exceptions import PlanValidationError

CAPACITY_PROFILES = (8192, 32768, 166912, 262144)


@dataclass(frozen=True)
class MlaNumericalContract:
    """Absorbed multi-head latent attention arithmetic.

    Scores are fp32 ``(q_c . latent + q_rope . k_rope) * qk_head_dim**-0.5``; softmax statistics are fp32;
    the unnormalized probability is rounded to bf16 before it multiplies the latent; the result is
    normalized once at the end and rounded to bf16.  A row with no valid key yields zeros.
    """

    score_dtype: str = "float32"
    probability_rounding: str = "unnormalized_bf16_before_pv"
    position_order: str = "ascending_global_position"
    empty_row: str = "zeros"


@dataclass(frozen=True)
class DsaNumericalContract:
    """Lightning-indexer arithmetic and the top-k order.

    ``score = sum_h w_h * relu(q_h . k * index_head_dim**-0.5)`` in fp32 with ``w = (x @ weights_proj.T) *
    index_heads**-0.5``.  Selection is by descending score, ties to the lowest position, under the total
    fp32 order in which ``+0 > -0``; positions at or beyond the context length never win; the tail of a
    short selection is ``-1``; the selected list is returned in ascending position order.
    """

    tie_policy: str = "descending_score_then_lowest_position"
    sentinel: int = -1
    key_norm_eps: float = 1e-6
    nonfinite_score: str = "health_false"


@dataclass(frozen=True)
class MoeNumericalContract:
    """Router and expert arithmetic.

    Router logits, sigmoid and weights are fp32; the correction bias enters the choice only; ties go to the
    lowest expert id; weights are ``s / (sum s + 1e-20)``.  Expert gate/up accumulate in fp32 and round to
    bf16; ``act = bf16(silu(g) * u)`` from the rounded values; the down output rounds to bf16 and is scaled by
    the bf16 route weight; routes are summed in fp32; ``out = bf16(bf16(routed * scale) + shared)``.
    """

    router_dtype: str = "float32"
    route_sum_dtype: str = "float32"
    weight_decode: str = "bf16(f32(e4m3)*scale_inv)"


@dataclass(frozen=True)
class CacheConfig:
    geometry: ModelGeometry
    context_capacity: int
    world: int = 1
    stripe: int = 64
    lanes: int = 1
    mla: MlaNumericalContract = field(default_factory=MlaNumericalContract)
    dsa: DsaNumericalContract = field(default_factory=DsaNumericalContract)
    moe: MoeNumericalContract = field(default_factory=MoeNumericalContract)

    def __post_init__(self) -> None:
        if self.world < 1 or self.stripe < 1 or self.lanes < 1:
            raise PlanValidationError("world, stripe and lanes must be positive")
        if self.lanes > 8:
            raise PlanValidationError("at most 8 concurrent lanes are supported")
        if self.context_capacity % self.page:
            raise PlanValidationError(f"context capacity {self.context_capacity} is not a multiple of the page ({self.page})")

    @property
    def page(self) -> int:
        return self.stripe * self.world

    @property
    def local_capacity(self) -> int:
        return self.context_capacity // self.world

    def owner(self, position: int) -> int:
        return (position // self.stripe) % self.world

    def local_row(self, position: int) -> int:
        return (position // self.page) * self.stripe + position % self.stripe

    def global_position(self, rank: int, local_row: int) -> int:
        return (local_row // self.stripe) * self.page + rank * self.stripe + local_row % self.stripe

    def owned_count(self, rank: int, context_length: int) -> int:
        """How many of the positions ``0..context_length-1`` are stored on ``rank``."""
        full_pages, rest = divmod(context_length, self.page)
        extra = min(max(rest - rank * self.stripe, 0), self.stripe)
        return full_pages * self.stripe + extra

    @property
    def kv_cache_shape(self) -> tuple[int, int, int, int]:
        g = self.geometry
        return (self.lanes, g.num_layers, self.local_capacity, g.kv_row_width)

    @property
    def index_cache_shape(self) -> tuple[int, int, int, int]:
        g = self.geometry
        return (self.lanes, len(g.full_layers), self.local_capacity, g.index_head_dim)

    def cache_bytes_per_gpu(self) -> int:
        kv = 1
        for n in self.kv_cache_shape:
            kv *= n
        ix = 1
        for n in self.index_cache_shape:
            ix *= n
        return 2 * (kv + ix)

"""Model identity and geometry of ``GlmMoeDsaForCausalLM`` (GLM-5.3).

The geometry is the set of plain dimensions every other layer of the engine is
derived from.  It can be built from a Hugging Face ``config.json`` mapping
(``ModelGeometry.from_hf_config``), from the built-in GLM-5.3 constants
(``glm53_geometry``), truncated to the first ``n`` layers for scaling runs
(``ModelGeometry.truncated``) or shrunk to a CPU-sized fixture (``tiny_geometry``).

Parity: reference ``glm_tpu/config/model.py:70-256`` (``ModelGeometry``,
``geometry_hash``) and the pinned ``hf_config/config.json``.
"""

from __future__ import annotations

import dataclasses
import hashlib
from dataclasses import dataclass
from typing import Any, Mapping

from glm_tpu_b200.utils.json_utils import canonical_hash_bytes

MODEL_ID = "zai-org/GLM-5.3"
MODEL_REVISION = "aca966e4e02791568aa6a4ced368624b3d897f42"
EOS_IDS = (154820, 154827, 154829)


ASSUMED_SWITCHES = {
    "hidden_act": "silu",             # SwiGLU with SiLU in dense, shared and routed MLPs
    "norm_topk_prob": True,           # the top-k route weights are renormalised to sum to one before the scaling factor
    "attention_bias": False,          # no bias on the attention projections
    "tie_word_embeddings": False,     # lm_head has its own table
    "rope_interleave": True,          # rotary pairs are (2i, 2i + 1) in the attention heads ...
    "indexer_rope_interleave": True,  # ... and in the indexer's query and key
    "moe_layer_freq": 1,              # every layer after the dense ones is a MoE layer (mlp_layer_types says which)
}


@dataclass(frozen=True)
class ModelGeometry:
    vocab_size: int
    hidden_size: int
    num_layers: int
    attention_heads: int
    q_lora_rank: int
    kv_lora_rank: int
    qk_nope_head_dim: int
    qk_rope_head_dim: int
    v_head_dim: int
    dense_intermediate_size: int
    moe_intermediate_size: int
    num_routed_experts: int
    routed_top_k: int
    num_shared_experts: int
    routed_scaling_factor: float
    index_heads: int
    index_head_dim: int
    index_top_k: int
    indexer_types: tuple[str, ...]
    mlp_layer_types: tuple[str, ...]
    rope_theta: float
    rms_norm_eps: float
    fp8_block_shape: tuple[int, int] = (128, 128)
    eos_ids: tuple[int, ...] = EOS_IDS

    def __post_init__(self) -> None:
        if len(self.indexer_types) != self.num_layers or len(self.mlp_layer_types) != self.num_layers:
            raise ValueError("per-layer type lists must have num_layers entries")
        if self.indexer_types[0] != "full":
            raise ValueError("layer 0 must be a full DSA layer")
        if set(self.indexer_types) - {"full", "shared"}:
            raise ValueError("indexer types are 'full' or 'shared'")
        if set(self.mlp_layer_types) - {"dense", "sparse"}:
            raise ValueError("mlp layer types are 'dense' or 'sparse'")
        if self.qk_rope_head_dim % 2 or self.index_head_dim < self.qk_rope_head_dim:
            raise ValueError("RoPE width must be even and fit in the indexer head")
        if self.routed_top_k > self.num_routed_experts:
            raise ValueError("routed_top_k exceeds the expert count")

    # ---- derived sizes -------------------------------------------------
    @property
    def qk_head_dim(self) -> int:
        return self.qk_nope_head_dim + self.qk_rope_head_dim

    @property
    def kv_row_width(self) -> int:
        """Width of one cached row: the normalized latent followed by the rotated RoPE key."""
        return self.kv_lora_rank + self.qk_rope_head_dim

    @property
    def kv_b_rows_per_head(self) -> int:
        return self.qk_nope_head_dim + self.v_head_dim

    @property
    def full_layers(self) -> tuple[int, ...]:
        return tuple(i for i, kind in enumerate(self.indexer_types) if kind == "full")

    @property
    def sparse_layers(self) -> tuple[int, ...]:
        return tuple(i for i, kind in enumerate(self.mlp_layer_types) if kind == "sparse")

    def index_slot(self, layer: int) -> int:
        """Slot of ``layer``'s index cache (a shared layer maps to its preceding full layer's slot)."""
        return sum(1 for kind in self.indexer_types[: layer + 1] if kind == "full") - 1

    # ---- constructors --------------------------------------------------
    @classmethod
    def from_hf_config(cls, config: Mapping[str, Any]) -> "ModelGeometry":
        if config.get("model_type") != "glm_moe_dsa":
            raise ValueError("not a glm_moe_dsa config")
        quant = config.get("quantization_config") or {}
        block = tuple(quant.get("weight_block_size", (128, 128)))
        eos = config.get("eos_token_id", EOS_IDS)
        eos = (eos,) if isinstance(eos, int) else tuple(eos)
        if config.get("scoring_func", "sigmoid") != "sigmoid" or config.get("topk_method", "noaux_tc") != "noaux_tc":
            raise ValueError("only the sigmoid noaux_tc router is supported")
        if config.get("n_group", 1) != 1 or config.get("topk_group", 1) != 1:
            raise ValueError("grouped routing is not part of this model")
        # Switches of the architecture that the kernels assume one way.  They are not part of the geometry (and not of its hash):
        # a configuration that sets one of them the other way describes another computation and is refused, not approximated.
        for key, assumed in ASSUMED_SWITCHES.items():
            if config.get(key, assumed) != assumed:
                raise ValueError(f"{key} = {config[key]!r} is not supported (the engine computes {key} = {assumed!r})")
        return cls(
            vocab_size=int(config["vocab_size"]),
            hidden_size=int(config["hidden_size"]),
            num_layers=int(config["num_hidden_layers"]),
            attention_heads=int(config["num_attention_heads"]),
            q_lora_rank=int(config["q_lora_rank"]),
            kv_lora_rank=int(config["kv_lora_rank"]),
            qk_nope_head_dim=int(config["qk_nope_head_dim"]),
            qk_rope_head_dim=int(config["qk_rope_head_dim"]),
            v_head_dim=int(config["v_head_dim"]),
            dense_intermediate_size=int(config["intermediate_size"]),
            moe_intermediate_size=int(config["moe_intermediate_size"]),
            num_routed_experts=int(config["n_routed_experts"]),
            routed_top_k=int(config["num_experts_per_tok"]),
            num_shared_experts=int(config.get("n_shared_experts", 1)),
            routed_scaling_factor=float(config["routed_scaling_factor"]),
            index_heads=int(config["index_n_heads"]),
            index_head_dim=int(config["index_head_dim"]),
            index_top_k=int(config["index_topk"]),
            indexer_types=tuple(config["indexer_types"]),
            mlp_layer_types=tuple(config["mlp_layer_types"]),
            rope_theta=float(config["rope_parameters"]["rope_theta"]),
            rms_norm_eps=float(config["rms_norm_eps"]),
            fp8_block_shape=(int(block[0]), int(block[1])),
            eos_ids=eos,
        )

    def truncated(self, num_layers: int) -> "ModelGeometry":
        """The same architecture cut to its first ``num_layers`` layers (scaling runs on fewer GPUs)."""
        if not 1 <= num_layers <= self.num_layers:
            raise ValueError("truncation must keep between 1 and num_layers layers")
        return dataclasses.replace(
            self,
            num_layers=num_layers,
            indexer_types=self.indexer_types[:num_layers],
            mlp_layer_types=self.mlp_layer_types[:num_layers],
        )

    def as_dict(self) -> dict[str, Any]:
        out = dataclasses.asdict(self)
        for key in ("indexer_types", "mlp_layer_types", "fp8_block_shape", "eos_ids"):
            out[key] = list(out[key])
        return out

    @property
    def geometry_hash(self) -> str:
        """SHA-256 of the canonical (ASCII, sorted) JSON of every field."""
        return hashlib.sha256(canonical_hash_bytes(self.as_dict())).hexdigest()

    # ---- parameter accounting -----------------------------------------
    def routed_bytes_per_layer(self) -> int:
        per = 3 * self.moe_intermediate_size * self.hidden_size
        return self.num_routed_experts * per


def _glm53_layer_types() -> tuple[tuple[str, ...], tuple[str, ...]]:
    # Layers 0-2 are full indexers; after that one full layer every fourth layer
    # (index_topk_freq 4, index_skip_topk_offset 3): 6, 10, 14, ... 74.
    indexer = tuple("full" if (i < 3 or (i >= 6 and (i - 6) % 4 == 0)) else "shared" for i in range(78))
    mlp = tuple("dense" if i < 3 else "sparse" for i in range(78))
    return indexer, mlp


def glm53_geometry() -> ModelGeometry:
    """The GLM-5.3 geometry (78 layers, hidden 6144, 256 routed experts, DSA top-2048)."""
    indexer, mlp = _glm53_layer_types()
    return ModelGeometry(
        vocab_size=154880,
        hidden_size=6144,
        num_layers=78,
        attention_heads=64,
        q_lora_rank=2048,
        kv_lora_rank=512,
        qk_nope_head_dim=192,
        qk_rope_head_dim=64,
        v_head_dim=256,
        dense_intermediate_size=12288,
        moe_intermediate_size=2048,
        num_routed_experts=256,
        routed_top_k=8,
        num_shared_experts=1,
        routed_scaling_factor=2.5,
        index_heads=32,
        index_head_dim=128,
        index_top_k=2048,
        indexer_types=indexer,
        mlp_layer_types=mlp,
        rope_theta=8000000.0,
        rms_norm_eps=1e-5,
    )


def tiny_geometry() -> ModelGeometry:
    """CPU-sized fixture: 2 layers (dense then MoE), hidden 256, 8 experts top-2, DSA top-16."""
    return ModelGeometry(
        vocab_size=1024,
        hidden_size=256,
        num_layers=2,
        attention_heads=4,
        q_lora_rank=128,
        kv_lora_rank=64,
        qk_nope_head_dim=32,
        qk_rope_head_dim=16,
        v_head_dim=32,
        dense_intermediate_size=512,
        moe_intermediate_size=128,
        num_routed_experts=8,
        routed_top_k=2,
        num_shared_experts=1,
        routed_scaling_factor=2.5,
        index_heads=2,
        index_head_dim=32,
        index_top_k=16,
        indexer_types=("full", "shared"),
        mlp_layer_types=("dense", "sparse"),
        rope_theta=8000000.0,
        rms_norm_eps=1e-5,
        eos_ids=(1020, 1021, 1022),
    )


def small_geometry(num_layers: int = 4) -> ModelGeometry:
    """Mid-sized fixture that exercises IndexShare groups and several MoE layers (GPU tests)."""
    kinds = ("full", "shared", "full", "shared", "shared", "shared", "full", "shared")
    return ModelGeometry(
        vocab_size=2048,
        hidden_size=512,
        num_layers=num_layers,
        attention_heads=8,
        q_lora_rank=256,
        kv_lora_rank=128,
        qk_nope_head_dim=64,
        qk_rope_head_dim=32,
        v_head_dim=64,
        dense_intermediate_size=1024,
        moe_intermediate_size=256,
        num_routed_experts=16,
        routed_top_k=4,
        num_shared_experts=1,
        routed_scaling_factor=2.5,
        index_heads=4,
        index_head_dim=64,
        index_top_k=32,
        indexer_types=kinds[:num_layers],
        mlp_layer_types=("dense",) + ("sparse",) * (num_layers - 1),
        rope_theta=8000000.0,
        rms_norm_eps=1e-5,
        eos_ids=(2040, 2041, 2042),
    )

"""Declarative placement: which Hugging Face source tensor feeds which packed tensor, on which GPU.

Source names are the Hugging Face ones (``...experts.{e}.gate_proj.weight`` + ``.weight_scale_inv`` per expert,
``...q_a_proj.weight`` + ``.weight_scale_inv``, bf16 norms/router/indexer tables).  Packed (runtime) names are the ones
of ``models/glm_moe_dsa/weights.py``: FP8 pairs become ``<prefix>.weight_bits`` / ``<prefix>.scale_inv``, routed experts
are stacked per layer and cut per GPU -- whole experts (``split="whole"``: expert ``e`` goes to GPU ``e // experts_local``) or
a column slice of every expert (``split="sliced"``: GPU ``r`` gets rows ``[r c, (r + 1) c)`` of every gate/up table and the same
columns of every down table, with the block scales cut alongside) -- everything else goes to the shared file whole (each GPU
decodes and slices it at load).  ``require_source_contract`` binds every source role to the exact dtype and shape the geometry
implies; tensors of layers beyond ``num_layers`` (a truncation, the unused multi-token-prediction layer) are skipped.

Parity: reference ``glm_tpu/model_loader/placement.py:24-39,75-196,416-570``.
"""

from __future__ import annotations

import re
from dataclasses import dataclass

from glm_tpu_b200.config.model import ModelGeometry
from glm_tpu_b200.exceptions import PlanValidationError
from glm_tpu_b200.models.glm_moe_dsa.weights import plain_shapes, projection_shapes

_LAYER = re.compile(r"model\.layers\.(\d+)\.")
_ROUTED = re.compile(r"(model\.layers\.(\d+)\.mlp\.experts)\.(\d+)\.(gate_proj|up_proj|down_proj)\.(weight|weight_scale_inv)")


@dataclass(frozen=True)
class Placement:
    source: str
    target: str  # packed tensor name
    file: str  # "shared" or "experts"
    rank: int | None  # owning GPU for expert tensors (None: shared file, or every GPU takes a slice)
    expert_slot: int | None  # index inside the stacked per-rank tensor
    dtype: str
    shape: tuple  # of the source tensor
    axis: int | None = None  # sliced experts: the axis of the source tensor that is cut over the GPUs ...
    unit: int = 0  # ... and how many entries of it each GPU takes

    def piece_shape(self) -> tuple:
        """Shape of what one GPU stores of this source tensor."""
        if self.axis is None:
            return tuple(self.shape)
        return tuple(self.unit if a == self.axis else d for a, d in enumerate(self.shape))

    def cut(self, tensor, rank: int):
        """One GPU's part of the source tensor."""
        if self.axis is None:
            return tensor
        return tensor.narrow(self.axis, rank * self.unit, self.unit)


def _blocks(shape, block):
    return (*shape[:-2], -(-shape[-2] // block[0]), -(-shape[-1] // block[1]))


def expected_sources(g: ModelGeometry) -> dict:
    """Every source tensor the geometry implies: name -> (dtype, shape)."""
    out = {"model.embed_tokens.weight": ("BF16", (g.vocab_size, g.hidden_size)), "lm_head.weight": ("BF16", (g.vocab_size, g.hidden_size)),
           "model.norm.weight": ("BF16", (g.hidden_size,))}
    for i in range(g.num_layers):
        for prefix, shape in projection_shapes(g, i).items():
            if ".experts." in prefix:
                stem, proj = prefix.rsplit(".", 1)
                for e in range(shape[0]):
                    out[f"{stem}.{e}.{proj}.weight"] = ("F8_E4M3", tuple(shape[1:]))
                    out[f"{stem}.{e}.{proj}.weight_scale_inv"] = ("F32", _blocks(shape[1:], g.fp8_block_shape))
            else:
                out[prefix + ".weight"] = ("F8_E4M3", tuple(shape))
                out[prefix + ".weight_scale_inv"] = ("F32", _blocks(shape, g.fp8_block_shape))
        for name, (shape, dtype) in plain_shapes(g, i).items():
            out[name] = ("F32" if "e_score_correction_bias" in name else "BF16", tuple(shape))
    return out


def require_source_contract(name: str, dtype: str, shape: tuple, g: ModelGeometry, expected: dict | None = None) -> bool:
    """True if the tensor is used; raises on a used tensor whose dtype/shape drifted; False for skipped layers."""
    m = _LAYER.match(name)
    if m and int(m.group(1)) >= g.num_layers:
        return False
    expected = expected if expected is not None else expected_sources(g)
    if name not in expected:
        raise PlanValidationError(f"no source geometry contract for {name!r}")
    if (dtype, tuple(shape)) != expected[name]:
        raise PlanValidationError(f"source geometry drifted for {name!r}: observed {(dtype, tuple(shape))}, expected {expected[name]}")
    return True


def _check_split(g: ModelGeometry, world: int, split: str) -> None:
    if split not in ("whole", "sliced"):
        raise PlanValidationError("split is 'whole' or 'sliced'")
    if g.num_routed_experts % world:
        raise PlanValidationError("experts do not divide over the GPUs")
    if split == "sliced":
        cols, (bn, bk) = g.moe_intermediate_size // world, g.fp8_block_shape
        if g.moe_intermediate_size % world or cols % bn or cols % bk:
            raise PlanValidationError(f"sliced experts need moe_intermediate_size / world = {cols} to be a multiple of the FP8 block")


def placements(g: ModelGeometry, world: int, split: str = "whole") -> list[Placement]:
    """The full plan, in a fixed order."""
    _check_split(g, world, split)
    per = g.num_routed_experts // world
    cols, (bn, bk) = g.moe_intermediate_size // world, g.fp8_block_shape
    plan = []
    for name, (dtype, shape) in expected_sources(g).items():
        m = _ROUTED.fullmatch(name)
        if m:
            stem, _, expert, proj, role = m.groups()
            e = int(expert)
            suffix = "weight_bits" if role == "weight" else "scale_inv"
            if split == "whole":
                plan.append(Placement(name, f"{stem}.{proj}.{suffix}", "experts", e // per, e % per, dtype, shape))
            else:  # gate/up [I, H]: rows; down [H, I]: columns; scales in blocks
                axis = 1 if proj == "down_proj" else 0
                unit = cols if role == "weight" else cols // (bk if axis == 1 else bn)
                plan.append(Placement(name, f"{stem}.{proj}.{suffix}", "experts", None, e, dtype, shape, axis, unit))
        elif name.endswith(".weight_scale_inv"):
            plan.append(Placement(name, name[: -len(".weight_scale_inv")] + ".scale_inv", "shared", None, None, dtype, shape))
        elif dtype == "F8_E4M3":
            plan.append(Placement(name, name[: -len(".weight")] + ".weight_bits", "shared", None, None, dtype, shape))
        else:
            plan.append(Placement(name, name, "shared", None, None, dtype, shape))
    return plan


def packed_tensor_shapes(g: ModelGeometry, world: int, rank: int | None, split: str = "whole") -> dict:
    """Names, dtypes and shapes a packed file must hold (``rank=None``: the shared file)."""
    stacked = g.num_routed_experts if split == "sliced" else g.num_routed_experts // world
    out = {}
    for p in placements(g, world, split):
        if rank is None and p.file == "shared":
            out[p.target] = (p.dtype, p.shape)
        elif rank is not None and p.file == "experts" and p.rank in (None, rank):
            out[p.target] = (p.dtype, (stacked, *p.piece_shape()))
    return out

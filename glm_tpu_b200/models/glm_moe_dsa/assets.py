"""Pinned model assets: the Hugging Face style ``config.json`` and ``generation_config.json`` of GLM-5.3 that ship with the package.

The files under ``hf_config/`` are written from :func:`glm_tpu_b200.config.model.glm53_geometry` (``write_assets``) and pinned by
SHA-256 here; ``load_pinned_geometry`` refuses a file whose bytes differ, and the geometry rebuilt from the file must equal the
built-in one.  A downloaded checkpoint's own ``config.json`` goes through the same ``ModelGeometry.from_hf_config`` and its
``geometry_hash`` is compared with the pinned one before anything is packed.  The chat template is code
(``glm_tpu_b200/tokenizer/chat_template.py``), not a Jinja file: nothing here evaluates templates.

Reference counterpart: ``glm_tpu/models/glm_moe_dsa/hf_config/`` with the pins in ``glm_tpu/config/model.py:27-45``.
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path

from glm_tpu_b200.config.model import MODEL_ID, MODEL_REVISION, ModelGeometry, glm53_geometry

ASSET_DIR = Path(__file__).resolve().parent / "hf_config"
PINS = {
    "config.json": "59855ce1c173debb65b5b98ab36a07b3a2bc928dbc50150c89b714d0fba31240",
    "generation_config.json": "aad734bff2a95e4db0513accca3e1dff5c5b9b0ba486332aa4e00be8e4862030",
}


class AssetMismatch(ValueError):
    """A pinned asset is missing or its bytes differ from the pin."""


def asset_bytes(name: str) -> bytes:
    if name not in PINS:
        raise AssetMismatch(f"{name} is not a pinned asset")
    path = ASSET_DIR / name
    if not path.is_file():
        raise AssetMismatch(f"{path} is missing")
    data = path.read_bytes()
    digest = hashlib.sha256(data).hexdigest()
    if digest != PINS[name]:
        raise AssetMismatch(f"{name}: sha256 {digest} differs from the pin {PINS[name]}")
    return data


def load_pinned_geometry() -> ModelGeometry:
    """The geometry rebuilt from the pinned ``config.json``; it must be the built-in GLM-5.3 geometry."""
    g = ModelGeometry.from_hf_config(json.loads(asset_bytes("config.json")))
    if g.geometry_hash != glm53_geometry().geometry_hash:
        raise AssetMismatch("the pinned config.json no longer describes the built-in GLM-5.3 geometry")
    return g


def generation_config() -> dict:
    return json.loads(asset_bytes("generation_config.json"))


def check_source_config(config: dict) -> ModelGeometry:
    """Geometry of a checkpoint's own ``config.json``; refused unless it hashes like the pinned one (same architecture)."""
    g = ModelGeometry.from_hf_config(config)
    pinned = load_pinned_geometry()
    if g.geometry_hash != pinned.geometry_hash:
        raise AssetMismatch(f"checkpoint geometry {g.geometry_hash[:12]} differs from the pinned {MODEL_ID}@{MODEL_REVISION[:8]} geometry "
                            f"{pinned.geometry_hash[:12]}")
    return g


def write_assets(root: Path = ASSET_DIR) -> dict:
    """Regenerate the asset files from the built-in geometry; returns ``{name: sha256}`` (update ``PINS`` with it)."""
    from glm_tpu_b200.model_loader.export import hf_config

    g = glm53_geometry()
    cfg = hf_config(g)
    cfg["_source"] = {"model_id": MODEL_ID, "revision": MODEL_REVISION,
                      "note": "written from ModelGeometry by glm_tpu_b200.models.glm_moe_dsa.assets.write_assets"}
    gen = {"do_sample": False, "eos_token_id": list(g.eos_ids), "temperature": None, "top_p": None,
           "_note": "greedy decoding only: sampling parameters are refused by the API"}
    root.mkdir(parents=True, exist_ok=True)
    out = {}
    for name, value in (("config.json", cfg), ("generation_config.json", gen)):
        data = (json.dumps(value, sort_keys=True, indent=1) + "\n").encode()
        (root / name).write_bytes(data)
        out[name] = hashlib.sha256(data).hexdigest()
    return out

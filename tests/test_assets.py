"""Pinned model assets: bytes match their pins, the geometry round-trips, and a tampered or foreign config is refused."""

import json

import pytest

from glm_tpu_b200.config.model import glm53_geometry, tiny_geometry
from glm_tpu_b200.model_loader.export import hf_config
from glm_tpu_b200.models.glm_moe_dsa import assets


def test_pinned_assets_match_and_round_trip(tmp_path):
    assert assets.load_pinned_geometry() == glm53_geometry()
    gen = assets.generation_config()
    assert gen["do_sample"] is False and tuple(gen["eos_token_id"]) == glm53_geometry().eos_ids
    assert assets.write_assets(tmp_path) == assets.PINS  # regenerating from the geometry reproduces the pinned bytes


def test_tampered_asset_is_refused(tmp_path, monkeypatch):
    assets.write_assets(tmp_path)
    cfg = json.loads((tmp_path / "config.json").read_text())
    cfg["num_hidden_layers"] = 77
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    monkeypatch.setattr(assets, "ASSET_DIR", tmp_path)
    with pytest.raises(assets.AssetMismatch, match="differs from the pin"):
        assets.load_pinned_geometry()
    with pytest.raises(assets.AssetMismatch, match="not a pinned asset"):
        assets.asset_bytes("tokenizer.json")


def test_source_config_of_another_architecture_is_refused():
    assert assets.check_source_config(hf_config(glm53_geometry())) == glm53_geometry()
    with pytest.raises(assets.AssetMismatch, match="differs from the pinned"):
        assets.check_source_config(hf_config(tiny_geometry()))

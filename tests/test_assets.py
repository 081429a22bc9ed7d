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


def test_architecture_switches_the_kernels_assume_are_checked():
    """A configuration may carry the switches of the published one (they are not part of the geometry); set the other way they
    describe another computation and the configuration is refused."""
    import json

    from glm_tpu_b200.config.model import ASSUMED_SWITCHES, ModelGeometry, glm53_geometry
    from glm_tpu_b200.models.glm_moe_dsa import assets

    base = json.loads(assets.asset_bytes("config.json"))
    published = dict(base, hidden_act="silu", norm_topk_prob=True, attention_bias=False, tie_word_embeddings=False, rope_interleave=True,
                     indexer_rope_interleave=True, moe_layer_freq=1, first_k_dense_replace=3, num_nextn_predict_layers=1, use_cache=True,
                     transformers_version="5.0.0", max_position_embeddings=202752)
    assert ModelGeometry.from_hf_config(published).geometry_hash == glm53_geometry().geometry_hash  # extra keys change nothing
    other = {"hidden_act": "gelu", "norm_topk_prob": False, "attention_bias": True, "tie_word_embeddings": True, "rope_interleave": False,
             "indexer_rope_interleave": False, "moe_layer_freq": 2}
    assert set(other) == set(ASSUMED_SWITCHES)
    for key, value in other.items():
        with pytest.raises(ValueError, match=f"{key} = {value!r} is not supported"):
            ModelGeometry.from_hf_config(dict(published, **{key: value}))
        with pytest.raises(ValueError):
            assets.check_source_config(dict(published, **{key: value}))
    for key, value, sentence in (("scoring_func", "softmax", "sigmoid noaux_tc"), ("topk_method", "greedy", "sigmoid noaux_tc"),
                                 ("n_group", 8, "grouped routing"), ("model_type", "deepseek_v3", "not a glm_moe_dsa")):
        with pytest.raises(ValueError, match=sentence):
            ModelGeometry.from_hf_config(dict(published, **{key: value}))

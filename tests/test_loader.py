"""Checkpoint pipeline on a tiny model: export -> inventory -> marker -> pack -> verify -> load, plus tamper cases."""

import json
import os

import pytest
import torch

from glm_tpu_b200.config.model import tiny_geometry
from glm_tpu_b200.config.parallel import ParallelLayout
from glm_tpu_b200.exceptions import CheckpointValidationError, PlanValidationError
from glm_tpu_b200.executor.pack_job import pack_checkpoint
from glm_tpu_b200.model_loader import export, placement, source_inventory, source_marker
from glm_tpu_b200.model_loader.sharded_state import format as fmt
from glm_tpu_b200.model_loader.sharded_state import loader, seal, verify
from glm_tpu_b200.models.glm_moe_dsa.weights import random_checkpoint, shard_checkpoint


@pytest.fixture(scope="module")
def packed(tmp_path_factory):
    root = tmp_path_factory.mktemp("ckpt")
    g = tiny_geometry()
    arrays = random_checkpoint(g, seed=3)
    export.export_source(arrays, g, root / "src", shards=3)
    source_marker.mark_source(root / "src")
    report = pack_checkpoint(root / "src", root / "packed", 2, jobs=1)
    return g, arrays, root, report


def test_canonical_file_is_deterministic(tmp_path):
    t = {"b": torch.arange(6, dtype=torch.float32).reshape(2, 3), "a": torch.ones(4, dtype=torch.bfloat16)}
    r1 = fmt.write_file(tmp_path / "x.safetensors", t, {"k": "v"})
    r2 = fmt.write_file(tmp_path / "y.safetensors", dict(reversed(list(t.items()))), {"k": "v"})
    assert r1["sha256"] == r2["sha256"] == fmt.file_sha256(tmp_path / "x.safetensors")
    header, start = fmt.read_header(tmp_path / "x.safetensors")
    assert start % 8 == 0 and torch.equal(fmt.read_tensor(tmp_path / "x.safetensors", header, start, "b"), t["b"])


def test_fp8_nan_codes_are_refused(tmp_path):
    bits = torch.tensor([[0x10, 0x7F]], dtype=torch.uint8)
    with pytest.raises(CheckpointValidationError, match="NaN"):
        fmt.write_file(tmp_path / "n.safetensors", {"w": bits}, {}, {"w"})


def test_header_bounds(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\xff" * 8 + b"{}")
    with pytest.raises(CheckpointValidationError):
        fmt.read_header(p)


def test_inventory_is_header_only_and_content_addressed(packed):
    g, arrays, root, _ = packed
    inv = source_inventory.read_source_inventory(root / "src")
    assert set(inv.tensors) == set(placement.expected_sources(g))
    assert source_inventory.authenticated_inventory(root / "src", inv.sha256).sha256 == inv.sha256
    with pytest.raises(CheckpointValidationError):
        source_inventory.authenticated_inventory(root / "src", "0" * 64)


def test_source_contract_rejects_drift():
    g = tiny_geometry()
    name = "model.layers.0.self_attn.q_a_proj.weight"
    assert placement.require_source_contract(name, "F8_E4M3", (g.q_lora_rank, g.hidden_size), g)
    with pytest.raises(PlanValidationError, match="drifted"):
        placement.require_source_contract(name, "BF16", (g.q_lora_rank, g.hidden_size), g)
    with pytest.raises(PlanValidationError, match="no source geometry"):
        placement.require_source_contract("model.layers.0.self_attn.bogus.weight", "BF16", (1,), g)
    assert placement.require_source_contract(f"model.layers.{g.num_layers}.anything", "BF16", (1,), g) is False


def test_pack_verify_load_round_trip(packed):
    g, arrays, root, report = packed
    assert report["ok"] and report["world"] == 2 and len(report["files"]) == 3
    assert verify.verify_runtime_checkpoint(root / "packed")["ok"]
    assert loader.read_geometry(root / "packed") == g
    full = loader.load_full_checkpoint(root / "packed")
    assert set(full) == set(arrays)
    for name, t in arrays.items():
        assert full[name].dtype == t.dtype and torch.equal(full[name], t), name


def test_rank_load_equals_sharding_the_full_checkpoint(packed):
    g, arrays, root, _ = packed
    for rank in range(2):
        layout = ParallelLayout(g, world=2, rank=rank)
        want = shard_checkpoint(arrays, layout, "cpu", use_kernel=False)
        got = shard_checkpoint(loader.load_rank_checkpoint(root / "packed", rank, 2), layout, "cpu", use_kernel=False)
        assert torch.equal(got.lm_head, want.lm_head) and torch.equal(got.embed, want.embed)
        for lw, lg in zip(want.layers, got.layers):
            for key, value in vars(lw).items():
                if isinstance(value, torch.Tensor):
                    assert torch.equal(getattr(lg, key), value), key
    with pytest.raises(ValueError, match="another rank"):
        shard_checkpoint(loader.load_rank_checkpoint(root / "packed", 0, 2), ParallelLayout(g, world=2, rank=1), "cpu", use_kernel=False)


def test_packing_is_reproducible_and_parallel_workers_agree(packed, tmp_path):
    g, arrays, root, report = packed
    again = pack_checkpoint(root / "src", tmp_path / "again", 2, jobs=2)
    assert again["manifest_sha256"] == report["manifest_sha256"]
    with pytest.raises(CheckpointValidationError, match="already"):
        pack_checkpoint(root / "src", tmp_path / "again", 2, jobs=1)


def test_unmarked_or_changed_source_is_refused(packed, tmp_path):
    g, arrays, root, _ = packed
    export.export_source(arrays, g, tmp_path / "src2", shards=2)
    with pytest.raises(CheckpointValidationError, match="mark-source"):
        pack_checkpoint(tmp_path / "src2", tmp_path / "p", 2, jobs=1)
    source_marker.mark_source(tmp_path / "src2")
    shard = sorted((tmp_path / "src2").glob("*.safetensors"))[0]
    with shard.open("ab") as f:
        f.write(b"\0" * 8)
    with pytest.raises(CheckpointValidationError, match="changed"):
        pack_checkpoint(tmp_path / "src2", tmp_path / "p", 2, jobs=1)


def _copy(src, dst):
    import shutil

    shutil.copytree(src, dst)
    return dst


def test_tampering_is_detected(packed, tmp_path):
    g, arrays, root, _ = packed
    # a flipped payload byte
    bad = _copy(root / "packed", tmp_path / "flip")
    path = bad / fmt.expert_file(1, 2)
    raw = bytearray(path.read_bytes())
    raw[-1] ^= 1
    path.write_bytes(bytes(raw))
    with pytest.raises(CheckpointValidationError, match="digest"):
        verify.verify_runtime_checkpoint(bad)
    assert verify.verify_runtime_checkpoint(bad, files=[fmt.SHARED_FILE])["ok"]  # a worker checks only its own files
    with pytest.raises(CheckpointValidationError):
        loader.load_rank_checkpoint(bad, 1, 2)
    # a missing seal, an edited manifest, an edited seal
    bad = _copy(root / "packed", tmp_path / "noseal")
    os.remove(bad / fmt.SEAL_FILE)
    with pytest.raises(CheckpointValidationError, match="SUCCESS"):
        verify.verify_runtime_checkpoint(bad)
    bad = _copy(root / "packed", tmp_path / "manifest")
    man = json.loads((bad / fmt.MANIFEST_FILE).read_text())
    man["total_bytes"] += 1
    (bad / fmt.MANIFEST_FILE).write_text(json.dumps(man))
    with pytest.raises(CheckpointValidationError, match="seal closes"):
        verify.verify_runtime_checkpoint(bad)
    bad = _copy(root / "packed", tmp_path / "seal")
    s = json.loads((bad / fmt.SEAL_FILE).read_text())
    s["world"] = 4
    (bad / fmt.SEAL_FILE).write_text(json.dumps(s))
    with pytest.raises(CheckpointValidationError, match="own digest"):
        seal.read_seal(bad)
    # wrong world, wrong pin
    with pytest.raises(CheckpointValidationError):
        loader.load_rank_checkpoint(root / "packed", 0, 4)
    with pytest.raises(CheckpointValidationError, match="pinned"):
        verify.verify_runtime_checkpoint(root / "packed", pins={"manifest_sha256": "0" * 64})

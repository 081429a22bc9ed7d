"""The SUCCESS seal, the geometry file and the source marker are read fail-closed: every way in which one of them can be absent,
unreadable, foreign, edited or out of step with its neighbours ends in ``CheckpointValidationError`` -- never in a stray
``KeyError`` / ``JSONDecodeError``, and never in a load.

Reference counterparts: ``tests/model_loader/sharded_state/test_seal.py``, ``tests/model_loader/test_source_marker.py``."""

import hashlib
import json
import os
import shutil

import pytest

from glm_tpu_b200.config.model import tiny_geometry
from glm_tpu_b200.exceptions import CheckpointValidationError
from glm_tpu_b200.executor.pack_job import pack_checkpoint
from glm_tpu_b200.model_loader import export, source_marker
from glm_tpu_b200.model_loader.sharded_state import format as fmt
from glm_tpu_b200.model_loader.sharded_state import loader, seal, verify
from glm_tpu_b200.models.glm_moe_dsa.weights import random_checkpoint
from glm_tpu_b200.utils.json_utils import canonical_hash_bytes, canonical_wire_bytes


@pytest.fixture(scope="module")
def pristine(tmp_path_factory):
    root = tmp_path_factory.mktemp("sealed")
    g = tiny_geometry()
    export.export_source(random_checkpoint(g, seed=5), g, root / "src", shards=2)
    source_marker.mark_source(root / "src")
    pack_checkpoint(root / "src", root / "packed", 2, jobs=1)
    return root


@pytest.fixture
def packed(pristine, tmp_path):
    shutil.copytree(pristine / "packed", tmp_path / "packed")
    return tmp_path / "packed"


@pytest.fixture
def source(pristine, tmp_path):
    shutil.copytree(pristine / "src", tmp_path / "src")
    return tmp_path / "src"


def rewrite(path, value):
    if path.exists():
        os.chmod(path, 0o600)
    path.write_bytes(value if isinstance(value, bytes) else canonical_wire_bytes(value) + b"\n")


def resealed(body: dict) -> dict:
    body = {k: v for k, v in body.items() if k != "seal_sha256"}
    return dict(body, seal_sha256=hashlib.sha256(canonical_hash_bytes(body)).hexdigest())


def refused(target, match):
    with pytest.raises(CheckpointValidationError, match=match):
        seal.read_seal(target)
    with pytest.raises(CheckpointValidationError, match=match):
        verify.verify_runtime_checkpoint(target)
    with pytest.raises(CheckpointValidationError, match=match):
        loader.load_rank_checkpoint(target, 0, 2)


def test_a_sealed_checkpoint_reads_back(packed):
    s, manifest = seal.read_seal(packed)
    assert sorted(s) == sorted(seal.SEAL_KEYS) and s == seal.success_record(manifest)
    assert s["world"] == 2 and s["total_bytes"] == sum(r["size"] for r in manifest["files"].values())
    assert verify.verify_runtime_checkpoint(packed)["ok"]
    for name in (fmt.SEAL_FILE, fmt.MANIFEST_FILE, fmt.GEOMETRY_FILE):
        assert (packed / name).stat().st_mode & 0o077 == 0  # private files
    with pytest.raises(FileExistsError):
        seal.install(packed, tiny_geometry(), manifest)  # create-once: a sealed directory is never sealed again


def test_no_seal_no_checkpoint(packed):
    (packed / fmt.SEAL_FILE).unlink()
    refused(packed, "never completed")


@pytest.mark.parametrize("content,match", [
    (b"", "cannot be read as JSON"),
    (b"{not json", "cannot be read as JSON"),
    (b"\xff\xfe\x00", "cannot be read as JSON"),
    (b"[1, 2, 3]\n", "not a JSON object"),
    (b'"SUCCESS"\n', "not a JSON object"),
])
def test_an_unreadable_seal(packed, content, match):
    rewrite(packed / fmt.SEAL_FILE, content)
    refused(packed, match)


def test_a_seal_with_other_keys_or_schema(packed):
    good = json.loads((packed / fmt.SEAL_FILE).read_text())
    for edit in ({"extra": 1}, {"schema": "glm_b200_seal_v0"}):
        rewrite(packed / fmt.SEAL_FILE, resealed(dict(good, **edit)))  # self-consistent, but not this record
        refused(packed, "not a glm_b200_seal_v1 record")
    short = {k: v for k, v in good.items() if k != "total_bytes"}
    rewrite(packed / fmt.SEAL_FILE, resealed(short))
    refused(packed, "not a glm_b200_seal_v1 record")


def test_an_edited_seal_fails_its_own_digest(packed):
    good = json.loads((packed / fmt.SEAL_FILE).read_text())
    for key, value in (("world", 4), ("total_bytes", good["total_bytes"] + 1), ("manifest_sha256", "0" * 64), ("geometry_sha256", "0" * 64)):
        rewrite(packed / fmt.SEAL_FILE, dict(good, **{key: value}))
        refused(packed, "does not match its own digest")


def test_a_resealed_lie_is_caught_by_the_manifest(packed):
    """Someone who can recompute the seal's own digest still has to match the manifest on disk, and the facts in both."""
    good = json.loads((packed / fmt.SEAL_FILE).read_text())
    rewrite(packed / fmt.SEAL_FILE, resealed(dict(good, manifest_sha256="1" * 64)))
    refused(packed, "not the one the seal closes")
    for key, value in (("world", 4), ("total_bytes", 1), ("geometry_sha256", "2" * 64)):
        rewrite(packed / fmt.SEAL_FILE, resealed(dict(good, **{key: value})))
        refused(packed, f"state different {key}")


def test_the_manifest_must_be_the_sealed_one(packed):
    manifest = json.loads((packed / fmt.MANIFEST_FILE).read_text())
    (packed / fmt.MANIFEST_FILE).unlink()
    refused(packed, "the manifest is missing")
    rewrite(packed / fmt.MANIFEST_FILE, b"{broken")
    refused(packed, "the manifest cannot be read as JSON")
    rewrite(packed / fmt.MANIFEST_FILE, b"[]")
    refused(packed, "the manifest is not a JSON object")
    rewrite(packed / fmt.MANIFEST_FILE, dict(manifest, world=manifest["world"]))  # the same content reads back
    seal.read_seal(packed)
    rewrite(packed / fmt.MANIFEST_FILE, dict(manifest, total_bytes=manifest["total_bytes"] + 1))
    refused(packed, "not the one the seal closes")
    # a manifest edited AND resealed is a different checkpoint: only a pin notices, which is what the pin is for
    edited = dict(manifest, created_by="someone else")
    rewrite(packed / fmt.MANIFEST_FILE, edited)
    rewrite(packed / fmt.SEAL_FILE, seal.success_record(edited))
    s, _ = seal.read_seal(packed)
    with pytest.raises(CheckpointValidationError, match="not the pinned one"):
        verify.verify_runtime_checkpoint(packed, pins={"manifest_sha256": seal.success_record(manifest)["manifest_sha256"]})
    assert verify.verify_runtime_checkpoint(packed, pins={"manifest_sha256": s["manifest_sha256"]})["ok"]


@pytest.mark.parametrize("content,match", [
    (None, "the geometry file is missing"),
    (b"{", "the geometry file cannot be read as JSON"),
    (b"[]", "the geometry file is not a JSON object"),
    (b"{}", "does not describe a model geometry"),
    (b'{"hidden_size": 64}', "does not describe a model geometry"),
])
def test_the_geometry_file_is_read_fail_closed(packed, content, match):
    if content is None:
        (packed / fmt.GEOMETRY_FILE).unlink()
    else:
        rewrite(packed / fmt.GEOMETRY_FILE, content)
    with pytest.raises(CheckpointValidationError, match=match):
        verify.verify_runtime_checkpoint(packed)
    with pytest.raises(CheckpointValidationError, match=match):
        loader.load_rank_checkpoint(packed, 0, 2)


def test_another_geometry_is_refused(packed):
    raw = json.loads((packed / fmt.GEOMETRY_FILE).read_text())
    rewrite(packed / fmt.GEOMETRY_FILE, dict(raw, rms_norm_eps=raw["rms_norm_eps"] * 2))
    with pytest.raises(CheckpointValidationError, match="geometry, manifest and seal disagree"):
        verify.verify_runtime_checkpoint(packed)


# ------------------------------------------------------------------------------------------------ source marker
def test_marker_round_trip_and_create_once(source):
    marker = source_marker.require_marker(source)
    assert marker["schema"] == "glm_b200_source_marker_v1" and set(marker["small_files"]) >= {"config.json"}
    assert (source / source_marker.MARKER_FILE).stat().st_mode & 0o077 == 0
    with pytest.raises(FileExistsError):
        source_marker.mark_source(source)


def test_a_source_without_marker_is_not_packed(source, tmp_path):
    (source / source_marker.MARKER_FILE).unlink()
    with pytest.raises(CheckpointValidationError, match="mark-source"):
        source_marker.require_marker(source)
    with pytest.raises(CheckpointValidationError, match="mark-source"):
        pack_checkpoint(source, tmp_path / "out", 2, jobs=1)
    assert not (tmp_path / "out" / fmt.SEAL_FILE).exists()


@pytest.mark.parametrize("content,match", [
    (b"", "cannot be read as JSON"),
    (b"{oops", "cannot be read as JSON"),
    (b"[]", "not a glm_b200_source_marker_v1 record"),
    (b'{"schema": "something_else"}', "not a glm_b200_source_marker_v1 record"),
])
def test_an_unreadable_or_foreign_marker(source, content, match):
    rewrite(source / source_marker.MARKER_FILE, content)
    with pytest.raises(CheckpointValidationError, match=match):
        source_marker.require_marker(source)


def test_changes_after_marking_are_noticed(source):
    marker = json.loads((source / source_marker.MARKER_FILE).read_text())
    config = source / "config.json"
    original = config.read_bytes()
    config.write_bytes(original.replace(b"{", b"{ ", 1))  # same meaning, other bytes
    with pytest.raises(CheckpointValidationError, match="config.json changed"):
        source_marker.require_marker(source)
    config.write_bytes(original)
    source_marker.require_marker(source)

    (source / "tokenizer_config.json").write_text("{}")  # a configuration file that was not there when the source was marked
    with pytest.raises(CheckpointValidationError, match="added or removed.*tokenizer_config.json"):
        source_marker.require_marker(source)
    (source / "tokenizer_config.json").unlink()

    shard = sorted(marker["shards"])[0]
    rewrite(source / source_marker.MARKER_FILE, dict(marker, shards={k: v for k, v in marker["shards"].items() if k != shard}))
    with pytest.raises(CheckpointValidationError, match="shard list differs"):
        source_marker.require_marker(source)
    rewrite(source / source_marker.MARKER_FILE, dict(marker, shards=dict(marker["shards"], **{shard: {"size": 1}})))
    with pytest.raises(CheckpointValidationError, match="shard list differs"):
        source_marker.require_marker(source)
    rewrite(source / source_marker.MARKER_FILE, dict(marker, small_files=None))
    with pytest.raises(CheckpointValidationError, match="lists no small files"):
        source_marker.require_marker(source)
    rewrite(source / source_marker.MARKER_FILE, dict(marker, inventory_sha256="0" * 64))
    with pytest.raises(CheckpointValidationError, match="changed after it was marked"):
        source_marker.require_marker(source)
    rewrite(source / source_marker.MARKER_FILE, marker)
    source_marker.require_marker(source)


def test_expected_checksums_gate_the_marker(source):
    (source / source_marker.MARKER_FILE).unlink()
    marker = source_marker.mark_source(source, hash_shards=True)  # digests of every shard, for a checksums file
    (source / source_marker.MARKER_FILE).unlink()
    shard = sorted(marker["shards"])[0]
    good = {shard: dict(marker["shards"][shard])}
    (source / source_marker.CHECKSUMS_FILE).write_text(json.dumps({shard: {"size": good[shard]["size"] + 1}}))
    with pytest.raises(CheckpointValidationError, match="differs from the expected"):
        source_marker.mark_source(source)
    (source / source_marker.CHECKSUMS_FILE).write_text(json.dumps({shard: {"size": good[shard]["size"], "sha256": "0" * 64}}))
    with pytest.raises(CheckpointValidationError, match="content differs from the expected digest"):
        source_marker.mark_source(source)
    assert not (source / source_marker.MARKER_FILE).exists()  # a refused source is never marked
    (source / source_marker.CHECKSUMS_FILE).write_text(json.dumps(good))
    again = source_marker.mark_source(source)
    assert again["shards"][shard] == good[shard] and "sha256" not in again["shards"][sorted(marker["shards"])[1]]

"""The pack job as a whole: what it refuses, what a failed worker leaves behind (never a seal), the lease it holds, and the manifest
it assembles from receipts only.

Reference counterparts: ``tests/executor/test_pack_job.py``, ``tests/model_loader/sharded_state/test_manifest.py``."""

import json
import shutil
import threading

import pytest

from glm_tpu_b200.config.model import tiny_geometry
from glm_tpu_b200.exceptions import CheckpointValidationError
from glm_tpu_b200.executor import pack_job
from glm_tpu_b200.executor.jobs import LEASE_FILE, LeaseHeld, workload_lease
from glm_tpu_b200.executor.pack_job import pack_checkpoint
from glm_tpu_b200.model_loader import export, pack_worker, source_marker
from glm_tpu_b200.model_loader.sharded_state import format as fmt
from glm_tpu_b200.model_loader.sharded_state import manifest as manifest_mod
from glm_tpu_b200.model_loader.sharded_state import verify
from glm_tpu_b200.models.glm_moe_dsa.weights import random_checkpoint


@pytest.fixture(scope="module")
def source(tmp_path_factory):
    root = tmp_path_factory.mktemp("packjob") / "src"
    g = tiny_geometry()
    export.export_source(random_checkpoint(g, seed=8), g, root, shards=2)
    source_marker.mark_source(root)
    return root


def sealed(target) -> bool:
    return (target / fmt.SEAL_FILE).exists() or (target / fmt.MANIFEST_FILE).exists()


# ------------------------------------------------------------------------------------------------ manifest from receipts
def receipt(*names):
    return {n: {"size": 10 + i, "sha256": "0" * 64, "header_sha256": "1" * 64, "tensors": {}} for i, n in enumerate(names)}


def test_manifest_needs_exactly_one_receipt_per_file():
    g = tiny_geometry()
    names = manifest_mod.expected_files(2)
    assert names == ["shared.safetensors", "experts.rank0of2.safetensors", "experts.rank1of2.safetensors"]
    man = manifest_mod.assemble_manifest([receipt(names[0]), receipt(names[1], names[2])], g, 2, "a" * 64, "sliced")
    assert list(man["files"]) == sorted(names) and man["total_bytes"] == 10 + 10 + 11 and man["world"] == 2
    assert man["expert_split"] == "sliced" and man["format"] == fmt.FORMAT_VERSION and man["source_inventory_sha256"] == "a" * 64
    with pytest.raises(CheckpointValidationError, match="two receipts claim shared.safetensors"):
        manifest_mod.assemble_manifest([receipt(names[0]), receipt(*names)], g, 2, "a" * 64)
    with pytest.raises(CheckpointValidationError, match="the checkpoint needs"):
        manifest_mod.assemble_manifest([receipt(names[0], names[1])], g, 2, "a" * 64)  # a rank's file is missing
    with pytest.raises(CheckpointValidationError, match="the checkpoint needs"):
        manifest_mod.assemble_manifest([receipt(*names), receipt("experts.rank2of2.safetensors")], g, 2, "a" * 64)  # one too many
    with pytest.raises(CheckpointValidationError, match="the checkpoint needs"):
        manifest_mod.assemble_manifest([receipt(*names)], g, 4, "a" * 64)  # receipts of another world size


# ------------------------------------------------------------------------------------------------ the job
def test_a_sealed_target_is_never_packed_again(source, tmp_path):
    first = pack_checkpoint(source, tmp_path / "packed", 2, jobs=1)
    assert first["ok"] and first["world"] == 2 and first["source_marker"] and first["files"] == sorted(manifest_mod.expected_files(2))
    seal_bytes = (tmp_path / "packed" / fmt.SEAL_FILE).read_bytes()
    with pytest.raises(CheckpointValidationError, match="already a sealed checkpoint"):
        pack_checkpoint(source, tmp_path / "packed", 2, jobs=1)
    assert (tmp_path / "packed" / fmt.SEAL_FILE).read_bytes() == seal_bytes
    again = pack_checkpoint(source, tmp_path / "again", 2, jobs=3)  # other worker count, same bytes
    assert again["manifest_sha256"] == first["manifest_sha256"] and again["total_bytes"] == first["total_bytes"]


def test_world_sizes_and_truncation_change_the_identity(source, tmp_path):
    two = pack_checkpoint(source, tmp_path / "w2", 2, jobs=1)
    one = pack_checkpoint(source, tmp_path / "w1", 1, jobs=1)
    assert one["manifest_sha256"] != two["manifest_sha256"] and one["geometry_sha256"] == two["geometry_sha256"]
    short = pack_checkpoint(source, tmp_path / "short", 2, jobs=1, layers=1)
    assert short["geometry_sha256"] != two["geometry_sha256"] and short["total_bytes"] < two["total_bytes"]
    assert verify.read_geometry(tmp_path / "short").num_layers == 1
    whole = pack_checkpoint(source, tmp_path / "whole", 2, jobs=1, expert_split="whole")
    assert whole["expert_split"] == "whole" and verify.verify_runtime_checkpoint(tmp_path / "whole")["expert_split"] == "whole"


def test_a_failing_worker_in_process_seals_nothing(source, tmp_path, monkeypatch):
    def broken(*args, **kw):
        raise CheckpointValidationError("tensor 'x' holds a NaN code")

    monkeypatch.setattr(pack_worker, "run", broken)
    with pytest.raises(CheckpointValidationError, match="NaN code"):
        pack_checkpoint(source, tmp_path / "t", 2, jobs=1)
    assert not sealed(tmp_path / "t")
    with pytest.raises(CheckpointValidationError):
        verify.verify_runtime_checkpoint(tmp_path / "t")


def test_a_failing_worker_process_fails_the_job_and_leaves_its_log(source, tmp_path):
    target = tmp_path / "t"
    target.mkdir()
    (target / fmt.SHARED_FILE).mkdir()  # the worker that owns the shared file cannot create it
    with pytest.raises(CheckpointValidationError, match=r"pack workers failed: \[\('receipt\.0\.json', [1-9-]"):
        pack_checkpoint(source, target, 2, jobs=3)
    assert not sealed(target)
    assert (target / "receipts" / "worker.0.log").stat().st_size > 0  # what went wrong is on disk, not on a lost pipe
    assert (target / "receipts" / "receipt.1.json").exists() and (target / "receipts" / "receipt.2.json").exists()  # the others finished
    fresh = pack_checkpoint(source, tmp_path / "fresh", 2, jobs=3)  # the same source packs into a clean target
    assert fresh["ok"]


def test_workers_that_overrun_the_deadline_are_stopped(source, tmp_path):
    with pytest.raises(CheckpointValidationError, match="pack workers failed"):
        pack_checkpoint(source, tmp_path / "t", 2, jobs=2, timeout=0.0)
    assert not sealed(tmp_path / "t")


def test_receipts_that_do_not_cover_the_checkpoint_seal_nothing(source, tmp_path, monkeypatch):
    real = pack_worker.run

    def forgetful(src, target, world, files, *rest, **kw):
        return real(src, target, world, [f for f in files if f != "1"], *rest, **kw)  # rank 1's file is never written

    monkeypatch.setattr(pack_worker, "run", forgetful)
    with pytest.raises(CheckpointValidationError, match="the checkpoint needs"):
        pack_checkpoint(source, tmp_path / "t", 2, jobs=1)
    assert not sealed(tmp_path / "t")


def test_the_source_must_be_marked_and_unchanged(source, tmp_path):
    copy = tmp_path / "src"
    shutil.copytree(source, copy)
    (copy / source_marker.MARKER_FILE).unlink()
    with pytest.raises(CheckpointValidationError, match="mark-source"):
        pack_checkpoint(copy, tmp_path / "t", 2, jobs=1)
    assert not (tmp_path / "t").exists()  # refused before anything was created
    report = pack_checkpoint(copy, tmp_path / "unmarked", 2, jobs=1, require_marker=False)  # fixtures may skip the marker; the report says so
    assert report["source_marker"] is False


def test_the_job_holds_the_workload_lease(source, tmp_path):
    run_root = tmp_path / "runs"
    with workload_lease(run_root):
        assert (run_root / LEASE_FILE).read_text().strip().isdigit()
        with pytest.raises(LeaseHeld, match="another controller holds"):
            pack_checkpoint(source, tmp_path / "t", 2, jobs=1, run_root=run_root)
        assert not sealed(tmp_path / "t")
    assert pack_checkpoint(source, tmp_path / "t", 2, jobs=1, run_root=run_root)["ok"]  # released: the next job gets it

    entered, release = threading.Event(), threading.Event()
    real = pack_worker.run

    def slow(*args, **kw):
        entered.set()
        release.wait(30)
        return real(*args, **kw)

    pack_worker.run = slow
    try:
        worker = threading.Thread(target=pack_checkpoint, args=(source, tmp_path / "t2", 2), kwargs={"jobs": 1, "run_root": run_root})
        worker.start()
        assert entered.wait(30)
        with pytest.raises(LeaseHeld):  # while a pack job runs, no other workload starts from this run root
            with workload_lease(run_root):
                pass
        release.set()
        worker.join(60)
    finally:
        pack_worker.run = real
        release.set()
    assert (tmp_path / "t2" / fmt.SEAL_FILE).exists()
    with workload_lease(run_root):
        pass


def test_the_report_is_json_and_names_what_to_pin(source, tmp_path):
    report = pack_checkpoint(source, tmp_path / "t", 2, jobs=1)
    json.dumps(report)
    seal = json.loads((tmp_path / "t" / fmt.SEAL_FILE).read_text())
    assert report["manifest_sha256"] == seal["manifest_sha256"] and len(report["manifest_sha256"]) == 64
    assert report["source_inventory_sha256"] == json.loads((tmp_path / "t" / fmt.MANIFEST_FILE).read_text())["source_inventory_sha256"]
    assert verify.verify_runtime_checkpoint(tmp_path / "t", pins={"manifest_sha256": report["manifest_sha256"]})["ok"]
    assert pack_job.__doc__ and "seal" in pack_job.__doc__


def test_preflight_checks_everything_and_writes_nothing(source, tmp_path):
    plan = pack_checkpoint(source, tmp_path / "t", 2, jobs=1, preflight_only=True)
    assert plan["ok"] and plan["preflight_only"] and not (tmp_path / "t").exists()
    real = pack_checkpoint(source, tmp_path / "t", 2, jobs=1)
    on_disk = {p.name: p.stat().st_size for p in (tmp_path / "t").glob("*.safetensors")}
    assert plan["planned_bytes"] == on_disk and plan["total_bytes"] == real["total_bytes"] == sum(on_disk.values())  # sizes known from the shapes alone
    assert plan["files"] == real["files"] and plan["expert_split"] == real["expert_split"] and plan["geometry_sha256"] == real["geometry_sha256"]
    assert plan["source_marker_sha256"] == real["source_marker_sha256"] and plan["free_bytes"] > plan["total_bytes"]
    with pytest.raises(CheckpointValidationError, match="already a sealed checkpoint"):
        pack_checkpoint(source, tmp_path / "t", 2, jobs=1, preflight_only=True)
    with pytest.raises(CheckpointValidationError, match="not the pinned one"):
        pack_checkpoint(source, tmp_path / "u", 2, jobs=1, preflight_only=True, pins={"source_marker_sha256": "0" * 64})


def test_a_target_without_room_is_refused_before_anything_is_written(source, tmp_path):
    with pytest.raises(CheckpointValidationError, match=r"needs [\d,]+ bytes, 1,000 are free"):
        pack_checkpoint(source, tmp_path / "deep" / "t", 2, jobs=1, free_bytes=lambda target: 1000)
    assert not (tmp_path / "deep").exists()


def test_a_source_that_lacks_tensors_is_refused_before_anything_is_written(source, tmp_path):
    import shutil

    from glm_tpu_b200.model_loader.sharded_state import format as fmt_mod
    from glm_tpu_b200.model_loader import source_inventory

    copy = tmp_path / "src"
    shutil.copytree(source, copy)
    shard = sorted(copy.glob("*.safetensors"))[0]
    header, start = fmt_mod.read_header(shard)
    victim = sorted(n for n in header if n != "__metadata__")[0]
    tensors = {n: fmt_mod.read_tensor(shard, header, start, n) for n in header if n not in ("__metadata__", victim)}
    shard.unlink()
    fmt_mod.write_file(shard, tensors, {})
    with pytest.raises(CheckpointValidationError, match="index names tensors that no shard holds"):
        pack_checkpoint(copy, tmp_path / "t", 2, jobs=1, require_marker=False, preflight_only=True)  # the index still promises it
    index = copy / source_inventory.INDEX_FILE
    listing = json.loads(index.read_text())
    del listing["weight_map"][victim]
    index.write_text(json.dumps(listing))
    with pytest.raises(CheckpointValidationError, match="lacks 1 tensors"):
        pack_checkpoint(copy, tmp_path / "t", 2, jobs=1, require_marker=False, preflight_only=True)  # a consistent source of another model
    assert victim not in source_inventory.read_source_inventory(copy).tensors and not (tmp_path / "t").exists()

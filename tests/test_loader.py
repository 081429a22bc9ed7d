"""Checkpoint pipeline on a tiny model: export -> inventory -> marker -> pack -> verify -> load, plus tamper cases."""

import json
import os

import pytest

from tests.conftest import scaled
import torch
from pathlib import Path

ROOT_DIR = Path(__file__).resolve().parents[1]

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


def _raw_file(path, header: dict, payload: bytes):
    import struct

    raw = json.dumps(header).encode()
    path.write_bytes(struct.pack("<Q", len(raw)) + raw + payload)
    return path


def test_header_ranges_must_tile_the_payload(tmp_path):
    ok = {"a": {"dtype": "U8", "shape": [4], "data_offsets": [0, 4]}, "b": {"dtype": "U8", "shape": [4], "data_offsets": [4, 8]}}
    fmt.read_header(_raw_file(tmp_path / "ok.safetensors", ok, b"\0" * 8))
    gap = {"a": ok["a"], "b": {"dtype": "U8", "shape": [4], "data_offsets": [6, 10]}}
    with pytest.raises(CheckpointValidationError, match="gap"):
        fmt.read_header(_raw_file(tmp_path / "gap.safetensors", gap, b"\0" * 10))
    overlap = {"a": ok["a"], "b": {"dtype": "U8", "shape": [4], "data_offsets": [2, 6]}}
    with pytest.raises(CheckpointValidationError, match="overlapping"):
        fmt.read_header(_raw_file(tmp_path / "overlap.safetensors", overlap, b"\0" * 6))
    with pytest.raises(CheckpointValidationError, match="follow the last tensor"):
        fmt.read_header(_raw_file(tmp_path / "tail.safetensors", ok, b"\0" * 9))


def test_writer_fills_tensors_piece_by_piece_and_refuses_holes(tmp_path, monkeypatch):
    monkeypatch.setattr(fmt, "PIECE_BYTES", 64)
    specs = {"w": ("F8_E4M3", (4, 100)), "s": ("F32", (10,))}
    w = fmt.FileWriter(tmp_path / "f.safetensors", specs, {"k": "v"})
    bits = (torch.arange(400) % 100).to(torch.uint8).reshape(4, 100)
    for row in bits:  # one "expert" at a time, never stacked
        w.append("w", row)
    with pytest.raises(CheckpointValidationError, match="not written completely"):
        w.close()
    assert not (tmp_path / "f.safetensors").exists()
    w.abort()
    w = fmt.FileWriter(tmp_path / "f.safetensors", specs, {"k": "v"})
    for row in bits:
        w.append("w", row)
    w.append("s", torch.arange(10, dtype=torch.float32))
    receipt = w.close()
    whole = fmt.write_file(tmp_path / "g.safetensors", {"w": bits, "s": torch.arange(10, dtype=torch.float32)}, {"k": "v"}, {"w"})
    assert receipt == whole and (tmp_path / "f.safetensors").read_bytes() == (tmp_path / "g.safetensors").read_bytes()
    reader = fmt.TensorReader(tmp_path / "f.safetensors")
    assert torch.equal(reader.read("w", expect_sha256=receipt["tensors"]["w"]["sha256"]), bits)
    assert reader.largest_piece <= 64 and reader.bytes_read == 400
    with pytest.raises(CheckpointValidationError, match="content digest"):
        reader.read("s", expect_sha256="0" * 64)
    nan = fmt.FileWriter(tmp_path / "n.safetensors", {"s": ("F32", (2,))}, {})
    with pytest.raises(CheckpointValidationError, match="non-finite"):
        nan.append("s", torch.tensor([1.0, float("inf")]))
    nan.abort()


def test_rank_load_streams_every_byte_once_in_bounded_pieces(packed, monkeypatch):
    g, arrays, root, _ = packed
    monkeypatch.setattr(fmt, "PIECE_BYTES", 4096)
    streamed = loader.load_rank_checkpoint(root / "packed", 0, 2)
    assert streamed.io_stats() == {"bytes_read": 0, "largest_piece": 0}  # nothing is read before a tensor is asked for
    shard_checkpoint(streamed, ParallelLayout(g, world=2, rank=0, expert_split=streamed["__expert_split__"]), "cpu", use_kernel=False)
    payload = 0
    for name in (fmt.SHARED_FILE, fmt.expert_file(0, 2)):
        header, start = fmt.read_header(root / "packed" / name)
        payload += (root / "packed" / name).stat().st_size - start
    stats = streamed.io_stats()
    assert stats["bytes_read"] == payload and 0 < stats["largest_piece"] <= 4096


def test_sliced_experts_pack_and_load(tmp_path):
    import dataclasses

    g = dataclasses.replace(tiny_geometry(), moe_intermediate_size=256)
    arrays = random_checkpoint(g, seed=4)
    export.export_source(arrays, g, tmp_path / "src", shards=2)
    source_marker.mark_source(tmp_path / "src")
    report = pack_checkpoint(tmp_path / "src", tmp_path / "sliced", 2, jobs=2, expert_split="sliced")
    assert report["expert_split"] == "sliced" and verify.verify_runtime_checkpoint(tmp_path / "sliced")["expert_split"] == "sliced"
    whole = pack_checkpoint(tmp_path / "src", tmp_path / "whole", 2, jobs=1, expert_split="whole")
    assert whole["manifest_sha256"] != report["manifest_sha256"] and abs(whole["total_bytes"] - report["total_bytes"]) < 4096  # the same payload; the headers differ in a few digits
    full = loader.load_full_checkpoint(tmp_path / "sliced")
    assert set(full) == set(arrays) and all(torch.equal(full[n], arrays[n]) for n in arrays)
    for rank in range(2):
        layout = ParallelLayout(g, world=2, rank=rank, expert_split="sliced")
        want = shard_checkpoint(arrays, layout, "cpu", use_kernel=False)
        loaded = loader.load_rank_checkpoint(tmp_path / "sliced", rank, 2)
        assert loaded["__expert_split__"] == "sliced"
        got = shard_checkpoint(loaded, layout, "cpu", use_kernel=False)
        for lw, lg in zip(want.layers, got.layers):
            for key, value in vars(lw).items():
                if isinstance(value, torch.Tensor):
                    assert torch.equal(getattr(lg, key), value), key
        if lg.exp_down_bits is not None:
            assert lg.exp_down_bits.shape == (g.num_routed_experts, g.hidden_size, 128)
        # a checkpoint cut one way does not load into the other layout
        with pytest.raises(ValueError, match="shape"):
            shard_checkpoint(loaded, ParallelLayout(g, world=2, rank=rank, expert_split="whole"), "cpu", use_kernel=False)
    with pytest.raises(PlanValidationError, match="FP8 block"):
        pack_checkpoint(tmp_path / "src", tmp_path / "bad", 4, jobs=1, expert_split="sliced")


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
        layout = ParallelLayout(g, world=2, rank=rank, expert_split=loader.load_rank_checkpoint(root / "packed", rank, 2)["__expert_split__"])
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
    with pytest.raises(CheckpointValidationError, match="changed|follow the last tensor"):
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
    with pytest.raises(CheckpointValidationError, match="digest"):
        loader.load_rank_checkpoint(bad, 1, 2, rehash=True)
    # without the whole-file pass the flipped byte is caught when its tensor streams in (the last tensor of the file here)
    streamed = loader.load_rank_checkpoint(bad, 1, 2)
    last = max(streamed._readers[fmt.expert_file(1, 2)].names(), key=lambda n: streamed._readers[fmt.expert_file(1, 2)].header[n]["data_offsets"][1])
    with pytest.raises(CheckpointValidationError, match="content digest of"):
        streamed[last]
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


def test_pack_and_load_never_hold_more_than_a_few_pieces(tmp_path):
    """Peak resident memory of a process that packs a ~200 MB source and then streams one rank's files tensor by tensor, with 1 MB
    pieces: it stays within a small multiple of the largest single tensor (25 MB), far below the size of the files it moved."""
    import dataclasses
    import subprocess
    import sys
    import textwrap

    g = dataclasses.replace(tiny_geometry(), hidden_size=1024, moe_intermediate_size=512, num_routed_experts=96, vocab_size=8192,
                            eos_ids=(8189, 8190, 8191), q_lora_rank=256, dense_intermediate_size=1024)
    arrays = random_checkpoint(g, seed=8)
    export.export_source(arrays, g, tmp_path / "src", shards=4)
    source_marker.mark_source(tmp_path / "src")
    source_bytes = sum(p.stat().st_size for p in (tmp_path / "src").glob("*.safetensors"))
    del arrays
    script = textwrap.dedent(f"""
        import json, threading, time
        import psutil, torch
        from glm_tpu_b200.executor.pack_job import pack_checkpoint
        from glm_tpu_b200.model_loader.sharded_state import format as fmt, loader
        fmt.PIECE_BYTES = 1 << 20
        torch.zeros(1)
        me, peak, stop = psutil.Process(), [0], threading.Event()
        def sample():
            while not stop.is_set():
                peak[0] = max(peak[0], me.memory_info().rss)
                time.sleep(0.002)
        base = me.memory_info().rss
        watcher = threading.Thread(target=sample); watcher.start()
        pack_checkpoint({str(tmp_path / "src")!r}, {str(tmp_path / "packed")!r}, 2, jobs=1)
        ckpt = loader.load_rank_checkpoint({str(tmp_path / "packed")!r}, 0, 2)
        read = 0
        for name in list(ckpt):
            if not name.startswith("__"):
                t = ckpt[name]
                read += t.numel() * t.element_size()
                del t
        stop.set(); watcher.join()
        print(json.dumps({{"base": base, "peak": peak[0], "read": read, "io": ckpt.io_stats()}}))
    """)
    out = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, timeout=scaled(600), cwd=str(ROOT_DIR))
    assert out.returncode == 0, out.stderr[-2000:]
    report = json.loads(out.stdout.strip().splitlines()[-1])
    grown_mb = (report["peak"] - report["base"]) / 2**20
    assert source_bytes > 150e6 and report["read"] > 80e6 and report["io"]["largest_piece"] <= 1 << 20
    assert report["io"]["bytes_read"] == report["read"]  # every byte once
    print("peak growth MB", round(grown_mb, 1))
    assert grown_mb < 80, (grown_mb, report)  # measured 52 MB: a fraction of the ~190 MB packed and the ~115 MB loaded

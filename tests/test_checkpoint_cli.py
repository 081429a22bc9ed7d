"""``glm-b200 checkpoint ...`` from the command line: one JSON report per action, the two pins of the site file enforced where
they belong (the source marker by ``pack``, the manifest by ``verify``), and every refusal as exit status 2 with one JSON line on
stderr -- never a traceback, never a half-done target.

Reference counterpart: ``tests/entrypoints/cli/test_checkpoint.py``."""

import json
import os
import subprocess
import sys

import pytest

from glm_tpu_b200.config.model import tiny_geometry
from glm_tpu_b200.entrypoints.cli import main as cli
from glm_tpu_b200.model_loader import export, source_marker
from glm_tpu_b200.model_loader.sharded_state import format as fmt
from glm_tpu_b200.models.glm_moe_dsa.weights import random_checkpoint


@pytest.fixture
def source(tmp_path, monkeypatch):
    monkeypatch.setenv("GLM_B200_RUN_ROOT", str(tmp_path / "runs"))
    monkeypatch.setenv("GLM_B200_SITE_CONFIG", str(tmp_path / "no-site.toml"))
    monkeypatch.delenv("GLM_B200_MODEL_PATH", raising=False)
    g = tiny_geometry()
    export.export_source(random_checkpoint(g, seed=6), g, tmp_path / "src", shards=2)
    return tmp_path / "src"


def site_file(tmp_path, **pins):
    path = tmp_path / "site.toml"
    path.write_text('[paths]\nrun_root = "%s"\n[checkpoint]\n' % (tmp_path / "runs") + "".join(f'{k} = "{v}"\n' for k, v in pins.items()))
    os.chmod(path, 0o600)
    return path


def run(capsys, *argv):
    code = cli.main([str(a) for a in argv])
    captured = capsys.readouterr()
    return code, captured.out, captured.err


def refusal(err: str) -> dict:
    lines = err.strip().splitlines()
    assert len(lines) == 1, err  # one line, no traceback
    report = json.loads(lines[0])
    assert report["ok"] is False and set(report) == {"ok", "refused", "message"}
    return report


def test_each_action_prints_one_report(source, tmp_path, capsys):
    code, out, err = run(capsys, "checkpoint", "inventory", source)
    inv = json.loads(out)
    assert code == 0 and err == "" and inv["ok"] and inv["shards"] == 2 and inv["tensors"] > 10 and len(inv["inventory_sha256"]) == 64
    assert inv["matches_pinned_glm53"] is False and sum(inv["bytes_by_dtype"].values()) <= inv["total_bytes"]

    code, out, _ = run(capsys, "checkpoint", "mark-source", source)
    marked = json.loads(out)
    assert code == 0 and marked["inventory_sha256"] == inv["inventory_sha256"] and marked["tensor_count"] == inv["tensors"]
    assert marked["marker_sha256"] == fmt.file_sha256(source / source_marker.MARKER_FILE)  # the value a site file pins

    code, out, _ = run(capsys, "checkpoint", "pack", source, tmp_path / "packed", "--gpus", "2", "--expert-split", "whole")
    packed = json.loads(out)
    assert code == 0 and packed["ok"] and packed["world"] == 2 and packed["expert_split"] == "whole"
    assert packed["source_marker_sha256"] == marked["marker_sha256"] and packed["source_inventory_sha256"] == inv["inventory_sha256"]

    code, out, _ = run(capsys, "checkpoint", "verify", tmp_path / "packed")
    verified = json.loads(out)
    assert code == 0 and verified["ok"] and verified["manifest_sha256"] == packed["manifest_sha256"] and "manifest_files" not in verified
    assert sorted(verified["files"]) == sorted(packed["files"])


def test_pack_enforces_the_pinned_source_marker(source, tmp_path, capsys):
    assert run(capsys, "checkpoint", "mark-source", source)[0] == 0
    good = fmt.file_sha256(source / source_marker.MARKER_FILE)
    code, out, err = run(capsys, "checkpoint", "pack", source, tmp_path / "packed", "--gpus", "2", "--site", site_file(tmp_path, source_marker_sha256="0" * 64))
    assert code == 2 and out == ""
    assert refusal(err) == {"ok": False, "refused": "CheckpointValidationError",
                            "message": "the source's marker is not the pinned one ([checkpoint] source_marker_sha256)"}
    assert not (tmp_path / "packed").exists()  # refused before the target was touched
    code, out, _ = run(capsys, "checkpoint", "pack", source, tmp_path / "packed", "--gpus", "2", "--site", site_file(tmp_path, source_marker_sha256=good))
    assert code == 0 and json.loads(out)["source_marker_sha256"] == good


def test_verify_enforces_the_pinned_manifest(source, tmp_path, capsys):
    run(capsys, "checkpoint", "mark-source", source)
    manifest = json.loads(run(capsys, "checkpoint", "pack", source, tmp_path / "packed", "--gpus", "2")[1])["manifest_sha256"]
    code, out, err = run(capsys, "checkpoint", "verify", tmp_path / "packed", "--site", site_file(tmp_path, manifest_sha256="f" * 64))
    assert code == 2 and out == "" and refusal(err)["message"] == "the checkpoint is not the pinned one"
    assert run(capsys, "checkpoint", "verify", tmp_path / "packed", "--site", site_file(tmp_path, manifest_sha256=manifest))[0] == 0


def test_refusals_are_one_json_line_and_exit_status_2(source, tmp_path, capsys):
    code, _, err = run(capsys, "checkpoint", "pack", source, tmp_path / "packed", "--gpus", "2")  # never marked
    assert code == 2 and "mark-source" in refusal(err)["message"]
    empty = tmp_path / "empty"
    empty.mkdir()
    code, _, err = run(capsys, "checkpoint", "inventory", empty)
    assert code == 2 and refusal(err)["refused"] == "CheckpointValidationError"
    code, _, err = run(capsys, "checkpoint", "verify", empty)
    assert code == 2 and "never completed" in refusal(err)["message"]
    run(capsys, "checkpoint", "mark-source", source)
    run(capsys, "checkpoint", "pack", source, tmp_path / "packed", "--gpus", "2")
    code, _, err = run(capsys, "checkpoint", "pack", source, tmp_path / "packed", "--gpus", "2")
    assert code == 2 and "already a sealed checkpoint" in refusal(err)["message"]
    shard = tmp_path / "packed" / fmt.SHARED_FILE
    os.chmod(shard, 0o600)
    with open(shard, "r+b") as f:
        f.seek(-1, os.SEEK_END)
        last = f.read(1)
        f.seek(-1, os.SEEK_END)
        f.write(bytes([last[0] ^ 1]))
    code, _, err = run(capsys, "checkpoint", "verify", tmp_path / "packed")
    assert code == 2 and "content digest differs" in refusal(err)["message"]
    bad_site = tmp_path / "bad.toml"
    bad_site.write_text("[paths]\n")
    os.chmod(bad_site, 0o644)
    code, _, err = run(capsys, "checkpoint", "verify", tmp_path / "packed", "--site", bad_site)
    assert code == 2 and refusal(err)["refused"] == "ConfigValidationError" and "0600" in refusal(err)["message"]


def test_a_defect_still_looks_like_a_defect(source, tmp_path, capsys):
    run(capsys, "checkpoint", "mark-source", source)
    with pytest.raises(FileExistsError):  # not one of the refusals: the marker is create-once and the caller asked twice
        cli.main(["checkpoint", "mark-source", str(source)])


def test_a_fresh_process_reports_the_same_way(source, tmp_path):
    env = dict(os.environ, GLM_B200_RUN_ROOT=str(tmp_path / "runs"), GLM_B200_SITE_CONFIG=str(tmp_path / "no-site.toml"))
    done = subprocess.run([sys.executable, "-m", "glm_tpu_b200", "checkpoint", "verify", str(tmp_path / "nothing")], capture_output=True, text=True,
                          env=env, timeout=300)
    assert done.returncode == 2 and done.stdout == "" and "Traceback" not in done.stderr
    assert refusal(done.stderr)["refused"] == "CheckpointValidationError"
    done = subprocess.run([sys.executable, "-m", "glm_tpu_b200", "checkpoint", "inventory", str(source)], capture_output=True, text=True, env=env, timeout=300)
    assert done.returncode == 0 and json.loads(done.stdout)["ok"] and done.stderr == ""


def test_another_copy_of_the_source_is_checked_against_an_earlier_marker(source, tmp_path, capsys):
    """``mark-source --upstream-marker``: this copy against the marker made from another copy; the copy itself is not written to."""
    import shutil

    assert run(capsys, "checkpoint", "mark-source", source, "--hash-shards")[0] == 0
    upstream = tmp_path / "upstream.json"
    shutil.copy(source / source_marker.MARKER_FILE, upstream)
    copy = tmp_path / "copy"
    shutil.copytree(source, copy)
    (copy / source_marker.MARKER_FILE).unlink()
    code, out, _ = run(capsys, "checkpoint", "mark-source", copy, "--upstream-marker", upstream, "--output", tmp_path / "scratch.json")
    report = json.loads(out)
    assert code == 0 and report["matches_upstream"] and report["shards_compared_by_content"] and report["upstream_marker_sha256"] == fmt.file_sha256(upstream)
    assert not (copy / source_marker.MARKER_FILE).exists()  # compared, not marked
    assert json.loads((tmp_path / "scratch.json").read_text()) == json.loads(upstream.read_text())  # the same source gives the same record

    shard = sorted(copy.glob("*.safetensors"))[0]
    with open(shard, "r+b") as f:
        f.seek(-1, os.SEEK_END)
        last = f.read(1)
        f.seek(-1, os.SEEK_END)
        f.write(bytes([last[0] ^ 1]))  # one bit of one weight: same size, same headers
    code, _, err = run(capsys, "checkpoint", "mark-source", copy, "--upstream-marker", upstream)
    assert code == 2 and f"{shard.name}: content differs" in refusal(err)["message"]
    (copy / "config.json").write_text((copy / "config.json").read_text() + " ")
    code, _, err = run(capsys, "checkpoint", "mark-source", copy, "--upstream-marker", upstream)
    assert code == 2 and "2 respect(s)" in refusal(err)["message"] and "config.json: differs" in refusal(err)["message"]

    upstream.write_text("{oops")
    assert run(capsys, "checkpoint", "mark-source", source, "--upstream-marker", upstream)[0] == 2
    upstream.write_text(json.dumps({"schema": "something_else"}))
    code, _, err = run(capsys, "checkpoint", "mark-source", source, "--upstream-marker", upstream)
    assert code == 2 and "not a glm_b200_source_marker_v1 record" in refusal(err)["message"]
    code, _, err = run(capsys, "checkpoint", "mark-source", copy, "--output", tmp_path / "x.json")
    assert code == 2 and "goes with --upstream-marker" in refusal(err)["message"]


def test_verify_can_be_limited_to_some_files_or_to_the_headers(source, tmp_path, capsys):
    run(capsys, "checkpoint", "mark-source", source)
    run(capsys, "checkpoint", "pack", source, tmp_path / "packed", "--gpus", "2")
    mine = "experts.rank1of2.safetensors"
    code, out, _ = run(capsys, "checkpoint", "verify", tmp_path / "packed", "--files", fmt.SHARED_FILE, mine)
    assert code == 0 and sorted(json.loads(out)["files"]) == sorted([fmt.SHARED_FILE, mine]) and json.loads(out)["rehashed"] is True
    code, _, err = run(capsys, "checkpoint", "verify", tmp_path / "packed", "--files", "experts.rank5of2.safetensors")
    assert code == 2 and "is not part of this checkpoint" in refusal(err)["message"]
    other = tmp_path / "packed" / "experts.rank0of2.safetensors"
    os.chmod(other, 0o600)
    with open(other, "r+b") as f:
        f.seek(-1, os.SEEK_END)
        last = f.read(1)
        f.seek(-1, os.SEEK_END)
        f.write(bytes([last[0] ^ 1]))
    assert run(capsys, "checkpoint", "verify", tmp_path / "packed", "--files", mine)[0] == 0  # only what was asked for is read
    code, out, _ = run(capsys, "checkpoint", "verify", tmp_path / "packed", "--headers-only")
    assert code == 0 and json.loads(out)["rehashed"] is False  # sizes and headers are intact; the payload was not read
    code, _, err = run(capsys, "checkpoint", "verify", tmp_path / "packed")
    assert code == 2 and "experts.rank0of2.safetensors: content digest differs" in refusal(err)["message"]


def test_the_inventory_can_be_written_to_a_file(source, tmp_path, capsys):
    import hashlib

    from glm_tpu_b200.utils.json_utils import canonical_hash_bytes

    code, out, _ = run(capsys, "checkpoint", "inventory", source, "--output", tmp_path / "inventory.json")
    report = json.loads(out)
    assert code == 0 and report["output"] == str(tmp_path / "inventory.json")
    record = json.loads((tmp_path / "inventory.json").read_text())
    assert record["schema"] == "glm_b200_source_inventory_v1" and record["inventory_sha256"] == report["inventory_sha256"]
    assert len(record["tensors"]) == report["tensors"] and sum(record["shards"].values()) == report["total_bytes"]
    # the digest is the digest of the listing itself: anyone can recompute it from the file
    assert hashlib.sha256(canonical_hash_bytes({"tensors": record["tensors"], "shards": record["shards"]})).hexdigest() == record["inventory_sha256"]
    name, (dtype, shape, shard, begin, end) = sorted(record["tensors"].items())[0]
    assert (source / shard).stat().st_size >= end > begin and isinstance(shape, list) and dtype in ("BF16", "F32", "F8_E4M3")
    assert (tmp_path / "inventory.json").stat().st_mode & 0o077 == 0
    with pytest.raises(FileExistsError):
        cli.main(["checkpoint", "inventory", str(source), "--output", str(tmp_path / "inventory.json")])  # create-once


def test_ask_refuses_in_one_json_line_too(tmp_path, monkeypatch, capsys):
    monkeypatch.setenv("GLM_B200_RUN_ROOT", str(tmp_path / "runs"))
    monkeypatch.setenv("GLM_B200_SITE_CONFIG", str(tmp_path / "no-site.toml"))
    questions = tmp_path / "q.json"
    questions.write_text(json.dumps(["one"] * 11))
    os.chmod(questions, 0o600)
    code, out, err = run(capsys, "ask", "--questions", questions, "--model", "random:tiny", "--capacity", "128", "--prepare-only")
    assert code == 2 and out == "" and refusal(err) == {"ok": False, "refused": "RequestValidationError", "message": "provide one to ten nonempty question strings"}
    code, _, err = run(capsys, "ask", "x" * 400, "--model", "random:tiny", "--capacity", "128", "--prepare-only")
    assert code == 2 and "no room for an answer" in refusal(err)["message"] or "exceed" in refusal(err)["message"]
    code, out, _ = run(capsys, "ask", "2+2?", "--model", "random:tiny", "--capacity", "128", "--prepare-only")
    assert code == 0 and out.startswith("PRIVATE_INPUT ")


def test_two_asks_in_the_same_second_get_their_own_input_directories(tmp_path, monkeypatch, capsys):
    monkeypatch.setenv("GLM_B200_RUN_ROOT", str(tmp_path / "runs"))
    monkeypatch.setenv("GLM_B200_SITE_CONFIG", str(tmp_path / "no-site.toml"))
    import time as time_module

    monkeypatch.setattr(time_module, "strftime", lambda fmt, *a: "20260101T000000")  # the clock stands still
    staged = []
    for question in ("one?", "two?", "three?"):
        code, out, _ = run(capsys, "ask", question, "--model", "random:tiny", "--capacity", "128", "--prepare-only")
        assert code == 0
        staged.append(out.split("PRIVATE_INPUT ", 1)[1].strip())
    assert len(set(staged)) == 3 and all(os.path.exists(p) for p in staged)

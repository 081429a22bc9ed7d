"""Thin wrappers over ``tools/equivalence``: the gates must match their goldens, and the mutation self-test must catch every mutant."""

import json
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[2]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from tools.equivalence import compare_run, driver, imports  # noqa: E402


@pytest.mark.parametrize("gate", ["g2_production_defaults", "g3_oracle_digests", "g4_checkpoint_identity", "g9_wire_formats"])
def test_gate_matches_golden(gate):
    assert driver.check({gate}) == {}


@pytest.mark.gpu
def test_launch_programs_match_golden():
    """The ordered launch list (entry point + integer arguments) of a decode step and a prefill chunk, per configuration."""
    if not (driver.DATA / "g1_launch_programs.json").exists():
        pytest.skip("no launch programs recorded yet: python -m tools.equivalence.driver update g1_launch_programs on a B200")
    golden = driver.load("g1_launch_programs")
    assert {"glm53x8.shard-of-8.chats1", "glm53x8.shard-of-8.chats4", "small4.gpus1.chats1"} <= set(golden)
    assert driver.check({"g1_launch_programs"}) == {}


@pytest.mark.slow
def test_import_closures_only_shrink():
    assert driver.check({"g6_import_closures"}) == {}


def test_executed_function_set_matches_golden():
    from tools.equivalence import executed

    assert driver.check({"g7_executed_functions"}) == {}
    golden = driver.load("g7_executed_functions")["functions"]
    assert "glm_tpu_b200.engine.llm_engine:LLMEngine.generate" in golden and "glm_tpu_b200.oracle.contract:top_k_positions" in golden
    assert not any(name.startswith(("glm_tpu_b200.ops", "glm_tpu_b200.runner.gpu_runner")) for name in golden)  # the CPU scenario stays device-free
    moved = executed.difference({"functions": ["a:f", "a:g"]}, {"functions": ["a:g", "b:h"]})
    assert moved == {"no_longer_executed": ["a:f"], "newly_executed": ["b:h"]}


def test_entry_points_stay_light():
    golden = driver.load("g6_import_closures")
    assert golden["glm_tpu_b200.entrypoints.cli.main"]["heavy"] == []  # `info` and `--help` never import torch
    assert "torch" not in golden["glm_tpu_b200.config.site"]["heavy"]
    assert not any(m.startswith("glm_tpu_b200.ops") for m in golden["glm_tpu_b200.engine.llm_engine"]["modules"])  # the engine is device-free
    assert not any(m.startswith("glm_tpu_b200.models") for m in golden["glm_tpu_b200.entrypoints.serve.http_handler"]["modules"])
    assert imports.grown(golden, golden) == {}
    assert imports.grown({"x": {"modules": ["a"], "heavy": []}}, {"x": {"modules": ["a", "b"], "heavy": ["torch"]}}) == {"x": {"modules": ["b"], "heavy": ["torch"]}}


@pytest.mark.slow
def test_mutation_selftest_catches_every_mutant():
    from tools.equivalence import selftest

    results = selftest.run()
    assert results and all(results.values()), results


def test_compare_run(tmp_path):
    def make(run, tokens):
        d = tmp_path / run
        d.mkdir()
        (d / "runner.rank0.json").write_text(json.dumps({"requests": [{"request_id": "question-01", "request_sha256": "ab" * 32}]}))
        (d / "tokens.jsonl").write_text("".join(json.dumps({"request_id": "question-01", "index": i, "token_id": t, "finish_reason": None}) + "\n"
                                                for i, t in enumerate(tokens)))
        return d

    a, b, c = make("a", [5, 6, 7]), make("b", [5, 6, 7]), make("c", [5, 9, 7])
    assert compare_run.compare(a, b) == (1, [])
    matched, diffs = compare_run.compare(a, c)
    assert matched == 1 and diffs[0]["first_difference"] == 1
    assert compare_run.main([str(a), str(b)]) == 0 and compare_run.main([str(a), str(c)]) == 1 and compare_run.main([str(a), str(tmp_path)]) in (0, 1, 2)


def test_the_gate_command_line(tmp_path, monkeypatch, capsys):
    """``python -m tools.equivalence.driver check|update [gate ...]``: exit status 0 and one line when the goldens match, 1 and the
    differing keys (golden against current) when they do not; ``update`` rewrites only the gates it is given."""
    import shutil

    data = tmp_path / "data"
    shutil.copytree(driver.DATA, data)
    monkeypatch.setattr(driver, "DATA", data)
    assert driver.main(["check", "g9_wire_formats", "g4_checkpoint_identity"]) == 0
    assert capsys.readouterr().out.strip() == "all gates match"

    golden = json.loads((data / "g9_wire_formats.json").read_text())
    (data / "g9_wire_formats.json").write_text(json.dumps(dict(golden, sse_chunks="0" * 64, retired_key="x")))
    before_g4 = (data / "g4_checkpoint_identity.json").read_bytes()
    assert driver.main(["check", "g9_wire_formats", "g4_checkpoint_identity"]) == 1
    report = json.loads(capsys.readouterr().out)
    assert set(report) == {"g9_wire_formats"} and set(report["g9_wire_formats"]) == {"sse_chunks", "retired_key"}
    assert report["g9_wire_formats"]["sse_chunks"] == {"golden": "0" * 64, "current": golden["sse_chunks"]}
    assert report["g9_wire_formats"]["retired_key"] == {"golden": "x", "current": None}

    assert driver.main(["update", "g9_wire_formats"]) == 0
    assert json.loads((data / "g9_wire_formats.json").read_text()) == golden and (data / "g4_checkpoint_identity.json").read_bytes() == before_g4
    assert driver.main(["check", "g9_wire_formats"]) == 0
    assert sorted(p.name for p in data.iterdir()) == sorted(p.name for p in driver.DATA.iterdir())  # nothing else was written


def test_goldens_are_canonical_files():
    """Sorted keys, one-space indent, newline at the end: a regenerated golden that did not change gives no diff."""
    for path in sorted(driver.DATA.glob("*.json")):
        text = path.read_text()
        assert text == json.dumps(json.loads(text), indent=1, sort_keys=True) + "\n", path.name
    assert {p.stem for p in driver.DATA.glob("*.json")} == set(driver.gates())

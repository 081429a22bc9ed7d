"""Unit tier (pure Python, no GPU): file discipline, canonical JSON, environment registry, cache striping arithmetic, memory admission,
the static collective plan check and the launch policy on real temporary git repositories.

Mirrors the reference's `tests/utils/test_io_utils.py`, `tests/config/test_cache.py`, `tests/runner/test_admission.py` and
`tests/executor/test_launch_policy.py`.
"""

import json
import os
import stat
import subprocess

import pytest

from glm_tpu_b200.config.cache import CacheConfig
from glm_tpu_b200.config.model import glm53_geometry, tiny_geometry
from glm_tpu_b200.config.parallel import ParallelLayout
from glm_tpu_b200.exceptions import ConfigValidationError, PlanValidationError
from glm_tpu_b200.executor import launch_policy
from glm_tpu_b200.runner import admission
from glm_tpu_b200.utils import io_utils, json_utils


# ------------------------------------------------------------------------------------------------------- files
def test_exclusive_private_create_never_overwrites(tmp_path):
    target = tmp_path / "record.json"
    io_utils.create_private_exclusive(target, b"one")
    assert stat.S_IMODE(target.stat().st_mode) == 0o600 and target.read_bytes() == b"one"
    with pytest.raises(FileExistsError):
        io_utils.create_private_exclusive(target, b"two")
    link = tmp_path / "link"
    link.symlink_to(tmp_path / "elsewhere")
    with pytest.raises(OSError):
        io_utils.create_private_exclusive(link, b"x")  # O_NOFOLLOW | O_EXCL: a planted link is not followed
    assert not (tmp_path / "elsewhere").exists()


def test_collected_records_are_kept_side_by_side_when_they_differ(tmp_path):
    divergent: list[str] = []
    io_utils.write_collected(tmp_path, "summary.json", b'{"a": 1}', divergent)
    io_utils.write_collected(tmp_path, "summary.json", b'{"a":1}', divergent)  # the same JSON value: nothing to keep
    assert divergent == [] and not (tmp_path / "final").exists()
    io_utils.write_collected(tmp_path, "summary.json", b'{"a": 2}', divergent)
    io_utils.write_collected(tmp_path, "summary.json", b'{"a": 3}', divergent)
    io_utils.write_collected(tmp_path, "summary.json", b'{"a": 3}', divergent)
    assert divergent == ["summary.json"]
    assert (tmp_path / "summary.json").read_bytes() == b'{"a": 1}'  # the first record is never replaced
    assert sorted(p.name for p in (tmp_path / "final").iterdir()) == ["summary.json", "summary.json.1"]
    for bad in ("", ".", "..", "a/b", "a\0b"):
        with pytest.raises(ValueError):
            io_utils.write_collected(tmp_path, bad, b"x", divergent)


def test_bounded_reads_and_plain_paths(tmp_path):
    small = tmp_path / "in.json"
    small.write_bytes(b"12345")
    assert io_utils.read_bounded(small, 5) == b"12345"
    with pytest.raises(ValueError):
        io_utils.read_bounded(small, 4)
    (tmp_path / "empty").write_bytes(b"")
    with pytest.raises(ValueError):
        io_utils.read_bounded(tmp_path / "empty", 10)
    real = tmp_path / "real"
    real.mkdir()
    (real / "f").write_bytes(b"x")
    (tmp_path / "alias").symlink_to(real)
    with pytest.raises(ValueError, match="symlink"):
        io_utils.read_bounded(tmp_path / "alias" / "f", 10)
    with pytest.raises(ValueError):
        io_utils.read_bounded(real, 10)  # a directory is not a regular file


def test_private_files_are_required_to_be_closed_to_others(tmp_path):
    key = tmp_path / "api.key"
    key.write_text("secret")
    os.chmod(key, 0o644)
    with pytest.raises(ValueError, match="closed to group and others"):
        io_utils.require_private(key)
    os.chmod(key, 0o600)
    io_utils.require_private(key)


def test_atomic_and_persisted_json_leave_no_temporary_file(tmp_path):
    io_utils.atomic_json(tmp_path / "state.json", {"ü": 1})
    io_utils.persist_json(tmp_path / "report.json", {"b": 2, "a": 1})
    assert json.loads((tmp_path / "state.json").read_text(encoding="utf-8")) == {"ü": 1}
    assert (tmp_path / "report.json").read_text() == '{\n  "a": 1,\n  "b": 2\n}\n'
    assert sorted(p.name for p in tmp_path.iterdir()) == ["report.json", "state.json"]


# ------------------------------------------------------------------------------------------------------- canonical JSON
def test_wire_bytes_are_utf8_and_hash_bytes_are_ascii():
    value = {"b": [1, 2.5, None, True], "a": "grüß"}
    assert json_utils.canonical_wire_bytes(value) == '{"a":"grüß","b":[1,2.5,null,true]}'.encode("utf-8")
    assert json_utils.canonical_hash_bytes(value) == b'{"a":"gr\\u00fc\\u00df","b":[1,2.5,null,true]}'
    assert json_utils.fingerprint(value) == json_utils.fingerprint({"a": "grüß", "b": [1, 2.5, None, True]})
    assert json_utils.fingerprint(value) != json_utils.fingerprint({"a": "gruß", "b": [1, 2.5, None, True]})
    with pytest.raises(ValueError):
        json_utils.canonical_wire_bytes({"x": float("nan")})


# ------------------------------------------------------------------------------------------------------- environment registry
def test_environment_registry_is_lazy_and_rejects_unknown_names(monkeypatch):
    from glm_tpu_b200 import envs

    monkeypatch.delenv("GLM_B200_RUN_ROOT", raising=False)
    assert not envs.is_set("GLM_B200_RUN_ROOT")
    monkeypatch.setenv("GLM_B200_RUN_ROOT", "/tmp/run-root")
    assert envs.is_set("GLM_B200_RUN_ROOT") and str(envs.GLM_B200_RUN_ROOT) == "/tmp/run-root"  # read when asked, not at import
    monkeypatch.setenv("GLM_B200_RUN_ROOT", "relative/path")
    with pytest.raises(Exception):
        envs.GLM_B200_RUN_ROOT  # noqa: B018  (paths are absolute)
    with pytest.raises(AttributeError):
        envs.GLM_B200_NO_SUCH_VARIABLE  # noqa: B018
    report = envs.describe()
    assert "GLM_B200_RUN_ROOT" in dir(envs) and set(report) >= {"GLM_B200_RUN_ROOT", "GLM_B200_SITE_CONFIG"}
    assert report["GLM_B200_RUN_ROOT"].startswith("<invalid")  # the environment report lists a bad value instead of failing


# ------------------------------------------------------------------------------------------------------- cache striping
@pytest.mark.parametrize("world,stripe", [(1, 64), (2, 64), (8, 64), (4, 16)])
def test_striping_is_a_bijection_and_owned_counts_add_up(world, stripe):
    cache = CacheConfig(tiny_geometry(), context_capacity=world * stripe * 4, world=world, stripe=stripe)
    seen = set()
    for pos in range(cache.context_capacity):
        rank, row = cache.owner(pos), cache.local_row(pos)
        assert 0 <= rank < world and 0 <= row < cache.local_capacity
        assert cache.global_position(rank, row) == pos
        seen.add((rank, row))
    assert len(seen) == cache.context_capacity
    for ctx in (0, 1, stripe - 1, stripe, stripe + 1, cache.page, cache.page + 3, cache.context_capacity):
        counts = [cache.owned_count(r, ctx) for r in range(world)]
        assert sum(counts) == ctx
        assert counts == [sum(1 for p in range(ctx) if cache.owner(p) == r) for r in range(world)]
        for r in range(world):  # the rows a rank owns below ctx are exactly its first owned_count rows
            rows = sorted(cache.local_row(p) for p in range(ctx) if cache.owner(p) == r)
            assert rows == list(range(counts[r]))


def test_cache_config_refusals_and_production_sizes():
    g = glm53_geometry()
    with pytest.raises(PlanValidationError):
        CacheConfig(g, context_capacity=32768 + 64, world=8)   # not a multiple of the 512-position page
    with pytest.raises(PlanValidationError):
        CacheConfig(g, context_capacity=32768, lanes=9)
    with pytest.raises(PlanValidationError):
        CacheConfig(g, context_capacity=32768, world=0)
    striped = CacheConfig(g, context_capacity=32768, world=8)
    assert striped.page == 512 and striped.local_capacity == 4096
    assert striped.kv_cache_shape == (1, 78, 4096, 576) and striped.index_cache_shape == (1, 21, 4096, 128)
    replica = CacheConfig(g, context_capacity=32768, world=1)
    assert replica.cache_bytes_per_gpu() == 8 * striped.cache_bytes_per_gpu() == 32768 * (78 * 576 + 21 * 128) * 2


# ------------------------------------------------------------------------------------------------------- admission
def test_memory_admission_admits_the_published_profiles_and_refuses_what_cannot_fit():
    g = glm53_geometry()
    layout = ParallelLayout(g, 8, 0)
    weights = 95 << 30  # about what one of eight GPUs holds
    for capacity, lanes in ((32768, 4), (166912, 1), (262144, 1)):
        cache = CacheConfig(g, context_capacity=capacity, world=1, lanes=lanes)
        projection = admission.project_memory(g, layout, cache, weights, staging_bytes=256 << 20)
        assert projection["admitted"] and projection["total"] == sum(projection[k] for k in ("weights", "caches", "staging", "workspace"))
        admission.require_admitted(projection)
    too_big = CacheConfig(g, context_capacity=262144, world=1, lanes=8)
    projection = admission.project_memory(g, layout, too_big, weights, staging_bytes=256 << 20)
    assert not projection["admitted"]
    with pytest.raises(PlanValidationError, match="memory admission refused"):
        admission.require_admitted(projection)


def test_collective_plan_check_enforces_the_exchange_protocol():
    ar = lambda ch, ctas=24, floats=256: {"kind": "allreduce", "channel": ch, "ctas": ctas, "floats_per_cta": floats}  # noqa: E731
    sig = lambda s: {"kind": "signal", "signal": s}  # noqa: E731
    layer = [sig(0), sig(1), sig(2), ar(0), ar(1)]
    admission.check_collective_plan(layer * 3, world=8)
    admission.check_collective_plan([ar(0), ar(0)], world=1)  # a single GPU exchanges nothing
    with pytest.raises(PlanValidationError, match="same channel"):
        admission.check_collective_plan([ar(0), sig(0), ar(0)], world=8)
    with pytest.raises(PlanValidationError, match="raised twice"):
        admission.check_collective_plan([sig(1), sig(1), ar(0)], world=8)
    with pytest.raises(PlanValidationError, match="exceeds"):
        admission.check_collective_plan([ar(0, ctas=2000)], world=8)
    with pytest.raises(PlanValidationError, match="exceeds"):
        admission.check_collective_plan([ar(0, floats=512)], world=8)


# ------------------------------------------------------------------------------------------------------- launch policy
def _git(repo, *args):
    subprocess.run(["git", "-C", str(repo), *args], check=True, capture_output=True,
                   env={**os.environ, "GIT_AUTHOR_NAME": "t", "GIT_AUTHOR_EMAIL": "t@t", "GIT_COMMITTER_NAME": "t", "GIT_COMMITTER_EMAIL": "t@t"})


def test_launch_policy_on_real_repositories(tmp_path):
    plain = tmp_path / "plain"
    plain.mkdir()
    identity = launch_policy.source_identity(plain)
    assert identity["git"] is False
    launch_policy.check(identity, "record")
    with pytest.raises(ConfigValidationError, match="git checkout"):
        launch_policy.check(identity, "strict")
    with pytest.raises(ConfigValidationError, match="'record' or 'strict'"):
        launch_policy.check(identity, "lenient")

    repo = tmp_path / "repo"
    repo.mkdir()
    _git(repo, "init", "-q", "-b", "main")
    (repo / "a.txt").write_text("1")
    _git(repo, "add", "a.txt")
    _git(repo, "commit", "-q", "-m", "one")
    clean = launch_policy.source_identity(repo)
    assert clean["git"] and clean["clean"] and clean["branch"] == "main" and len(clean["commit"]) == 40
    launch_policy.check(clean, "strict")
    (repo / "a.txt").write_text("2")
    dirty = launch_policy.source_identity(repo)
    assert dirty["clean"] is False and dirty["dirty_files"] == 1
    launch_policy.check(dirty, "record")
    with pytest.raises(ConfigValidationError, match="uncommitted"):
        launch_policy.check(dirty, "strict")
    _git(repo, "checkout", "-q", "--", "a.txt")
    _git(repo, "checkout", "-q", "--detach")
    with pytest.raises(ConfigValidationError, match="detached"):
        launch_policy.check(launch_policy.source_identity(repo), "strict")


def test_every_registered_variable_is_read_somewhere():
    """A variable in the registry that nothing reads would be documented, validated and without effect."""
    import re
    from pathlib import Path

    from glm_tpu_b200 import envs

    root = Path(__file__).resolve().parents[1]
    product = "\n".join(p.read_text() for p in (root / "glm_tpu_b200").rglob("*.py") if p.name != "envs.py") + (root / "bench.py").read_text()
    tests = "\n".join(p.read_text() for p in (root / "tests").rglob("*.py"))
    product += "\n".join(re.findall(r'value_of\("(GLM_B200_[A-Z0-9_]+)"\)', (root / "glm_tpu_b200" / "envs.py").read_text()))  # defaults built on another variable
    for name in envs.TABLE:
        where = tests if name.startswith("GLM_B200_TEST_") else product
        assert re.search(r"\b" + name + r"\b", where), f"{name} is registered but never read"
    # and the other way round: a GLM_B200_* name the product reads is one the registry knows (a typo would silently do nothing)
    for name in set(re.findall(r"\bGLM_B200_[A-Z0-9_]+\b", product)):
        assert name in envs.TABLE or name == "GLM_B200_WORKER", f"{name} is read but not registered"


def test_runner_defaults_follow_the_registry(monkeypatch):
    from glm_tpu_b200 import envs

    for name in ("GLM_B200_COMM", "GLM_B200_CUDA_GRAPHS", "GLM_B200_WAIT_LIMIT"):
        monkeypatch.delenv(name, raising=False)
    assert (envs.GLM_B200_COMM, envs.GLM_B200_CUDA_GRAPHS, envs.GLM_B200_WAIT_LIMIT) == ("fused", True, 2_000_000)
    monkeypatch.setenv("GLM_B200_COMM", "nccl")
    monkeypatch.setenv("GLM_B200_CUDA_GRAPHS", "0")
    monkeypatch.setenv("GLM_B200_WAIT_LIMIT", "500000")
    assert (envs.GLM_B200_COMM, envs.GLM_B200_CUDA_GRAPHS, envs.GLM_B200_WAIT_LIMIT) == ("nccl", False, 500000)
    monkeypatch.setenv("GLM_B200_COMM", "mpi")
    with pytest.raises(ValueError, match="GLM_B200_COMM must be one of fused, nccl"):
        envs.GLM_B200_COMM

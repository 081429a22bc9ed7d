"""What binds a worker to its controller, and what refuses it (CPU only; failures are made on the host).

The site's pins must reach the loader, the staged site / source manifest / topology binding must be the controller's, the
memory admission must refuse before anything is allocated and before every request, and the launch rules must refuse a
checkout that is dirty, on the wrong branch, from another origin or not pushed.
"""

import argparse
import hashlib
import json
import os
import subprocess
from pathlib import Path

import pytest
import torch

from glm_tpu_b200.config.model import tiny_geometry
from glm_tpu_b200.config.site import Paths, SiteConfig
from glm_tpu_b200.engine import request as rq
from glm_tpu_b200.engine.llm_engine import LLMEngine
from glm_tpu_b200.engine.request_session import LocalVote
from glm_tpu_b200.exceptions import CheckpointValidationError, ConfigValidationError, PlanValidationError
from glm_tpu_b200.executor import launch_policy, multiproc_executor, source_manifest
from glm_tpu_b200.model_loader import export, source_marker
from glm_tpu_b200.model_loader.sharded_state import loader
from glm_tpu_b200.models.glm_moe_dsa.weights import random_checkpoint
from glm_tpu_b200.parallel import topology as topo
from glm_tpu_b200.runner import admission
from glm_tpu_b200.worker import gpu_worker

REPO = Path(__file__).resolve().parents[1]


def _worker_args(run_dir, **over):
    base = dict(run_dir=str(run_dir), request=None, request_sha256=None, keep_loaded=True, backend="oracle", site_json=None, site_sha256=None,
                source_manifest=None, source_manifest_sha256=None, binding=None, binding_sha256=None)
    base.update(over)
    return argparse.Namespace(**base)


def _site(tmp_path, **over):
    return SiteConfig(gpus=2, paths=Paths(tmp_path / "runs", None, None, tmp_path / "state"), **over)


# ------------------------------------------------------------------------------------------------ site + pins
def test_staged_site_must_be_the_controllers(tmp_path):
    site = _site(tmp_path, manifest_sha256="a" * 64)
    run_dir = tmp_path / "runs" / "run-1"
    run_dir.mkdir(parents=True)
    args = multiproc_executor.stage_site(run_dir, site)
    assert args[0] == "--site-json" and args[3] == site.sha256
    back = SiteConfig.from_staged(Path(args[1]), site.sha256)
    assert back.sha256 == site.sha256 and back.checkpoint_pins["manifest_sha256"] == "a" * 64
    with pytest.raises(ConfigValidationError, match="digest differs"):
        SiteConfig.from_staged(Path(args[1]), "0" * 64)
    # bytes with the right digest that are not a canonical resolved site are refused too
    odd = run_dir / "odd.json"
    odd.write_bytes(b'{"gpus": 2}')
    with pytest.raises(ConfigValidationError):
        SiteConfig.from_staged(odd, hashlib.sha256(odd.read_bytes()).hexdigest())


def test_worker_authenticates_what_the_controller_staged(tmp_path):
    site = _site(tmp_path)
    run_dir = tmp_path / "runs" / "run-1"
    run_dir.mkdir(parents=True)
    staged = multiproc_executor.stage_site(run_dir, site) + multiproc_executor.stage_source_manifest(run_dir, REPO)
    flags = {staged[i][2:].replace("-", "_"): staged[i + 1] for i in range(0, len(staged), 2)}
    launch = gpu_worker.authenticate_launch(_worker_args(run_dir, **flags))
    assert launch["site"].sha256 == site.sha256 and launch["pins"] == site.checkpoint_pins and launch["binding"] is None
    # a run directory somewhere else than under the staged run_root
    elsewhere = tmp_path / "elsewhere" / "run-1"
    elsewhere.mkdir(parents=True)
    with pytest.raises(SystemExit, match="run_root"):
        gpu_worker.authenticate_launch(_worker_args(elsewhere, **flags))
    # a digest without its file
    with pytest.raises(SystemExit, match="come together"):
        gpu_worker.authenticate_launch(_worker_args(run_dir, site_sha256=site.sha256))
    # a manifest that is not the controller's
    with pytest.raises(SystemExit, match="source manifest"):
        gpu_worker.authenticate_launch(_worker_args(run_dir, **dict(flags, source_manifest_sha256="0" * 64)))


def test_source_manifest_catches_a_changed_tree(tmp_path):
    pkg = tmp_path / "glm_tpu_b200" / "worker"
    pkg.mkdir(parents=True)
    (pkg / "gpu_worker.py").write_text("x = 1\n")
    (tmp_path / "glm_tpu_b200" / "__init__.py").write_text("")
    manifest = source_manifest.build(tmp_path)
    assert set(manifest) == {"glm_tpu_b200/__init__.py", "glm_tpu_b200/worker/gpu_worker.py"}
    source_manifest.verify(tmp_path, manifest, must_contain="glm_tpu_b200/worker/gpu_worker.py")
    with pytest.raises(ConfigValidationError, match="does not list"):
        source_manifest.verify(tmp_path, manifest, must_contain="glm_tpu_b200/other.py")
    (pkg / "gpu_worker.py").write_text("x = 2\n")
    with pytest.raises(ConfigValidationError, match="differs"):
        source_manifest.verify(tmp_path, manifest)
    with pytest.raises(ConfigValidationError):
        source_manifest.verify(tmp_path, {"../outside.py": "0" * 64})


def test_a_wrong_checkpoint_pin_makes_the_worker_refuse_to_load(tmp_path):
    from glm_tpu_b200.executor.pack_job import pack_checkpoint

    g = tiny_geometry()
    export.export_source(random_checkpoint(g, seed=3), g, tmp_path / "src", shards=2)
    source_marker.mark_source(tmp_path / "src")
    report = pack_checkpoint(tmp_path / "src", tmp_path / "packed", 2, jobs=1)
    good = _site(tmp_path, manifest_sha256=report["manifest_sha256"]).checkpoint_pins
    assert "__experts_presliced__" in loader.load_rank_checkpoint(tmp_path / "packed", 0, 2, pins=good)
    wrong = _site(tmp_path, manifest_sha256="b" * 64).checkpoint_pins
    with pytest.raises(CheckpointValidationError, match="pinned"):
        loader.load_rank_checkpoint(tmp_path / "packed", 0, 2, pins=wrong)

    # the same through the worker: the staged site's pin travels into Worker.load
    run_dir = tmp_path / "runs" / "run-1"
    run_dir.mkdir(parents=True)
    site = _site(tmp_path, manifest_sha256="b" * 64)
    staged = multiproc_executor.stage_site(run_dir, site)
    args = gpu_worker.parse_args(["--run-dir", str(run_dir), "--keep-loaded", "--model", str(tmp_path / "packed"), "--backend", "oracle",
                                  "--site-json", staged[1], "--site-sha256", staged[3]])
    args.launch = gpu_worker.authenticate_launch(args)
    worker = gpu_worker.Worker(args, None)
    assert worker.launch["pins"]["manifest_sha256"] == "b" * 64


# ------------------------------------------------------------------------------------------------ topology binding
class _FakeNvml:
    NVML_P2P_CAPS_INDEX_NVLINK, NVML_P2P_STATUS_OK = 2, 0

    class NVMLError(Exception):
        pass

    def __init__(self, n=2, swap=False):
        self.n, self.swap = n, swap

    def nvmlInit(self):
        pass

    def nvmlShutdown(self):
        pass

    def nvmlDeviceGetCount(self):
        return self.n

    def nvmlDeviceGetHandleByIndex(self, i):
        return i

    def nvmlDeviceGetNvLinkState(self, h, link):
        return 1

    def nvmlDeviceGetCudaComputeCapability(self, h):
        return 10, 0

    def nvmlDeviceGetUUID(self, h):
        return f"GPU-{(h + 7 if self.swap else h):08d}-0000-0000-0000-000000000000"

    def nvmlDeviceGetName(self, h):
        return "NVIDIA B200"

    def nvmlDeviceGetPciInfo(self, h):
        return argparse.Namespace(busId=f"0000:{h + 1:02x}:00.0")

    def nvmlDeviceGetMemoryInfo(self, h):
        return argparse.Namespace(total=183359 << 20)

    def nvmlDeviceGetP2PStatus(self, a, b, caps):
        return 0

    def nvmlSystemGetDriverVersion(self):
        return "580.159"


def test_binding_is_authenticated_against_the_live_box_and_against_the_pin(tmp_path):
    binding = topo.derive_topology_binding(topo.discover_topology(_FakeNvml()), 2)
    state = tmp_path / "state"
    state.mkdir()
    (state / "topology_binding.json").write_text(json.dumps(binding))
    run_dir = tmp_path / "runs" / "run-1"
    run_dir.mkdir(parents=True)
    site = _site(tmp_path, topology_binding_sha256=binding["binding_sha256"])
    args, env = multiproc_executor.stage_binding(run_dir, site, None, 2, nvml=_FakeNvml())
    assert args[0] == "--binding" and args[3] == binding["binding_sha256"] and env["CUDA_VISIBLE_DEVICES"] == topo.visible_devices(binding)
    # the same binding on a box whose GPUs are others
    run2 = tmp_path / "runs" / "run-2"
    run2.mkdir()
    with pytest.raises(ConfigValidationError, match="not where the binding says"):
        multiproc_executor.stage_binding(run2, site, None, 2, nvml=_FakeNvml(swap=True))
    # another binding than the pinned one
    with pytest.raises(ConfigValidationError, match="pinned"):
        multiproc_executor.stage_binding(run2, _site(tmp_path, topology_binding_sha256="c" * 64), None, 2, nvml=_FakeNvml())
    # a launch over another number of GPUs than the binding's
    with pytest.raises(ConfigValidationError, match="GPUs"):
        multiproc_executor.stage_binding(run2, site, None, 4, nvml=_FakeNvml())
    # no pin, no binding: nothing is staged
    assert multiproc_executor.stage_binding(run2, _site(tmp_path), None, 2) == ([], {})

    # the worker: the staged binding must be the site's, and cuda:<local_rank> must be the GPU it names
    staged_site = multiproc_executor.stage_site(run_dir, site)
    flags = dict(site_json=staged_site[1], site_sha256=staged_site[3], binding=args[1], binding_sha256=args[3], backend="gpu")
    launch = gpu_worker.authenticate_launch(_worker_args(run_dir, **flags))
    assert launch["binding"]["binding_sha256"] == binding["binding_sha256"]
    with pytest.raises(SystemExit, match="staged none"):
        gpu_worker.authenticate_launch(_worker_args(run_dir, site_json=staged_site[1], site_sha256=staged_site[3], backend="gpu"))
    ns = _worker_args(run_dir, **flags)
    ns.launch = launch
    for field, value in (("model", "random:tiny"), ("lanes", 1), ("context", 0), ("comm", "fused"), ("kv_layout", "auto"), ("seed", 0)):
        setattr(ns, field, value)
    worker = gpu_worker.Worker(ns, None)
    worker.world, worker.rank, worker.local_rank = 2, 1, 1
    worker.digest_consensus = lambda digest: True
    worker.check_bound_device(device_uuid=lambda i: binding["ranks"][i]["uuid"])
    assert worker.record["topology_binding_sha256"] == binding["binding_sha256"]
    with pytest.raises(SystemExit, match="binding says"):
        worker.check_bound_device(device_uuid=lambda i: "GPU-elsewhere")


# ------------------------------------------------------------------------------------------------ admission
def test_live_admission_refuses_before_allocation_and_before_a_request():
    projection = {"weights": 90 << 30, "caches": 4 << 30, "staging": 1 << 30, "workspace": 1 << 30, "total": 96 << 30, "limit": 168 << 30, "admitted": True}
    # the weights are resident; 6 GiB more are needed, plus the reserve
    ok = admission.project_live(projection, free_bytes=10 << 30, total_bytes=179 << 30, already_resident=90 << 30)
    assert ok["admitted"] and ok["to_allocate"] == 6 << 30
    tight = admission.project_live(projection, free_bytes=6 << 30, total_bytes=179 << 30, already_resident=90 << 30)
    assert not tight["admitted"]
    with pytest.raises(PlanValidationError, match="admission refused"):
        admission.require_admitted(tight)
    # a static projection that does not fit stays refused whatever is free
    assert not admission.project_live(dict(projection, admitted=False), 170 << 30, 179 << 30, already_resident=0)["admitted"]


class _Runner:
    """The least an engine needs of a runner; ``admit_request`` fails when told to."""

    def __init__(self):
        self.lanes, self.fail = 1, False
        self.cache = argparse.Namespace(context_capacity=64)
        self.calls = []

    def admit_request(self):
        self.calls.append("admit")
        if self.fail:
            raise PlanValidationError("memory admission refused: needs 1.00 GiB, limit 0.50 GiB")

    def deactivate(self, lane):
        pass

    def prefill(self, lane, ids):
        self.calls.append("prefill")
        return 5

    def read_status(self):
        return 0

    def decode_step(self):
        self.calls.append("decode")

    def read_last_tokens(self):
        return [6]

    def read_step_tokens(self, index):
        return [6]


def test_engine_admits_every_request_and_a_refusal_poisons_it():
    profile = rq.RequestProfile.for_geometry(tiny_geometry(), (64,), concurrent_capacity=64)
    request = rq.from_token_ids([1, 2, 3], request_id="r1", max_new_tokens=2, context_capacity=64, profile=profile)
    runner, vote = _Runner(), LocalVote()
    engine = LLMEngine(runner, vote=vote, profile=profile)
    engine.generate(request, None)
    assert runner.calls[:2] == ["admit", "prefill"] and vote.log[0][0] == "admission"
    runner.calls.clear()
    runner.fail = True
    with pytest.raises(PlanValidationError):
        engine.generate(request, None)
    assert runner.calls == ["admit"] and engine.poisoned  # nothing ran after the refusal, and nothing will


# ------------------------------------------------------------------------------------------------ launch rules
def _git(cwd, *args):
    subprocess.run(["git", *args], cwd=cwd, check=True, capture_output=True,
                   env=dict(os.environ, GIT_AUTHOR_NAME="t", GIT_AUTHOR_EMAIL="t@t", GIT_COMMITTER_NAME="t", GIT_COMMITTER_EMAIL="t@t"))


def test_launch_rules_in_order_on_real_repositories(tmp_path):
    origin = tmp_path / "origin.git"
    _git(tmp_path, "init", "--bare", "-b", "main", str(origin))
    work = tmp_path / "work"
    _git(tmp_path, "clone", str(origin), str(work))
    (work / "a.txt").write_text("1\n")
    _git(work, "checkout", "-b", "main")
    _git(work, "add", "a.txt")
    _git(work, "commit", "-m", "one")
    rules = launch_policy.LaunchRules("strict", ("main", "release/*"), str(origin), True)
    ident = launch_policy.source_identity(work)
    assert ident["clean"] and ident["branch"] == "main" and ident["origin"]
    with pytest.raises(ConfigValidationError, match="pushed"):
        launch_policy.check(ident, rules)  # committed but origin does not have it
    _git(work, "push", "origin", "main")
    launch_policy.check(launch_policy.source_identity(work), rules)
    # origin: another one than expected (and a local path never passes for a remote of the same spelling)
    with pytest.raises(ConfigValidationError, match="expected_origin"):
        launch_policy.check(ident, launch_policy.LaunchRules("strict", ("main",), "github.com/someone/repo", False))
    assert launch_policy.normalize_origin("git@GitHub.com:Owner/Repo.git") == launch_policy.normalize_origin("https://user:pw@github.com/Owner/Repo/")
    assert launch_policy.normalize_origin("github.com/owner/repo", tmp_path)[0] == "local"
    # branch: not one of the allowed patterns; then detached
    _git(work, "checkout", "-b", "scratch")
    with pytest.raises(ConfigValidationError, match="allowed_branches"):
        launch_policy.check(launch_policy.source_identity(work), rules)
    _git(work, "checkout", "--detach")
    with pytest.raises(ConfigValidationError, match="detached"):
        launch_policy.check(launch_policy.source_identity(work), rules)
    # clean comes first: an untracked file refuses even on an allowed branch
    _git(work, "checkout", "main")
    (work / "stray.txt").write_text("x")
    with pytest.raises(ConfigValidationError, match="uncommitted"):
        launch_policy.check(launch_policy.source_identity(work), rules)
    launch_policy.check(launch_policy.source_identity(work), "record")  # 'record' applies no rule


def test_site_launch_table_is_parsed_fail_closed(tmp_path):
    path = tmp_path / "site.toml"
    text = ('[paths]\nrun_root = "/tmp/r"\n[launch]\npolicy = "strict"\nallowed_branches = ["main", "rel/*"]\n'
            'expected_origin = "github.com/o/r"\nrequire_pushed = true\n')
    path.write_text(text)
    path.chmod(0o600)
    site = SiteConfig.parse(path)
    rules = site.launch_rules
    assert rules.policy == "strict" and rules.allowed_branches == ("main", "rel/*") and rules.expected_origin == "github.com/o/r" and rules.require_pushed
    for bad in ('allowed_branches = []', 'allowed_branches = "main"', 'require_pushed = "yes"', 'expected_origin = "a b"'):
        key = bad.split(" =")[0]
        lines = [ln for ln in text.splitlines() if not ln.startswith(key)] + [bad]
        path.write_text("\n".join(lines) + "\n")
        with pytest.raises(ConfigValidationError):
            SiteConfig.parse(path)


def test_exchange_recorder_lists_what_a_launch_exchanges():
    from glm_tpu_b200.ops import native

    comm = native.PeerComm()
    comm.world = 8
    with native.record_exchanges() as plan:
        native._note_allreduce("skinny_bf16", comm, native.CH_ATTN, 768, 8)
        native._note_signal("step_finalize", comm, native.SIG_SAMPLE)
        native._note_allreduce("moe_combine", comm, native.CH_MLP, 384, 32)
        native._note_allreduce("single", None, native.CH_MLP, 1, 1)  # one GPU: nothing is exchanged, nothing is listed
    assert [op["kind"] for op in plan] == ["allreduce", "signal", "allreduce"] and native._exchanges is None
    admission.check_collective_plan(plan, world=8)
    with pytest.raises(PlanValidationError, match="same channel"):
        admission.check_collective_plan(plan + [dict(plan[2])], world=8)
    assert native._skinny_ksplit(3072, 2048) == 2 and native._skinny_ksplit(128, 6144) == 8 and native._skinny_ksplit(9680, 6144) == 1
    assert torch.tensor(1).item() == 1

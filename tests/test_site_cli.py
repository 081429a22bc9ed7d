"""Site file (fail-closed TOML), topology with a fake NVML, and the command line (argument snapshots, offline paths)."""

import json
import os
import subprocess
import sys
from pathlib import Path
from types import SimpleNamespace

import pytest

from tests.conftest import scaled

from glm_tpu_b200.config.site import SiteConfig
from glm_tpu_b200.entrypoints.cli import main as cli
from glm_tpu_b200.exceptions import ConfigValidationError
from glm_tpu_b200.executor import topology_job
from glm_tpu_b200.parallel import topology as topo

REPO = Path(__file__).resolve().parents[1]


def _site(tmp_path, text, mode=0o600):
    p = tmp_path / "site.toml"
    p.write_text(text)
    os.chmod(p, mode)
    return p


GOOD = '[box]\ngpus = 4\n[paths]\nrun_root = "/tmp/glm-runs"\npacked_path = "/data/packed"\n[checkpoint]\nmanifest_sha256 = "%s"\n[launch]\npolicy = "strict"\n' % ("a" * 64)


def test_site_parses_and_hashes(tmp_path):
    site = SiteConfig.parse(_site(tmp_path, GOOD))
    assert site.gpus == 4 and site.policy == "strict" and site.paths.packed_path == Path("/data/packed") and site.manifest_sha256 == "a" * 64
    again = SiteConfig.parse(_site(tmp_path, GOOD))
    assert site.sha256 == again.sha256 and json.loads(site.resolved_json())["paths"]["run_root"] == "/tmp/glm-runs"


@pytest.mark.parametrize("text,match", [
    (GOOD.replace("gpus = 4", "gpus = 3"), "gpus"),
    (GOOD + '[extra]\nx = 1\n', "unknown site tables"),
    (GOOD.replace('policy = "strict"', 'policy = "strict"\nsurprise = 1'), "unknown keys"),
    (GOOD.replace("a" * 64, "A" * 64), "64 lowercase hex"),
    (GOOD.replace("/tmp/glm-runs", "relative/runs"), "absolute plain"),
    (GOOD.replace("/tmp/glm-runs", "/tmp/../etc"), "absolute plain"),
    (GOOD.replace('policy = "strict"', 'policy = "yolo"'), "policy"),
    ('[box]\ngpus = 8\n', "run_root"),
    ("not toml [", "TOML"),
])
def test_site_is_fail_closed(tmp_path, text, match):
    with pytest.raises(ConfigValidationError, match=match):
        SiteConfig.parse(_site(tmp_path, text))


def test_site_permissions(tmp_path):
    with pytest.raises(ConfigValidationError, match="0600"):
        SiteConfig.parse(_site(tmp_path, GOOD, 0o644))
    link = tmp_path / "link.toml"
    link.symlink_to(_site(tmp_path, GOOD))
    with pytest.raises(ConfigValidationError, match="regular"):
        SiteConfig.parse(link)


def test_env_overrides_site(tmp_path, monkeypatch):
    monkeypatch.setenv("GLM_B200_RUN_ROOT", str(tmp_path / "elsewhere"))
    assert SiteConfig.load(_site(tmp_path, GOOD)).paths.run_root == tmp_path / "elsewhere"
    assert SiteConfig.load(tmp_path / "missing.toml").gpus == 8
    with pytest.raises(ConfigValidationError):
        SiteConfig.load(tmp_path / "missing.toml", required=True)


# ------------------------------------------------------------------------------------------------ topology
class FakeNvml:
    """The read-only NVML calls the discovery uses; records every call so that a test can prove nothing is set."""

    NVML_P2P_CAPS_INDEX_NVLINK = 2
    NVML_P2P_STATUS_OK = 0

    class NVMLError(Exception):
        pass

    def __init__(self, n=8, name="NVIDIA B200", cc=(10, 0), broken_pair=None, links=18):
        self.n, self.name, self.cc, self.broken, self.links, self.calls = n, name, cc, broken_pair, links, []

    def __getattr__(self, attr):
        if not attr.startswith("nvml"):
            raise AttributeError(attr)
        self.calls.append(attr)
        return getattr(self, "_" + attr)

    def _nvmlInit(self): pass
    def _nvmlShutdown(self): pass
    def _nvmlDeviceGetCount(self): return self.n
    def _nvmlDeviceGetHandleByIndex(self, i): return i
    def _nvmlDeviceGetUUID(self, h): return f"GPU-{h:08d}".encode()
    def _nvmlDeviceGetName(self, h): return self.name
    def _nvmlDeviceGetPciInfo(self, h): return SimpleNamespace(busId=f"00000000:{(7 - h) * 16 + 11:02X}:00.0")
    def _nvmlDeviceGetMemoryInfo(self, h): return SimpleNamespace(total=183359 << 20)
    def _nvmlDeviceGetCudaComputeCapability(self, h): return self.cc
    def _nvmlSystemGetDriverVersion(self): return "580.159"

    def _nvmlDeviceGetNvLinkState(self, h, link):
        if link >= self.links:
            raise self.NVMLError("no such link")
        return 1

    def _nvmlDeviceGetP2PStatus(self, a, b, caps):
        return 1 if self.broken in ((a, b), (b, a)) else 0


def test_topology_discovery_and_binding(tmp_path):
    nvml = FakeNvml()
    found = topo.discover_topology(nvml)
    assert len(found.devices) == 8 and found.devices[0].nvlink_active == 18 and all(all(r) for r in found.peer_nvlink)
    assert not [c for c in nvml.calls if "Set" in c or "Reset" in c or "Lock" in c]
    binding = topo.derive_topology_binding(found, 4)
    # ranks follow the PCI order (here the reverse of the NVML index), not the enumeration order
    assert [r["uuid"] for r in binding["ranks"]] == [f"GPU-{i:08d}" for i in (7, 6, 5, 4)]
    assert topo.visible_devices(binding).count(",") == 3
    topo.validate_live(binding, found)
    assert topo.Topology.from_dict(found.as_dict()).topology_hash == found.topology_hash


def test_topology_refusals():
    with pytest.raises(ConfigValidationError, match="not a B200"):
        topo.derive_topology_binding(topo.discover_topology(FakeNvml(name="NVIDIA H100", cc=(9, 0))), 8)
    with pytest.raises(ConfigValidationError, match="NVLink"):
        topo.derive_topology_binding(topo.discover_topology(FakeNvml(broken_pair=(0, 3))), 8)
    with pytest.raises(ConfigValidationError, match="needed"):
        topo.derive_topology_binding(topo.discover_topology(FakeNvml(n=2)), 4)
    with pytest.raises(ConfigValidationError, match="runs on"):
        topo.derive_topology_binding(topo.discover_topology(FakeNvml()), 3)


def test_topology_jobs_and_pins(tmp_path):
    nvml = FakeNvml()
    report = topology_job.capture_topology(tmp_path / "topology.json", nvml)
    assert report["gpus"] == 8
    bound = topology_job.bind_topology(tmp_path / "topology.json", 8, nvml=nvml)
    binding = topo.load_topology_binding(bound["output"], pin=bound["binding_sha256"])
    assert binding["gpus"] == 8
    with pytest.raises(ConfigValidationError, match="pinned"):
        topo.load_topology_binding(bound["output"], pin="0" * 64)
    # the live box changed: one GPU was swapped
    other = FakeNvml()
    other._nvmlDeviceGetUUID = lambda h: f"GPU-{h + 100:08d}"
    with pytest.raises(ConfigValidationError, match="not where"):
        topo.validate_live(binding, topo.discover_topology(other))
    raw = json.loads(Path(bound["output"]).read_text())
    raw["gpus"] = 4
    (tmp_path / "edited.json").write_text(json.dumps(raw))
    with pytest.raises(ConfigValidationError, match="own digest"):
        topo.load_topology_binding(tmp_path / "edited.json")
    with pytest.raises(FileExistsError):
        topology_job.capture_topology(tmp_path / "topology.json", nvml)


# ------------------------------------------------------------------------------------------------ command line
def test_cli_argument_snapshot():
    p = cli.build_parser()
    a = p.parse_args(["ask", "why?", "--context", "128k", "--keep-loaded", "--max-new-tokens", "7"])
    assert (a.question, a.context, a.keep_loaded, a.concurrent, a.max_new_tokens, a.wall_seconds) == ("why?", "128k", True, False, 7, 86400)
    a = p.parse_args(["checkpoint", "pack", "/s", "/t", "--gpus", "4"])
    assert (a.action, a.source, a.target, a.gpus) == ("pack", Path("/s"), Path("/t"), 4)
    a = p.parse_args(["topology", "bind", "/c.json"])
    assert (a.action, a.capture, a.gpus) == ("bind", Path("/c.json"), 8)
    for bad in (["ask"], ["ask", "q", "--questions", "/f"], ["ask", "q", "--context", "64k"], ["checkpoint"], ["nope"]):
        with pytest.raises(SystemExit):
            p.parse_args(bad)


def test_info_does_not_import_torch():
    code = "import sys; from glm_tpu_b200.entrypoints.cli.main import main; main(['info']); assert 'torch' not in sys.modules, 'torch imported'"
    done = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=REPO, timeout=scaled(120))
    assert done.returncode == 0, done.stderr
    assert json.loads(done.stdout)["decoding"].startswith("greedy")


def test_prepare_only_and_prepare_request(tmp_path, monkeypatch, capsys):
    monkeypatch.setenv("GLM_B200_RUN_ROOT", str(tmp_path / "runs"))
    monkeypatch.setenv("GLM_B200_SITE_CONFIG", str(tmp_path / "none.toml"))
    assert cli.main(["ask", "What is 2+2?", "--prepare-only", "--model", "random:tiny", "--capacity", "256", "--max-new-tokens", "4"]) == 0
    line = [ln for ln in capsys.readouterr().out.splitlines() if ln.startswith("PRIVATE_INPUT ")][0]
    request = json.loads(Path(line.split(" ", 1)[1]).read_text())
    assert request["max_new_tokens"] == 4 and request["context_capacity"] == 256
    assert oct(Path(line.split(" ", 1)[1]).stat().st_mode & 0o777) == "0o600"
    messages = tmp_path / "m.json"
    messages.write_text(json.dumps([{"role": "user", "content": "hi"}]))
    assert cli.main(["prepare-request", "--messages", str(messages), "--output", str(tmp_path / "p.json"), "--model", "random:tiny",
                     "--capacity", "256"]) == 0
    prepared = json.loads((tmp_path / "p.json").read_text())
    assert prepared["prompt_ids"] and len(prepared["request_sha256"]) == 64
    with pytest.raises(FileExistsError):
        cli.main(["prepare-request", "--messages", str(messages), "--output", str(tmp_path / "p.json"), "--model", "random:tiny", "--capacity", "256"])


def test_checkpoint_cli_round_trip(tmp_path, monkeypatch, capsys):
    from glm_tpu_b200.config.model import tiny_geometry
    from glm_tpu_b200.model_loader import export
    from glm_tpu_b200.models.glm_moe_dsa.weights import random_checkpoint

    monkeypatch.setenv("GLM_B200_RUN_ROOT", str(tmp_path / "runs"))
    monkeypatch.setenv("GLM_B200_SITE_CONFIG", str(tmp_path / "none.toml"))
    g = tiny_geometry()
    export.export_source(random_checkpoint(g, 5), g, tmp_path / "src")
    for argv in (["checkpoint", "inventory", str(tmp_path / "src")], ["checkpoint", "mark-source", str(tmp_path / "src")],
                 ["checkpoint", "pack", str(tmp_path / "src"), str(tmp_path / "packed"), "--gpus", "2"],
                 ["checkpoint", "verify", str(tmp_path / "packed")]):
        assert cli.main(argv) == 0
        assert json.loads(capsys.readouterr().out)["ok"]


def test_per_rank_topology_capture(tmp_path):
    """Two threads = two ranks with a rendezvous instead of the process group (no GPU, no torch.distributed)."""
    import threading

    from glm_tpu_b200.parallel import topology_capture as tc

    found = topo.discover_topology(FakeNvml(n=2))
    binding = topo.derive_topology_binding(found, 2)
    uuids = [r["uuid"] for r in binding["ranks"]]

    def run(assignment, bindings=(binding, binding)):
        box, barrier, errors = [None, None], threading.Barrier(2), [None, None]

        def gather_for(rank):
            def gather(obj):
                box[rank] = obj
                barrier.wait(timeout=10)
                return list(box)
            return gather

        def body(rank):
            try:
                out = tmp_path / f"case{len(list(tmp_path.iterdir()))}-{rank}"
                out.mkdir()
                tc.capture_rank(rank, bindings[rank], assignment[rank], gather_for(rank), out)
            except Exception as exc:  # noqa: BLE001
                errors[rank] = exc

        threads = [threading.Thread(target=body, args=(r,)) for r in range(2)]
        [t.start() for t in threads]
        [t.join() for t in threads]
        return errors

    assert run(uuids) == [None, None]
    swapped = run(uuids[::-1])
    assert all(isinstance(e, ConfigValidationError) and "binding gives it" in str(e) for e in swapped)
    doubled = run([uuids[0], uuids[0]])
    assert all(isinstance(e, ConfigValidationError) for e in doubled)
    other = dict(binding, binding_sha256="f" * 64)
    assert all(isinstance(e, ConfigValidationError) and "different topology bindings" in str(e) for e in run(uuids, (binding, other)))

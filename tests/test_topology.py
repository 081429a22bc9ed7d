"""GPU topology with a fake NVML: what discovery reads (and that it only reads), which boxes are refused and why, how ranks are
bound, and that captures and bindings are read fail-closed -- every way a file can be absent, foreign, edited or out of step with
the live box ends in ``ConfigValidationError``.

Reference counterparts: ``tests/distributed/test_topology.py``, ``tests/executor/test_topology_job.py``,
``tests/entrypoints/cli/test_topology.py``."""

import hashlib
import json
from types import SimpleNamespace

import pytest

from glm_tpu_b200.entrypoints.cli import main as cli
from glm_tpu_b200.exceptions import ConfigValidationError
from glm_tpu_b200.executor import topology_job
from glm_tpu_b200.parallel import topology as topo
from glm_tpu_b200.utils.json_utils import canonical_hash_bytes, canonical_wire_bytes


class Nvml:
    """Read-only NVML of a box described by the constructor; every call is recorded."""

    NVML_P2P_CAPS_INDEX_NVLINK, NVML_P2P_STATUS_OK = 2, 0

    class NVMLError(Exception):
        pass

    def __init__(self, n=8, name="NVIDIA B200", cc=(10, 0), links=18, broken=(), p2p_raises=(), uuids=None, bus=None, links_unsupported=False):
        self.n, self.name, self.cc, self.links, self.broken, self.p2p_raises = n, name, cc, links, set(broken), set(p2p_raises)
        self.uuids = uuids or [f"GPU-{i:08d}" for i in range(n)]
        self.bus = bus or [f"00000000:{(n - i) * 16 + 11:02X}:00.0" for i in range(n)]  # PCI order is the reverse of the index order
        self.links_unsupported, self.calls, self.open = links_unsupported, [], 0

    def nvmlInit(self): self.calls.append("nvmlInit"); self.open += 1
    def nvmlShutdown(self): self.calls.append("nvmlShutdown"); self.open -= 1
    def nvmlDeviceGetCount(self): self.calls.append("nvmlDeviceGetCount"); return self.n
    def nvmlDeviceGetHandleByIndex(self, i): return i
    def nvmlDeviceGetUUID(self, h): return self.uuids[h].encode()
    def nvmlDeviceGetName(self, h): return self.name if isinstance(self.name, str) else self.name[h]
    def nvmlDeviceGetPciInfo(self, h): return SimpleNamespace(busId=self.bus[h].encode())
    def nvmlDeviceGetMemoryInfo(self, h): return SimpleNamespace(total=183359 << 20)
    def nvmlDeviceGetCudaComputeCapability(self, h): return self.cc
    def nvmlSystemGetDriverVersion(self): return b"580.159"

    def nvmlDeviceGetNvLinkState(self, h, link):
        if self.links_unsupported or link >= self.links:
            raise self.NVMLError("not supported")
        return 1

    def nvmlDeviceGetP2PStatus(self, a, b, caps):
        assert caps == self.NVML_P2P_CAPS_INDEX_NVLINK
        if (a, b) in self.p2p_raises:
            raise self.NVMLError("unknown error")
        return 1 if (a, b) in self.broken or (b, a) in self.broken else 0


def reseal(binding: dict) -> dict:
    body = {k: v for k, v in binding.items() if k != "binding_sha256"}
    return dict(body, binding_sha256=hashlib.sha256(canonical_hash_bytes(body)).hexdigest())


# ------------------------------------------------------------------------------------------------ discovery
def test_discovery_reads_and_only_reads():
    nvml = Nvml()
    found = topo.discover_topology(nvml)
    assert nvml.open == 0 and nvml.calls[0] == "nvmlInit" and nvml.calls[-1] == "nvmlShutdown"  # closed again, whatever happened in between
    assert [d.index for d in found.devices] == list(range(8)) and found.driver == "580.159"
    first = found.devices[0]
    assert (first.uuid, first.name, first.memory_mib, first.compute_capability, first.nvlink_active) == ("GPU-00000000", "NVIDIA B200", 183359, (10, 0), 18)
    assert all(found.peer_nvlink[i][i] for i in range(8)) and all(all(row) for row in found.peer_nvlink)
    assert not [name for name in dir(Nvml) if any(word in name for word in ("Set", "Reset", "Lock", "Clear"))]  # the fake offers nothing that writes
    again = topo.discover_topology(Nvml())
    assert again.topology_hash == found.topology_hash and topo.Topology.from_dict(found.as_dict()).topology_hash == found.topology_hash
    assert topo.discover_topology(Nvml(links=12)).topology_hash != found.topology_hash  # six links down is another topology


def test_discovery_survives_what_a_driver_does_not_report():
    quiet = topo.discover_topology(Nvml(links_unsupported=True))
    assert all(d.nvlink_active == 0 for d in quiet.devices)  # no link state: counted as none, the peer table decides
    partial = topo.discover_topology(Nvml(p2p_raises={(0, 1)}))
    assert partial.peer_nvlink[0][1] is False and partial.peer_nvlink[1][0] is True  # a query that fails is "no path", not a crash

    class Failing(Nvml):
        def nvmlDeviceGetCount(self):
            raise self.NVMLError("driver not loaded")

    nvml = Failing()
    with pytest.raises(Nvml.NVMLError):
        topo.discover_topology(nvml)
    assert nvml.open == 0  # shut down on the way out


# ------------------------------------------------------------------------------------------------ which boxes
@pytest.mark.parametrize("nvml,gpus,match", [
    (Nvml(), 3, "runs on"), (Nvml(), 16, "runs on"), (Nvml(n=2), 4, "the box has 2 GPUs, 4 are needed"),
    (Nvml(name="NVIDIA H100 80GB HBM3", cc=(9, 0)), 8, "is not a B200"), (Nvml(cc=(9, 0)), 8, "is not a B200"),
    (Nvml(name="NVIDIA B100"), 1, "is not a B200"),
    (Nvml(broken={(0, 3)}), 8, "no NVLink peer path from GPU"), (Nvml(p2p_raises={(7, 6)}), 8, "no NVLink peer path from GPU 7 to GPU 6"),
    (Nvml(uuids=["GPU-same"] * 8), 8, "same UUID"),
])
def test_boxes_that_are_refused(nvml, gpus, match):
    with pytest.raises(ConfigValidationError, match=match):
        topo.derive_topology_binding(topo.discover_topology(nvml), gpus)


def test_a_fault_outside_the_chosen_gpus_does_not_matter():
    found = topo.discover_topology(Nvml(broken={(0, 1)}))  # indices 0 and 1 have the highest bus ids: not among the first four by PCI order
    binding = topo.derive_topology_binding(found, 4)
    assert [r["uuid"] for r in binding["ranks"]] == ["GPU-00000007", "GPU-00000006", "GPU-00000005", "GPU-00000004"]
    with pytest.raises(ConfigValidationError, match="no NVLink peer path"):
        topo.derive_topology_binding(found, 8)


@pytest.mark.parametrize("gpus", topo.SUPPORTED_GPUS)
def test_ranks_follow_the_pci_order(gpus):
    found = topo.discover_topology(Nvml())
    binding = topo.derive_topology_binding(found, gpus)
    assert [r["rank"] for r in binding["ranks"]] == list(range(gpus)) and binding["gpus"] == gpus
    assert [r["pci_bus_id"] for r in binding["ranks"]] == sorted(d.pci_bus_id for d in found.devices)[:gpus]
    assert topo.visible_devices(binding) == ",".join(f"GPU-{7 - r:08d}" for r in range(gpus))  # UUIDs, in rank order
    assert binding["topology_sha256"] == found.topology_hash and binding == reseal(binding)
    assert topo.derive_topology_binding(found, gpus) == binding  # the same box gives the same binding


# ------------------------------------------------------------------------------------------------ stored bindings
@pytest.fixture
def stored(tmp_path):
    found = topo.discover_topology(Nvml())
    binding = topo.derive_topology_binding(found, 4)
    path = tmp_path / "binding.json"
    path.write_bytes(canonical_wire_bytes(binding))
    return path, binding, found


def test_a_stored_binding_reads_back_and_is_pinned(stored):
    path, binding, found = stored
    assert topo.load_topology_binding(path) == binding and topo.load_topology_binding(path, pin=binding["binding_sha256"]) == binding
    with pytest.raises(ConfigValidationError, match="not the pinned one"):
        topo.load_topology_binding(path, pin="0" * 64)
    topo.validate_live(binding, found)


def test_bindings_are_read_fail_closed(stored, tmp_path):
    path, binding, _ = stored
    with pytest.raises(ConfigValidationError, match="does not exist"):
        topo.load_topology_binding(tmp_path / "absent.json")
    for content, match in ((b"", "cannot be read as JSON"), (b"{oops", "cannot be read as JSON"), (b"\xff\xfe", "cannot be read as JSON"),
                           (b"[]", "not a topology binding"), (b"{}", "not a topology binding"),
                           (canonical_wire_bytes(reseal(dict(binding, schema="other"))), "not a topology binding"),
                           (canonical_wire_bytes(reseal(dict(binding, note="extra"))), "not a topology binding"),
                           (canonical_wire_bytes({k: v for k, v in binding.items() if k != "driver"}), "not a topology binding")):
        path.write_bytes(content)
        with pytest.raises(ConfigValidationError, match=match):
            topo.load_topology_binding(path)
    for edit in ({"gpus": 2}, {"driver": "999"}, {"ranks": binding["ranks"][:3]}, {"topology_sha256": "0" * 64}):
        path.write_bytes(canonical_wire_bytes(dict(binding, **edit)))  # edited without recomputing the digest
        with pytest.raises(ConfigValidationError, match="own digest"):
            topo.load_topology_binding(path)
    ranks = binding["ranks"]
    for edit, match in (({"gpus": 3, "ranks": ranks[:3]}, "one GPU per rank of a supported box"), ({"ranks": ranks[:3]}, "one GPU per rank"),
                        ({"ranks": "all"}, "one GPU per rank"), ({"ranks": [dict(ranks[0], extra=1)] + ranks[1:]}, "rank entry of the binding is malformed"),
                        ({"ranks": [dict(ranks[0], uuid="")] + ranks[1:]}, "malformed"), ({"ranks": [dict(ranks[0], memory_mib="big")] + ranks[1:]}, "malformed"),
                        ({"ranks": [ranks[1], ranks[0]] + ranks[2:]}, "ranks are not 0..gpus-1"),
                        ({"ranks": [ranks[0], dict(ranks[1], uuid=ranks[0]["uuid"])] + ranks[2:]}, "one GPU for two ranks"),
                        ({"ranks": [ranks[0], dict(ranks[1], pci_bus_id=ranks[0]["pci_bus_id"])] + ranks[2:]}, "one GPU for two ranks")):
        path.write_bytes(canonical_wire_bytes(reseal(dict(binding, **edit))))  # self-consistent, but not a binding the engine could have written
        with pytest.raises(ConfigValidationError, match=match):
            topo.load_topology_binding(path)


def test_a_binding_is_checked_against_the_live_box(stored):
    _, binding, found = stored
    topo.validate_live(binding, topo.discover_topology(Nvml(links=12)))  # fewer links, same devices and paths: still this box
    swapped = Nvml(uuids=[f"GPU-{i + 100:08d}" for i in range(8)])
    with pytest.raises(ConfigValidationError, match="rank 0: GPU GPU-00000007 is not where the binding says"):
        topo.validate_live(binding, topo.discover_topology(swapped))
    moved = Nvml(bus=[f"00000000:{i * 16 + 11:02X}:00.0" for i in range(8)])  # same UUIDs in other slots
    with pytest.raises(ConfigValidationError, match="not where the binding says"):
        topo.validate_live(binding, topo.discover_topology(moved))
    with pytest.raises(ConfigValidationError, match="lost its NVLink path"):
        topo.validate_live(binding, topo.discover_topology(Nvml(broken={(7, 5)})))
    topo.validate_live(binding, topo.discover_topology(Nvml(broken={(0, 1)})))  # a fault between GPUs the binding does not use
    with pytest.raises(ConfigValidationError, match="not where"):
        topo.validate_live(binding, topo.discover_topology(Nvml(n=2)))  # the bound GPUs are gone


# ------------------------------------------------------------------------------------------------ captures and the job
def test_capture_and_bind_files(tmp_path):
    nvml = Nvml()
    report = topology_job.capture_topology(tmp_path / "capture.json", nvml)
    assert report["ok"] and report["gpus"] == 8 and report["names"] == ["NVIDIA B200"] and (tmp_path / "capture.json").stat().st_mode & 0o077 == 0
    with pytest.raises(FileExistsError):
        topology_job.capture_topology(tmp_path / "capture.json", nvml)  # create-once
    bound = topology_job.bind_topology(tmp_path / "capture.json", 8, nvml=nvml)
    assert bound["output"] == str(tmp_path / "topology_binding.json") and bound["visible_devices"].count(",") == 7
    assert topo.load_topology_binding(bound["output"], pin=bound["binding_sha256"])["gpus"] == 8
    with pytest.raises(FileExistsError):
        topology_job.bind_topology(tmp_path / "capture.json", 8, nvml=nvml)
    four = topology_job.bind_topology(tmp_path / "capture.json", 4, output=tmp_path / "four.json", nvml=nvml)
    assert four["binding_sha256"] != bound["binding_sha256"]
    with pytest.raises(ConfigValidationError, match="not where"):  # the capture is of another box than the live one
        topology_job.bind_topology(tmp_path / "capture.json", 2, output=tmp_path / "two.json", nvml=Nvml(uuids=[f"GPU-x{i}" for i in range(8)]))
    assert not (tmp_path / "two.json").exists()
    assert topology_job.bind_topology(tmp_path / "capture.json", 2, output=tmp_path / "two.json", check_live=False)["gpus"] == 2  # binding on a machine without the GPUs


def test_captures_are_read_fail_closed(tmp_path):
    topology_job.capture_topology(tmp_path / "capture.json", Nvml())
    raw = json.loads((tmp_path / "capture.json").read_text())
    bad = tmp_path / "bad.json"
    with pytest.raises(ConfigValidationError, match="does not exist"):
        topology_job.bind_topology(tmp_path / "absent.json", 8, check_live=False)
    for content, match in (("{oops", "cannot be read as JSON"), ("[]", "not a topology capture"), (json.dumps(dict(raw, schema="other")), "not a topology capture"),
                           (json.dumps(dict(raw, driver="999")), "own digest"), (json.dumps({k: v for k, v in raw.items() if k != "topology_sha256"}), "own digest"),
                           (json.dumps({k: v for k, v in raw.items() if k != "devices"}), "malformed"),
                           (json.dumps(dict(raw, devices=[dict(raw["devices"][0], color="green")] + raw["devices"][1:])), "malformed"),
                           (json.dumps(dict(raw, peer_nvlink=raw["peer_nvlink"][:7])), "peer table does not match"),
                           (json.dumps(dict(raw, devices=list(reversed(raw["devices"])))), "peer table does not match")):
        bad.write_text(content)
        with pytest.raises(ConfigValidationError, match=match):
            topology_job.bind_topology(bad, 8, output=tmp_path / "never.json", check_live=False)
    assert not (tmp_path / "never.json").exists()


def test_the_command_line_refuses_in_one_json_line(tmp_path, capsys):
    (tmp_path / "capture.json").write_text("{oops")
    code = cli.main(["topology", "bind", str(tmp_path / "capture.json"), "--gpus", "8"])
    out = capsys.readouterr()
    assert code == 2 and out.out == "" and json.loads(out.err)["refused"] == "ConfigValidationError" and "cannot be read as JSON" in json.loads(out.err)["message"]

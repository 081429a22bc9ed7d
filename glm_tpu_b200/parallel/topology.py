"""GPU topology of one box: discovery (NVML), validation, and the rank -> GPU binding.

The engine runs on 1, 2, 4 or 8 B200 GPUs of one NVLink/NVSwitch box.  Which physical GPU a rank uses matters twice:
the in-kernel collectives need peer access between every pair, and a run must be reproducible on the *same* devices.

* ``discover_topology(nvml)`` reads, read-only, every GPU's UUID, PCI bus id, name, memory, compute capability, active
  NVLink links, and the pairwise NVLink peer status.  ``nvml`` is the ``pynvml`` module or a fake with the same calls.
  Nothing is ever *set* through NVML.
* ``require_b200_box(topology, gpus)`` refuses a box that is not ``gpus`` x B200 (sm_100) with all-to-all NVLink access.
* ``derive_topology_binding(topology, gpus)`` orders the GPUs by PCI bus id, assigns ranks, and hashes the result;
  the digest is what a site file pins.  ``validate_live(binding, topology)`` authenticates a stored binding against the
  live devices (same UUIDs at the same bus ids), ``visible_devices(binding)`` is the ``CUDA_VISIBLE_DEVICES`` value
  (UUIDs in rank order) that makes ``cuda:<local_rank>`` the bound GPU in every worker.

Parity: reference ``glm_tpu/distributed/topology.py:49-143`` (validate fleet), ``:161-234`` (load/apply binding),
``:242-387`` (discover, require the supported shape, derive binding), ``:399-515`` (device/topology records + hashes).
"""

from __future__ import annotations

import hashlib
import json
from dataclasses import asdict, dataclass
from pathlib import Path

from glm_tpu_b200.exceptions import ConfigValidationError
from glm_tpu_b200.utils.json_utils import canonical_hash_bytes

SUPPORTED_GPUS = (1, 2, 4, 8)
MAX_NVLINKS = 18
BINDING_SCHEMA = "glm_b200_topology_binding_v1"
CAPTURE_SCHEMA = "glm_b200_topology_capture_v1"


@dataclass(frozen=True)
class GpuDevice:
    index: int
    uuid: str
    name: str
    pci_bus_id: str
    memory_mib: int
    compute_capability: tuple
    nvlink_active: int  # active NVLink links; -1 when the driver does not report them


@dataclass(frozen=True)
class Topology:
    devices: tuple
    peer_nvlink: tuple  # [n][n] bool: NVLink peer path from i to j (diagonal True)
    driver: str

    def as_dict(self) -> dict:
        return {"schema": CAPTURE_SCHEMA, "driver": self.driver,
                "devices": [dict(asdict(d), compute_capability=list(d.compute_capability)) for d in self.devices],
                "peer_nvlink": [list(row) for row in self.peer_nvlink]}

    @property
    def topology_hash(self) -> str:
        return hashlib.sha256(canonical_hash_bytes(self.as_dict())).hexdigest()

    @classmethod
    def from_dict(cls, raw: dict) -> "Topology":
        if not isinstance(raw, dict) or raw.get("schema") != CAPTURE_SCHEMA:
            raise ConfigValidationError("not a topology capture")
        try:
            devices = tuple(GpuDevice(**dict(d, compute_capability=tuple(d["compute_capability"]))) for d in raw["devices"])
            peers = tuple(tuple(bool(x) for x in row) for row in raw["peer_nvlink"])
            driver = raw["driver"]
        except (KeyError, TypeError) as exc:
            raise ConfigValidationError(f"the topology capture is malformed: {exc}") from None
        if len(peers) != len(devices) or any(len(row) != len(devices) for row in peers) or [d.index for d in devices] != list(range(len(devices))):
            raise ConfigValidationError("the topology capture is malformed: the peer table does not match the device list")
        return cls(devices, peers, driver)


def _text(value) -> str:
    return value.decode() if isinstance(value, bytes) else str(value)


def discover_topology(nvml=None) -> Topology:
    if nvml is None:
        import pynvml as nvml
    nvml.nvmlInit()
    try:
        count = nvml.nvmlDeviceGetCount()
        handles = [nvml.nvmlDeviceGetHandleByIndex(i) for i in range(count)]
        error = getattr(nvml, "NVMLError", Exception)
        devices = []
        for i, h in enumerate(handles):
            try:
                active = 0
                for link in range(MAX_NVLINKS):
                    try:
                        active += 1 if nvml.nvmlDeviceGetNvLinkState(h, link) else 0
                    except error:
                        break
            except error:
                active = -1
            major, minor = nvml.nvmlDeviceGetCudaComputeCapability(h)
            devices.append(GpuDevice(i, _text(nvml.nvmlDeviceGetUUID(h)), _text(nvml.nvmlDeviceGetName(h)),
                                     _text(nvml.nvmlDeviceGetPciInfo(h).busId), int(nvml.nvmlDeviceGetMemoryInfo(h).total) >> 20,
                                     (int(major), int(minor)), active))
        caps = getattr(nvml, "NVML_P2P_CAPS_INDEX_NVLINK", 2)
        ok = getattr(nvml, "NVML_P2P_STATUS_OK", 0)
        peer = []
        for i, a in enumerate(handles):
            row = []
            for j, b in enumerate(handles):
                if i == j:
                    row.append(True)
                    continue
                try:
                    row.append(nvml.nvmlDeviceGetP2PStatus(a, b, caps) == ok)
                except error:
                    row.append(False)
            peer.append(tuple(row))
        return Topology(tuple(devices), tuple(peer), _text(nvml.nvmlSystemGetDriverVersion()))
    finally:
        nvml.nvmlShutdown()


def require_b200_box(topology: Topology, gpus: int) -> list[GpuDevice]:
    """The ``gpus`` devices (lowest PCI bus ids) the engine would use, after checking that the box supports them."""
    if gpus not in SUPPORTED_GPUS:
        raise ConfigValidationError(f"the engine runs on {SUPPORTED_GPUS} GPUs, not {gpus}")
    if len(topology.devices) < gpus:
        raise ConfigValidationError(f"the box has {len(topology.devices)} GPUs, {gpus} are needed")
    chosen = sorted(topology.devices, key=lambda d: d.pci_bus_id)[:gpus]
    if len({d.uuid for d in chosen}) != gpus:
        raise ConfigValidationError("two GPUs report the same UUID")
    for d in chosen:
        if d.compute_capability != (10, 0) or "B200" not in d.name:
            raise ConfigValidationError(f"GPU {d.index} ({d.name}, sm_{d.compute_capability[0]}{d.compute_capability[1]}) is not a B200")
    for a in chosen:
        for b in chosen:
            if not topology.peer_nvlink[a.index][b.index]:
                raise ConfigValidationError(f"no NVLink peer path from GPU {a.index} to GPU {b.index}")
    return chosen


def derive_topology_binding(topology: Topology, gpus: int) -> dict:
    chosen = require_b200_box(topology, gpus)
    body = {"schema": BINDING_SCHEMA, "gpus": gpus, "driver": topology.driver, "topology_sha256": topology.topology_hash,
            "ranks": [{"rank": r, "uuid": d.uuid, "pci_bus_id": d.pci_bus_id, "memory_mib": d.memory_mib} for r, d in enumerate(chosen)]}
    return dict(body, binding_sha256=hashlib.sha256(canonical_hash_bytes(body)).hexdigest())


BINDING_KEYS = ("schema", "gpus", "driver", "topology_sha256", "ranks", "binding_sha256")
RANK_KEYS = ("rank", "uuid", "pci_bus_id", "memory_mib")


def load_topology_binding(path: Path, pin: str = "") -> dict:
    """The binding in ``path`` after checking that it is one: readable JSON with exactly the fields of a binding, hashing to its
    own digest (and to ``pin`` when one is given), for a supported GPU count, with one well-formed entry per rank and no GPU twice."""
    try:
        binding = json.loads(Path(path).read_text())
    except FileNotFoundError:
        raise ConfigValidationError(f"the topology binding {path} does not exist") from None
    except (OSError, UnicodeDecodeError, ValueError) as exc:
        raise ConfigValidationError(f"the topology binding cannot be read as JSON: {exc}") from None
    if not isinstance(binding, dict) or sorted(binding) != sorted(BINDING_KEYS) or binding["schema"] != BINDING_SCHEMA:
        raise ConfigValidationError("not a topology binding")
    body = {k: v for k, v in binding.items() if k != "binding_sha256"}
    if binding["binding_sha256"] != hashlib.sha256(canonical_hash_bytes(body)).hexdigest():
        raise ConfigValidationError("the topology binding does not match its own digest")
    if pin and binding["binding_sha256"] != pin:
        raise ConfigValidationError("the topology binding is not the pinned one")
    ranks = binding["ranks"]
    if binding["gpus"] not in SUPPORTED_GPUS or type(ranks) is not list or len(ranks) != binding["gpus"]:
        raise ConfigValidationError("the binding does not name one GPU per rank of a supported box")
    for entry in ranks:
        if (type(entry) is not dict or sorted(entry) != sorted(RANK_KEYS) or type(entry["uuid"]) is not str or not entry["uuid"]
                or type(entry["pci_bus_id"]) is not str or type(entry["memory_mib"]) is not int):
            raise ConfigValidationError("a rank entry of the binding is malformed")
    if [r["rank"] for r in ranks] != list(range(binding["gpus"])):
        raise ConfigValidationError("the binding's ranks are not 0..gpus-1")
    if len({r["uuid"] for r in ranks}) != len(ranks) or len({r["pci_bus_id"] for r in ranks}) != len(ranks):
        raise ConfigValidationError("the binding names one GPU for two ranks")
    return binding


def validate_live(binding: dict, topology: Topology) -> None:
    """Every bound GPU must be present with the same UUID at the same bus id, and still reach its peers."""
    by_uuid = {d.uuid: d for d in topology.devices}
    bound = []
    for entry in binding["ranks"]:
        d = by_uuid.get(entry["uuid"])
        if d is None or d.pci_bus_id != entry["pci_bus_id"]:
            raise ConfigValidationError(f"rank {entry['rank']}: GPU {entry['uuid']} is not where the binding says")
        bound.append(d)
    for a in bound:
        for b in bound:
            if not topology.peer_nvlink[a.index][b.index]:
                raise ConfigValidationError(f"GPU {a.index} lost its NVLink path to GPU {b.index}")


def visible_devices(binding: dict) -> str:
    return ",".join(entry["uuid"] for entry in binding["ranks"])

"""Topology jobs: capture the box's GPUs to a file, derive a binding from a capture.

``capture_topology`` is model-free and read-only (NVML queries); it writes ``topology.json`` create-once.
``bind_topology`` validates the capture for the requested GPU count, re-discovers the live box when NVML is present
(the capture must still describe it), and writes ``topology_binding.json``; the printed ``binding_sha256`` is what goes
into the site file's ``[topology]`` table.

Parity: reference ``glm_tpu/executor/topology_job.py`` (``capture_topology`` / ``bind_topology``).
"""

from __future__ import annotations

import json
from pathlib import Path

from glm_tpu_b200.exceptions import ConfigValidationError
from glm_tpu_b200.parallel import topology as topo
from glm_tpu_b200.utils.io_utils import create_private_exclusive
from glm_tpu_b200.utils.json_utils import canonical_wire_bytes


def capture_topology(output: Path, nvml=None) -> dict:
    found = topo.discover_topology(nvml)
    record = dict(found.as_dict(), topology_sha256=found.topology_hash)
    create_private_exclusive(Path(output), canonical_wire_bytes(record) + b"\n")
    return {"ok": True, "output": str(output), "gpus": len(found.devices), "topology_sha256": found.topology_hash,
            "names": sorted({d.name for d in found.devices})}


def bind_topology(capture: Path, gpus: int, output: Path | None = None, nvml=None, check_live: bool = True) -> dict:
    try:
        raw = json.loads(Path(capture).read_text())
    except FileNotFoundError:
        raise ConfigValidationError(f"the topology capture {capture} does not exist") from None
    except (OSError, UnicodeDecodeError, ValueError) as exc:
        raise ConfigValidationError(f"the topology capture cannot be read as JSON: {exc}") from None
    if not isinstance(raw, dict):
        raise ConfigValidationError("not a topology capture")
    claimed = raw.pop("topology_sha256", None)
    captured = topo.Topology.from_dict(raw)
    if claimed != captured.topology_hash:
        raise ConfigValidationError("the capture does not match its own digest")
    binding = topo.derive_topology_binding(captured, gpus)
    if check_live:
        try:
            live = topo.discover_topology(nvml)
        except ImportError:
            live = None
        if live is not None:
            topo.validate_live(binding, live)
    output = Path(output) if output is not None else Path(capture).with_name("topology_binding.json")
    create_private_exclusive(output, canonical_wire_bytes(binding) + b"\n")
    return {"ok": True, "output": str(output), "gpus": gpus, "binding_sha256": binding["binding_sha256"],
            "visible_devices": topo.visible_devices(binding)}

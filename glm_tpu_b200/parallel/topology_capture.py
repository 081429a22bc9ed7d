"""Per-rank topology check, run by every worker before it loads anything (model-free).

Each rank reports the UUID of the GPU it actually got (``cuda:<local_rank>`` under the ``CUDA_VISIBLE_DEVICES`` the controller
derived from the binding) together with the binding digest it was started with; the reports are all-gathered on the host, every rank
checks that (a) all ranks hold the same binding, (b) rank r sits on the GPU the binding gives to rank r, (c) no GPU is used twice, and
writes ``topology.rank<r>.json`` create-once.  Any mismatch raises on every rank at the same point.

    python -m glm_tpu_b200.parallel.topology_capture --binding topology_binding.json --out-dir RUN   (under torch.distributed.run)

Parity: reference ``glm_tpu/distributed/topology_capture.py:46-192`` (join runtime, all-gather device ids + contract digest, write
``topology.rank<r>.json``), ``parallel_state.py:23-78`` (authenticate the captures against the live devices).
"""

from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path

from glm_tpu_b200.exceptions import ConfigValidationError
from glm_tpu_b200.parallel import topology as topo
from glm_tpu_b200.utils.io_utils import create_private_exclusive
from glm_tpu_b200.utils.json_utils import canonical_wire_bytes


def local_gpu_uuid(local_rank: int) -> str:
    import torch

    return "GPU-" + str(torch.cuda.get_device_properties(local_rank).uuid)


def check_reports(binding: dict, reports: list[dict]) -> None:
    """``reports[r] = {"rank", "uuid", "binding_sha256"}`` as gathered from every rank."""
    if len(reports) != binding["gpus"]:
        raise ConfigValidationError(f"{len(reports)} ranks reported, the binding is for {binding['gpus']} GPUs")
    if {r["binding_sha256"] for r in reports} != {binding["binding_sha256"]}:
        raise ConfigValidationError("the ranks were started with different topology bindings")
    seen = set()
    for entry, report in zip(binding["ranks"], sorted(reports, key=lambda r: r["rank"])):
        if report["rank"] != entry["rank"] or report["uuid"] != entry["uuid"]:
            raise ConfigValidationError(f"rank {entry['rank']} runs on {report['uuid']}, the binding gives it {entry['uuid']}")
        if report["uuid"] in seen:
            raise ConfigValidationError(f"GPU {report['uuid']} is used by two ranks")
        seen.add(report["uuid"])


def capture_rank(rank: int, binding: dict, uuid: str, gather, out_dir: Path) -> dict:
    """``gather(obj) -> list`` is the host all-gather (``torch.distributed.all_gather_object`` or a test rendezvous)."""
    mine = {"rank": rank, "uuid": uuid, "binding_sha256": binding["binding_sha256"]}
    reports = gather(mine)
    check_reports(binding, reports)
    record = {"schema": "glm_b200_topology_rank_v1", **mine, "world": binding["gpus"], "peers": sorted(r["uuid"] for r in reports)}
    create_private_exclusive(Path(out_dir) / f"topology.rank{rank}.json", canonical_wire_bytes(record) + b"\n")
    return record


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="topology_capture")
    ap.add_argument("--binding", type=Path, required=True)
    ap.add_argument("--pin", default="")
    ap.add_argument("--out-dir", type=Path, required=True)
    args = ap.parse_args(argv)
    import torch.distributed as dist

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    binding = topo.load_topology_binding(args.binding, args.pin)
    dist.init_process_group("gloo")

    def gather(obj):
        out = [None] * world
        dist.all_gather_object(out, obj)
        return out

    try:
        capture_rank(rank, binding, local_gpu_uuid(int(os.environ.get("LOCAL_RANK", str(rank)))), gather, args.out_dir)
    finally:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())

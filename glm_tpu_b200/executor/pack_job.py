"""The pack job: inventory -> marker check -> workers -> receipts -> manifest -> seal -> verify.

The controller holds the workload lease, pins the source inventory digest, distributes the files of the packed
checkpoint (``shared`` + one expert file per GPU rank) over ``jobs`` worker processes, waits for every receipt, assembles
the manifest from the receipts only, installs geometry + manifest + ``SUCCESS`` create-once and finally re-verifies the
sealed directory from disk.  A failing worker fails the job; nothing is sealed and the partial target stays unusable.

Parity: reference ``glm_tpu/executor/pack_job.py:38-145``.
"""

from __future__ import annotations

import json
import subprocess
import sys
import time
from pathlib import Path

from glm_tpu_b200.exceptions import CheckpointValidationError
from glm_tpu_b200.executor.jobs import workload_lease
from glm_tpu_b200.model_loader import pack_worker, placement, source_inventory, source_marker
from glm_tpu_b200.model_loader.sharded_state import manifest as manifest_mod
from glm_tpu_b200.model_loader.sharded_state import seal, verify


def planned_bytes(geometry, world: int, expert_split: str) -> dict:
    """Size of every file of the packed checkpoint, from the shapes alone (header + payload)."""
    from glm_tpu_b200.model_loader.sharded_state import format as fmt
    from glm_tpu_b200.model_loader.sharded_state import writer

    sizes = {}
    for name, rank in [(fmt.SHARED_FILE, None)] + [(fmt.expert_file(r, world), r) for r in range(world)]:
        meta = writer.file_metadata(geometry, world, "shared" if rank is None else "experts", rank, expert_split)  # the header the packer will write
        head, _, payload = fmt.layout(placement.packed_tensor_shapes(geometry, world, rank, expert_split), meta)
        sizes[name] = len(head) + payload
    return sizes


def _free_bytes(target: Path) -> int:
    import shutil

    where = Path(target)
    while not where.exists():
        where = where.parent
    return shutil.disk_usage(where).free


def pack_checkpoint(source: Path, target: Path, world: int, *, run_root: Path | None = None, layers: int = 0, jobs: int = 0,
                    require_marker: bool = True, timeout: float = 24 * 3600.0, expert_split: str = "auto", pins: dict | None = None,
                    preflight_only: bool = False, free_bytes=None) -> dict:
    source, target = Path(source), Path(target)
    if (target / "SUCCESS").exists():
        raise CheckpointValidationError(f"{target} is already a sealed checkpoint")
    pinned = (pins or {}).get("source_marker_sha256", "")
    if pinned and not require_marker:
        raise CheckpointValidationError("a pinned source marker cannot be waived")
    marker = source_marker.require_marker(source, pinned) if require_marker else None
    inv = source_inventory.read_source_inventory(source)
    geometry = pack_worker.source_geometry(source, layers)
    if expert_split == "auto":  # the split the runner would choose for this geometry on this many GPUs
        from glm_tpu_b200.config.parallel import default_expert_split

        expert_split = default_expert_split(geometry, world)
    plan = planned_bytes(geometry, world, expert_split)
    needed = sum(plan.values())
    free = (free_bytes or _free_bytes)(target)
    if free < needed:
        raise CheckpointValidationError(f"the packed checkpoint needs {needed:,} bytes, {free:,} are free where {target} would be written")
    missing = [n for n in placement.expected_sources(geometry) if n not in inv.tensors]
    if missing:
        raise CheckpointValidationError(f"the source lacks {len(missing)} tensors, e.g. {missing[:3]}")
    if preflight_only:  # every check a pack makes before it writes, and nothing written
        return {"ok": True, "preflight_only": True, "target": str(target), "world": world, "expert_split": expert_split, "files": sorted(plan),
                "planned_bytes": plan, "total_bytes": needed, "free_bytes": free, "geometry_sha256": geometry.geometry_hash,
                "source_inventory_sha256": inv.sha256, "source_marker": bool(marker),
                "source_marker_sha256": source_marker.marker_sha256(source) if marker else ""}
    target.mkdir(parents=True, exist_ok=True, mode=0o700)
    files = ["shared"] + [str(r) for r in range(world)]
    jobs = max(1, min(jobs or len(files), len(files)))
    receipts_dir = target / "receipts"
    receipts_dir.mkdir(exist_ok=True)
    started = time.time()

    def body() -> dict:
        if jobs == 1:
            receipts = [pack_worker.run(source, target, world, files, inv.sha256, layers, expert_split)]
        else:
            procs = []
            for j in range(jobs):
                mine = files[j::jobs]
                receipt = receipts_dir / f"receipt.{j}.json"
                argv = [sys.executable, "-m", "glm_tpu_b200.model_loader.pack_worker", "--source", str(source), "--target", str(target),
                        "--world", str(world), "--files", ",".join(mine), "--inventory-sha256", inv.sha256, "--receipt", str(receipt),
                        "--layers", str(layers), "--expert-split", expert_split]
                log = (receipts_dir / f"worker.{j}.log").open("wb")
                procs.append((subprocess.Popen(argv, stdout=log, stderr=subprocess.STDOUT, stdin=subprocess.DEVNULL), receipt, log))
            failed = []
            deadline = time.monotonic() + timeout
            for proc, receipt, log in procs:
                try:
                    code = proc.wait(timeout=max(0.0, deadline - time.monotonic()))
                except subprocess.TimeoutExpired:
                    proc.kill()
                    code = -9
                log.close()
                if code != 0 or not receipt.exists():
                    failed.append((receipt.name, code))
            if failed:
                raise CheckpointValidationError(f"pack workers failed: {failed}; see {receipts_dir}")
            receipts = [json.loads(r.read_text()) for _, r, _ in procs]
        man = manifest_mod.assemble_manifest(receipts, geometry, world, inv.sha256, expert_split)
        sealed = seal.install(target, geometry, man)
        report = verify.verify_runtime_checkpoint(target)
        return {"ok": True, "target": str(target), "world": world, "expert_split": expert_split, "files": report["files"], "total_bytes": man["total_bytes"],
                "manifest_sha256": sealed["manifest_sha256"], "geometry_sha256": geometry.geometry_hash,
                "source_inventory_sha256": inv.sha256, "source_marker": bool(marker),
                "source_marker_sha256": source_marker.marker_sha256(source) if marker else "", "seconds": round(time.time() - started, 3)}

    if run_root is None:
        return body()
    with workload_lease(run_root):
        return body()

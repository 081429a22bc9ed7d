"""``glm-b200 checkpoint inventory|mark-source|pack|verify``.

Every action prints one JSON report.  ``pack`` holds the workload lease of the site's run root while it writes and refuses a
source whose marker is not the one the site pins (``[checkpoint] source_marker_sha256``, printed by ``mark-source``); ``verify``
refuses a checkpoint that is not the pinned one (``manifest_sha256``, printed by ``pack``).

Parity: reference ``glm_tpu/entrypoints/cli/checkpoint.py``.
"""

from __future__ import annotations

import json


def main(args) -> int:
    from glm_tpu_b200.config.site import SiteConfig
    from glm_tpu_b200.model_loader import source_inventory, source_marker

    if args.action == "inventory":
        inv = source_inventory.read_source_inventory(args.source)
        by_dtype: dict = {}
        for t in inv.tensors.values():
            by_dtype[t.dtype] = by_dtype.get(t.dtype, 0) + (t.end - t.begin)
        report = {"ok": True, "source": str(args.source), "inventory_sha256": inv.sha256, "tensors": len(inv.tensors),
                  "shards": len(inv.shards), "total_bytes": sum(inv.shards.values()), "bytes_by_dtype": dict(sorted(by_dtype.items()))}
        from pathlib import Path

        if getattr(args, "output", None) is not None:
            from glm_tpu_b200.utils.io_utils import create_private_exclusive
            from glm_tpu_b200.utils.json_utils import canonical_wire_bytes

            record = {"schema": "glm_b200_source_inventory_v1", "inventory_sha256": inv.sha256, **inv.listing()}
            create_private_exclusive(Path(args.output), canonical_wire_bytes(record) + b"\n")
            report["output"] = str(args.output)
        config = Path(args.source) / "config.json"
        if config.is_file():  # is this the architecture the package pins (models/glm_moe_dsa/hf_config)?
            from glm_tpu_b200.config.model import ModelGeometry
            from glm_tpu_b200.models.glm_moe_dsa import assets

            g = ModelGeometry.from_hf_config(json.loads(config.read_text()))
            report["geometry_hash"] = g.geometry_hash
            report["matches_pinned_glm53"] = g.geometry_hash == assets.load_pinned_geometry().geometry_hash
    elif args.action == "mark-source" and getattr(args, "upstream_marker", None) is not None:
        result = source_marker.check_against_upstream(args.source, args.upstream_marker, output=getattr(args, "output", None),
                                                      hash_shards=getattr(args, "hash_shards", False))
        marker = result.pop("marker")
        report = {"ok": True, "source": str(args.source), "inventory_sha256": marker["inventory_sha256"], "tensor_count": marker["tensor_count"],
                  "total_bytes": marker["total_bytes"], **result}
    elif args.action == "mark-source":
        if getattr(args, "output", None) is not None:
            from glm_tpu_b200.exceptions import ConfigValidationError

            raise ConfigValidationError("--output goes with --upstream-marker; a source is marked in place")
        marker = source_marker.mark_source(args.source, hash_shards=getattr(args, "hash_shards", False))
        report = {"ok": True, "source": str(args.source), "inventory_sha256": marker["inventory_sha256"],
                  "tensor_count": marker["tensor_count"], "total_bytes": marker["total_bytes"],
                  "marker_sha256": source_marker.marker_sha256(args.source)}
    elif args.action == "pack":
        from glm_tpu_b200.executor.pack_job import pack_checkpoint

        site = SiteConfig.load(getattr(args, "site", None))
        report = pack_checkpoint(args.source, args.target, args.gpus, run_root=site.paths.run_root, layers=args.layers,
                                 expert_split=getattr(args, "expert_split", "auto"), pins=site.checkpoint_pins,
                                 preflight_only=getattr(args, "preflight_only", False))
    else:
        from glm_tpu_b200.model_loader.sharded_state.verify import verify_runtime_checkpoint

        site = SiteConfig.load(getattr(args, "site", None))
        report = verify_runtime_checkpoint(args.target, files=getattr(args, "files", None), pins={"manifest_sha256": site.manifest_sha256},
                                           rehash=not getattr(args, "headers_only", False))
        report["rehashed"] = not getattr(args, "headers_only", False)
        report.pop("manifest_files", None)  # the per-tensor records stay in manifest.json
    print(json.dumps(report, indent=2, sort_keys=True))
    return 0

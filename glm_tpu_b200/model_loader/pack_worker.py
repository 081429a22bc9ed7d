"""One packing process: writes the files it is told to and leaves a receipt.

``python -m glm_tpu_b200.model_loader.pack_worker --source S --target T --world W --files shared,0,1 --inventory-sha256 H
--receipt R [--layers N] [--expert-split whole|sliced]``.  The worker re-reads the source inventory and refuses one that differs from the digest the
controller pinned, rebuilds the geometry from ``config.json``, packs its files and writes the receipt create-once.
Packing is host work (file IO and byte shuffling): it needs no GPU, so the controller may run as many workers as the
storage sustains.

Parity: reference ``glm_tpu/model_loader/pack_worker.py`` (worker entry with rendezvous barriers; here the barrier is the
controller waiting for every receipt).
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

from glm_tpu_b200.config.model import ModelGeometry
from glm_tpu_b200.model_loader import source_inventory
from glm_tpu_b200.model_loader.sharded_state import writer
from glm_tpu_b200.utils.io_utils import create_private_exclusive
from glm_tpu_b200.utils.json_utils import canonical_wire_bytes


def source_geometry(source: Path, layers: int = 0) -> ModelGeometry:
    g = ModelGeometry.from_hf_config(json.loads((Path(source) / "config.json").read_text()))
    return g.truncated(layers) if layers else g


def run(source: Path, target: Path, world: int, files: list, inventory_sha256: str, layers: int = 0, split: str = "whole") -> dict:
    inv = source_inventory.authenticated_inventory(source, inventory_sha256)
    geometry = source_geometry(source, layers)
    return writer.pack_files(inv, target, geometry, world, files, split)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="pack_worker")
    ap.add_argument("--source", type=Path, required=True)
    ap.add_argument("--target", type=Path, required=True)
    ap.add_argument("--world", type=int, required=True)
    ap.add_argument("--files", required=True, help="comma separated: 'shared' and/or rank numbers")
    ap.add_argument("--inventory-sha256", required=True)
    ap.add_argument("--receipt", type=Path, required=True)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--expert-split", default="whole", choices=["whole", "sliced"])
    args = ap.parse_args(argv)
    receipt = run(args.source, args.target, args.world, args.files.split(","), args.inventory_sha256, args.layers, args.expert_split)
    create_private_exclusive(args.receipt, canonical_wire_bytes(receipt) + b"\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())

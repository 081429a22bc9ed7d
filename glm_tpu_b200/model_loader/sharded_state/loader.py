"""Loading a packed checkpoint on one GPU rank.

``load_rank_checkpoint(dir, rank, world, device=...)`` verifies the seal, the manifest and the headers of this rank's two
files, and returns a *streamed* runtime-layout mapping ``name -> tensor``: nothing is read until a tensor is asked for, and
then it travels file -> staging buffer (at most ``format.PIECE_BYTES``, pinned) -> ``device`` piece by piece, hashed and
checked (FP8 NaN codes, finiteness) on the way; the digest is compared with the manifest's record of that tensor.  The
model code asks for each tensor once, decodes FP8 pairs to bf16 on the device and cuts heads / MLP columns / vocabulary
rows, so host memory never holds more than the staging buffer and every byte is read from disk once.  The routed experts of
this rank arrive already cut (whole experts ``[experts_local, N, K]`` or this GPU's column slice of every expert, as the
checkpoint was packed).  ``load_full_checkpoint`` reassembles the full stacked layout (CPU oracle, small models only).

Parity: reference ``glm_tpu/model_loader/sharded_state/loader.py:58-154``.
"""

from __future__ import annotations

from collections.abc import Mapping
from pathlib import Path

import torch

from glm_tpu_b200.exceptions import CheckpointValidationError
from glm_tpu_b200.model_loader.sharded_state import format as fmt
from glm_tpu_b200.model_loader.sharded_state.verify import read_geometry, verify_runtime_checkpoint

__all__ = ["read_geometry", "load_rank_checkpoint", "load_full_checkpoint", "StreamedCheckpoint"]


class StreamedCheckpoint(Mapping):
    """``name -> tensor`` over the files of a packed checkpoint; a tensor is streamed to ``device`` when it is looked up."""

    def __init__(self, target: Path, files: list, manifest_files: dict, device=None, extra: dict | None = None):
        self.device = device
        self._extra = dict(extra or {})
        self._where: dict = {}
        self._readers: dict = {}
        self._digests: dict = {}
        for name in files:
            reader = fmt.TensorReader(Path(target) / name)
            self._readers[name] = reader
            recorded = manifest_files[name]["tensors"]
            for tensor in reader.names():
                if tensor in self._where:
                    raise CheckpointValidationError(f"{tensor} appears in two files")
                self._where[tensor] = name
                self._digests[tensor] = recorded[tensor].get("sha256")
                if not self._digests[tensor]:
                    raise CheckpointValidationError(f"the manifest records no digest for {tensor}")

    def __getitem__(self, name: str):
        if name in self._extra:
            return self._extra[name]
        reader = self._readers[self._where[name]]
        return reader.read(name, device=self.device, expect_sha256=self._digests[name])

    def __iter__(self):
        yield from self._where
        yield from self._extra

    def __len__(self) -> int:
        return len(self._where) + len(self._extra)

    def __contains__(self, name) -> bool:
        return name in self._where or name in self._extra

    def io_stats(self) -> dict:
        return {"bytes_read": sum(r.bytes_read for r in self._readers.values()),
                "largest_piece": max((r.largest_piece for r in self._readers.values()), default=0)}

    def close(self) -> None:
        for reader in self._readers.values():
            reader.close()


def load_rank_checkpoint(target: Path, rank: int, world: int, *, pins: dict | None = None, rehash: bool = False, device=None) -> StreamedCheckpoint:
    """``rehash=True`` additionally re-hashes the two files whole before anything is loaded (a second pass over the bytes);
    by default the per-tensor digests checked while streaming carry the authentication."""
    target = Path(target)
    files = [fmt.SHARED_FILE, fmt.expert_file(rank, world)]
    report = verify_runtime_checkpoint(target, files=files, pins=pins, rehash=rehash)
    if report["world"] != world:
        raise CheckpointValidationError(f"the checkpoint was packed for {report['world']} GPUs, not {world}")
    extra = {"__experts_presliced__": torch.tensor([rank, world]), "__expert_split__": report["expert_split"]}
    return StreamedCheckpoint(target, files, report["manifest_files"], device=device, extra=extra)


def load_full_checkpoint(target: Path) -> dict:
    target = Path(target)
    report = verify_runtime_checkpoint(target)
    world, split = report["world"], report["expert_split"]
    shared = StreamedCheckpoint(target, [fmt.SHARED_FILE], report["manifest_files"])
    arrays = {name: shared[name] for name in shared}
    parts = [StreamedCheckpoint(target, [fmt.expert_file(r, world)], report["manifest_files"]) for r in range(world)]
    for name in parts[0]:
        pieces = [p[name] for p in parts]
        if split == "whole":
            arrays[name] = torch.cat(pieces, dim=0)
        else:  # gate/up tables and their scales were cut by row, down tables by column
            arrays[name] = torch.cat(pieces, dim=2 if ".down_proj." in name else 1)
    return arrays

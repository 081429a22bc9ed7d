"""G3: execution digests of the CPU contract oracle on the frozen fixture, and G4: checkpoint identity.

The oracle is what every GPU kernel is compared with, so its outputs on the fixture are pinned: the greedy tokens, the SHA-256 of
the bf16 logits, of every layer's cached rows, of the DSA selections and of the routed experts.  G4 pins the bytes of the fixture
checkpoint after export -> pack: per packed file the header digest and the content digest, plus the manifest digest.
"""

from __future__ import annotations

import hashlib
import tempfile
from pathlib import Path

import torch


def _tsha(t: torch.Tensor) -> str:
    t = t.contiguous()
    if t.dtype == torch.bfloat16:
        t = t.view(torch.int16)
    return hashlib.sha256(t.numpy().tobytes()).hexdigest()


def oracle_digests() -> dict:
    from glm_tpu_b200.oracle import contract
    from tools.equivalence import fixture as fx

    g, ckpt = fx.fixture_geometry(), fx.fixture_checkpoint()
    w = contract.OracleWeights.from_checkpoint(g, ckpt)
    seq = fx.fixture_prompt()
    generated = []
    for _ in range(fx.NEW_TOKENS):
        trace = contract.forward(w, seq, capacity=fx.CAPACITY)
        generated.append(int(trace.tokens[-1]))
        seq = seq + [generated[-1]]
    out = {"generated": generated, "logits": _tsha(trace.logits.to(torch.bfloat16)), "residual": _tsha(trace.residual.to(torch.bfloat16))}
    out["kv_rows"] = [_tsha(k.to(torch.bfloat16)) for k in trace.kv_rows]
    sel = trace.selected
    layers = sorted(sel) if isinstance(sel, dict) else range(len(sel))
    out["selected"] = {str(layer): hashlib.sha256(repr([r.tolist() for r in sel[layer]]).encode()).hexdigest() for layer in layers if sel[layer]}
    out["expert_ids"] = {str(layer): _tsha(ids.to(torch.int32)) for layer, ids in sorted(trace.expert_ids.items())}
    out["index_keys"] = {str(layer): _tsha(keys.to(torch.bfloat16)) for layer, keys in sorted(trace.index_keys.items())}
    out["index_scores"] = {str(layer): _tsha(torch.nan_to_num(s, neginf=-1e30).to(torch.float32)) for layer, s in sorted(trace.index_scores.items())}
    # tie rules on constructed inputs (random fixtures never tie exactly): lowest id / lowest position wins, -0 < +0
    tied = torch.tensor([[1.0, 3.0, 3.0, 2.0], [5.0, 5.0, 5.0, 5.0]])
    out["tie_rules"] = {
        "greedy": contract.greedy(tied).tolist(),
        "top_k": contract.top_k_positions(torch.tensor([0.5, 0.0, -0.0, 0.5, 0.5, 0.25]), 6, 3).tolist(),
        "router": contract.router(torch.eye(4), torch.tensor([[1.0, 0, 0, 0], [1.0, 0, 0, 0], [0, 0, 2.0, 0], [0, 0, 2.0, 0]]).T.contiguous(),
                                  torch.zeros(4), 2)[0].tolist(),
    }
    return out


def checkpoint_identity() -> dict:
    from glm_tpu_b200.executor.pack_job import pack_checkpoint
    from glm_tpu_b200.model_loader import export, source_marker
    from glm_tpu_b200.model_loader.sharded_state import format as fmt
    from tools.equivalence import fixture as fx

    g, ckpt = fx.fixture_geometry(), fx.fixture_checkpoint()
    with tempfile.TemporaryDirectory() as tmp:
        root = Path(tmp)
        export.export_source(ckpt, g, root / "src", shards=3)
        marker = source_marker.mark_source(root / "src")
        report = pack_checkpoint(root / "src", root / "packed", 4, jobs=1)
        files = {}
        for name in report["files"]:
            header, _ = fmt.read_header(root / "packed" / name)
            files[name] = {"header": hashlib.sha256(repr(sorted((k, str(v)) for k, v in header.items())).encode()).hexdigest(),
                           "content": fmt.file_sha256(root / "packed" / name)}
        return {"geometry_sha256": g.geometry_hash, "source_inventory_sha256": marker["inventory_sha256"], "manifest_sha256": report["manifest_sha256"],
                "total_bytes": report["total_bytes"], "files": files}

"""G1: the launch programs.  This engine has no compiler whose output could be fingerprinted; its "program" is the ordered list of
kernel launches a step issues (entry point of the CUDA library + every integer argument: sizes, strides, counts, modes, which
determine grid, block and shared memory inside the launcher).  The gate records that list for one decode step and one prefill
chunk of fixed configurations (single chat and four chats; one GPU and the shard of one GPU of eight) and freezes, per
configuration, the number of launches, the launches per entry point and a SHA-256 over the whole list.  A change of a kernel's
tiling, of the order of launches or of a fused path shows up as a changed fingerprint and has to be accepted on purpose
(``python -m tools.equivalence.driver update g1_launch_programs`` on a B200).

Needs a GPU (the launches are really issued, eagerly, on tiny tensors); on a machine without one the driver skips the gate.

Parity: reference ``tools/equivalence/programs.py`` (fingerprints of the lowered decode / prefill programs per profile).
"""

from __future__ import annotations

import hashlib
import json


def available() -> bool:
    import torch

    return torch.cuda.is_available()


def _fingerprint(rows) -> dict:
    listing = [[name, list(ints)] for name, ints, _ in rows]
    by_entry: dict = {}
    for name, _ in listing:
        by_entry[name] = by_entry.get(name, 0) + 1
    digest = hashlib.sha256(json.dumps(listing, separators=(",", ":")).encode()).hexdigest()
    return {"launches": len(listing), "by_entry": dict(sorted(by_entry.items())), "sha256": digest}


def _configurations():
    from glm_tpu_b200.config.model import glm53_geometry, small_geometry

    small, glm = small_geometry(4), glm53_geometry().truncated(8)
    # name, geometry, world (> 1: this process holds rank 0's shard and skips the exchanges), lanes, context, prefill rows
    return [("small4.gpus1.chats1", small, 1, 1, 256, 48), ("small4.gpus1.chats4", small, 1, 4, 256, 0),
            ("glm53x8.gpus1.chats1", glm, 1, 1, 4096, 256), ("glm53x8.shard-of-8.chats1", glm, 8, 1, 4096, 0),
            ("glm53x8.shard-of-8.chats4", glm, 8, 4, 4096, 0)]


def collect() -> dict:
    import torch

    from glm_tpu_b200.ops import native
    from glm_tpu_b200.runner.gpu_runner import build_runner

    out = {}
    for name, geometry, world, lanes, context, prefill_rows in _configurations():
        runner = build_runner(geometry, world=world, rank=0, device="cuda:0", seed=0, context_capacity=context, lanes=lanes, use_graphs=False,
                              emulate_shard=world > 1, kv_layout="replicated" if world > 1 else "auto", prefill_chunk=max(prefill_rows, 16))
        try:
            record = {"expert_split": runner.model.layout.expert_split, "decode_path": runner.decode_path}
            if prefill_rows:
                gen = torch.Generator().manual_seed(1)
                prompt = torch.randint(0, geometry.vocab_size, (prefill_rows,), generator=gen).tolist()
                with native.kernel_timeline() as tl:
                    runner.prefill(0, prompt)
                record["prefill_chunk"] = _fingerprint(tl.rows())
                first = 1
            else:
                first = 0
            for lane in range(first, lanes):
                runner.synthetic_context(lane, 100 + 7 * lane, seed=lane)
            runner.build_decode_program()
            runner.decode_step()  # the first step may allocate lazily; the recorded one is a steady-state step
            with native.kernel_timeline() as tl:
                runner.decode_step()
            record["decode_step"] = _fingerprint(tl.rows())
            runner.peer.check_status()
            out[name] = record
        finally:
            runner.close()
            del runner
            torch.cuda.empty_cache()
    return out

"""G6: import closures.  For each entry module, the set of ``glm_tpu_b200`` modules (and heavy third-party roots) that importing it
pulls in, measured in a fresh interpreter.  A closure may only shrink: a new edge (the CLI importing torch, the engine importing the
CUDA bindings, the HTTP handler importing the model) fails the gate until the golden is updated on purpose.
"""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
ENTRIES = ("glm_tpu_b200.entrypoints.cli.main", "glm_tpu_b200.engine.llm_engine", "glm_tpu_b200.engine.request", "glm_tpu_b200.config.site",
           "glm_tpu_b200.entrypoints.serve.http_handler", "glm_tpu_b200.entrypoints.openai.serving_chat", "glm_tpu_b200.executor.multiproc_executor",
           "glm_tpu_b200.model_loader.source_inventory", "glm_tpu_b200.parallel.topology", "glm_tpu_b200.tokenizer")
HEAVY = ("torch", "numpy", "transformers", "tokenizers")
_PROBE = ("import importlib, json, sys; importlib.import_module(sys.argv[1]); "
          "mods = sorted(m for m in sys.modules if m.startswith('glm_tpu_b200')); "
          "heavy = sorted(h for h in %r if h in sys.modules); print(json.dumps({'modules': mods, 'heavy': heavy}))" % (HEAVY,))


def closure(entry: str) -> dict:
    done = subprocess.run([sys.executable, "-c", _PROBE, entry], capture_output=True, text=True, cwd=ROOT, timeout=300)
    if done.returncode != 0:
        raise RuntimeError(f"importing {entry} failed:\n{done.stderr[-2000:]}")
    return json.loads(done.stdout.strip().splitlines()[-1])


def collect() -> dict:
    return {entry: closure(entry) for entry in ENTRIES}


def grown(golden: dict, current: dict) -> dict:
    """What the current closures contain that the golden ones do not (empty = gate passes)."""
    out = {}
    for entry, now in current.items():
        was = golden.get(entry, {"modules": [], "heavy": []})
        extra = {"modules": sorted(set(now["modules"]) - set(was["modules"])), "heavy": sorted(set(now["heavy"]) - set(was["heavy"]))}
        if extra["modules"] or extra["heavy"]:
            out[entry] = extra
    return out

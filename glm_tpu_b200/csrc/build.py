"""Build the CUDA library in-tree: every ``.cu`` under ``csrc/`` -> ``glm_tpu_b200/ops/libglmb200.so`` (sm_100a).

``python -m glm_tpu_b200.csrc.build`` (or ``build()``) cross-compiles without a GPU.  Objects are rebuilt
only when a source or header is newer.  The library links nothing but the CUDA runtime, so it loads in
any process (ctypes) and its path shows up in the process map.
"""

from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
OUT_DIR = CSRC.parent / "ops"
LIB = OUT_DIR / "libglmb200.so"
OBJ_DIR = CSRC / "build"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(d.stat().st_mtime > stamp for d in deps)


def build(verbose: bool = False, force: bool = False) -> Path:
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    OBJ_DIR.mkdir(exist_ok=True)
    OUT_DIR.mkdir(exist_ok=True)

    def compile_one(src: Path) -> Path:
        obj = OBJ_DIR / (src.stem + ".o")
        if force or _stale(obj, [src, *headers]):
            cmd = [NVCC, *FLAGS, "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
                print(" ".join(cmd), flush=True)
            done = subprocess.run(cmd, capture_output=True, text=True)
            if done.returncode != 0:
                raise RuntimeError(f"nvcc failed for {src.name}:\n{done.stdout}\n{done.stderr}")
            if verbose:
                print(done.stderr, flush=True)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources) or 1)) as pool:
        objects = list(pool.map(compile_one, sources))
    if force or _stale(LIB, objects):
        cmd = [NVCC, "-shared", "-o", str(LIB), *map(str, objects), "-lcudart"]
        done = subprocess.run(cmd, capture_output=True, text=True)
        if done.returncode != 0:
            raise RuntimeError(f"link failed:\n{done.stdout}\n{done.stderr}")
    return LIB


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print(path)

"""``collect-env`` / ``doctor``: what this machine has, checked against what the engine needs.

Reports Python, torch, CUDA toolkit, driver, GPUs (name, memory, clocks), NVLink peer access, the built library and the
registered environment variables; ``--profile`` selects which checks are errors (``serve`` needs GPUs and the library,
``dev`` only needs the toolchain).

Parity: reference ``glm_tpu/entrypoints/cli/collect_env.py:113-191`` (installed versions vs pins).
"""

from __future__ import annotations

import json
import platform
import shutil
import subprocess
import sys

REQUIRED = {"python": (3, 10), "torch": (2, 4), "cuda_toolkit": (12, 8)}


def _version_tuple(text: str) -> tuple:
    out = []
    for part in text.replace("+", ".").split("."):
        if part.isdigit():
            out.append(int(part))
        else:
            break
    return tuple(out)


def collect() -> dict:
    info: dict = {"python": platform.python_version(), "platform": platform.platform()}
    try:
        import torch

        info["torch"] = torch.__version__
        info["torch_cuda"] = torch.version.cuda
        info["cuda_available"] = torch.cuda.is_available()
        info["gpus"] = []
        if torch.cuda.is_available():
            for i in range(torch.cuda.device_count()):
                p = torch.cuda.get_device_properties(i)
                info["gpus"].append({"index": i, "name": p.name, "memory_gib": round(p.total_memory / 2**30, 1),
                                     "sm": f"{p.major}.{p.minor}", "sms": p.multi_processor_count})
            n = torch.cuda.device_count()
            info["peer_access"] = all(torch.cuda.can_device_access_peer(i, j) for i in range(n) for j in range(n) if i != j) if n > 1 else None
        import torch.distributed as dist

        info["nccl"] = ".".join(map(str, torch.cuda.nccl.version())) if dist.is_nccl_available() else None
    except ImportError:
        info["torch"] = None
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    try:
        out = subprocess.run([nvcc, "--version"], capture_output=True, text=True, timeout=20).stdout
        info["cuda_toolkit"] = next((ln.split("release ")[1].split(",")[0] for ln in out.splitlines() if "release " in ln), None)
    except (OSError, subprocess.TimeoutExpired):
        info["cuda_toolkit"] = None
    try:
        out = subprocess.run(["nvidia-smi", "--query-gpu=driver_version", "--format=csv,noheader"], capture_output=True, text=True, timeout=20)
        info["driver"] = out.stdout.splitlines()[0].strip() if out.returncode == 0 and out.stdout.strip() else None
    except (OSError, subprocess.TimeoutExpired):
        info["driver"] = None
    from glm_tpu_b200 import envs
    from glm_tpu_b200.ops import native

    info["library_built"] = native.available()
    info["env"] = envs.describe()
    return info


def check(info: dict, profile: str) -> list[str]:
    problems = []
    if _version_tuple(info["python"]) < REQUIRED["python"]:
        problems.append(f"python {info['python']} is older than {REQUIRED['python']}")
    if not info.get("torch") or _version_tuple(info["torch"]) < REQUIRED["torch"]:
        problems.append("torch >= 2.4 is required")
    if not info.get("cuda_toolkit") or _version_tuple(info["cuda_toolkit"]) < REQUIRED["cuda_toolkit"]:
        problems.append("CUDA toolkit >= 12.8 (nvcc with sm_100a) is required to build the kernels")
    if profile == "serve":
        if not info.get("gpus"):
            problems.append("no CUDA GPU is visible")
        elif any(g["sm"] != "10.0" for g in info["gpus"]):
            problems.append("the kernels are built for sm_100a (B200) only")
        if not info.get("library_built"):
            problems.append("libglmb200.so is not built: run `python -m glm_tpu_b200.csrc.build`")
        if info.get("peer_access") is False:
            problems.append("GPUs cannot access each other's memory (NVLink peer access is required for the fused collectives)")
    return problems


def main(args) -> int:
    info = collect()
    problems = check(info, args.profile)
    print(json.dumps({"profile": args.profile, "ok": not problems, "problems": problems, "info": info}, indent=2, sort_keys=True))
    return 0 if not problems else 1

"""``collect-env`` / ``doctor``: what this machine has, checked against what the engine needs.

Reports Python, torch, CUDA toolkit, driver, GPUs (name, memory, clocks), NVLink peer access, the built library and the
registered environment variables; ``--profile`` selects which checks are errors (``serve`` needs GPUs and the library,
``dev`` only needs the toolchain).  The installed distributions are compared with what the project declares
(``pyproject.toml``, or the installed distribution's metadata when there is no checkout): a declared package of the profile's
groups that is missing or older than its lower bound is an error, one of the other groups is only listed.

Parity: reference ``glm_tpu/entrypoints/cli/collect_env.py:113-191`` (installed versions vs pins).
"""

from __future__ import annotations

import json
import platform
import re
import shutil
import subprocess
import sys
from pathlib import Path

REQUIRED = {"python": (3, 10), "torch": (2, 4), "cuda_toolkit": (12, 8)}


def _version_tuple(text: str) -> tuple:
    out = []
    for part in text.replace("+", ".").split("."):
        if part.isdigit():
            out.append(int(part))
        else:
            break
    return tuple(out)


# which declared groups a profile needs ("core" = [project] dependencies, the others = optional-dependencies tables)
PROFILE_GROUPS = {"dev": ("core", "dev"), "serve": ("core",)}
PYPROJECT = Path(__file__).resolve().parents[3] / "pyproject.toml"
_REQUIREMENT = re.compile(r"\s*([A-Za-z0-9][A-Za-z0-9._-]*)\s*(?:(>=|==)\s*([0-9][0-9A-Za-z.+!-]*))?\s*")


def declared_packages(pyproject: Path | None = None, *, distribution=None) -> dict[str, dict[str, tuple[str, str]]]:
    """``{group: {package: (operator, version)}}`` as the project declares it: from ``pyproject.toml`` of a checkout, else from the
    metadata of the installed ``glm-tpu-b200`` distribution.  Only ``>=`` and ``==`` bounds (or none) are understood; anything else
    is refused rather than half-checked."""
    import tomllib
    from importlib import metadata

    pyproject = PYPROJECT if pyproject is None else pyproject
    rows: list[tuple[str, str]] = []
    if pyproject.is_file():
        project = tomllib.loads(pyproject.read_text()).get("project", {})
        if project.get("name") != "glm-tpu-b200":
            raise ValueError(f"{pyproject} does not declare the glm-tpu-b200 project")
        rows += [("core", r) for r in project.get("dependencies", [])]
        rows += [(group, r) for group, reqs in project.get("optional-dependencies", {}).items() for r in reqs]
    else:
        try:
            dist = metadata.distribution("glm-tpu-b200") if distribution is None else distribution
        except metadata.PackageNotFoundError:
            raise ValueError(f"no {pyproject} and no installed glm-tpu-b200 distribution: nothing declares the requirements") from None
        for r in dist.requires or ():
            spec, _, marker = r.partition(";")
            extra = re.search(r"extra\s*==\s*['\"]([^'\"]+)['\"]", marker)
            if marker.strip() and not extra:
                raise ValueError(f"unsupported requirement marker: {r}")
            rows.append((extra.group(1) if extra else "core", spec))
    groups: dict[str, dict[str, tuple[str, str]]] = {}
    for group, text in rows:
        m = _REQUIREMENT.fullmatch(text)
        if m is None:
            raise ValueError(f"unsupported requirement: {text!r}")
        groups.setdefault(group, {})[m.group(1).lower().replace("_", "-")] = (m.group(2) or "", m.group(3) or "")
    return groups


def package_rows(profile: str, groups: dict, installed_version=None) -> list[dict]:
    """One row per declared package: group, declared bound, installed version, whether it satisfies the bound and whether the
    profile needs it.  ``installed_version(name)`` returns a version string or raises ``PackageNotFoundError`` (tests inject a fake)."""
    from importlib import metadata

    installed_version = metadata.version if installed_version is None else installed_version
    needed = PROFILE_GROUPS[profile]
    rows = []
    for group in sorted(groups):
        for name, (op, bound) in sorted(groups[group].items()):
            try:
                have = installed_version(name)
            except metadata.PackageNotFoundError:
                have = None
            if have is None:
                ok = False
            elif op == ">=":
                ok = _version_tuple(have) >= _version_tuple(bound)
            elif op == "==":  # a pin without a local label also matches the same release with one (2.11.0+cu128 == 2.11.0)
                ok = have == bound or ("+" not in bound and have.split("+", 1)[0] == bound)
            else:
                ok = True
            rows.append({"group": group, "package": name, "declared": f"{op}{bound}" if op else "any", "installed": have, "ok": ok,
                         "required": group in needed})
    return rows


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
    try:
        info["declared"] = declared_packages()
    except ValueError as exc:
        info["declared"] = {}
        info["declared_error"] = str(exc)
    return info


def check(info: dict, profile: str) -> list[str]:
    problems = []
    if _version_tuple(info["python"]) < REQUIRED["python"]:
        problems.append(f"python {info['python']} is older than {REQUIRED['python']}")
    if not info.get("torch") or _version_tuple(info["torch"]) < REQUIRED["torch"]:
        problems.append("torch >= 2.4 is required")
    if not info.get("cuda_toolkit") or _version_tuple(info["cuda_toolkit"]) < REQUIRED["cuda_toolkit"]:
        problems.append("CUDA toolkit >= 12.8 (nvcc with sm_100a) is required to build the kernels")
    if info.get("declared_error"):
        problems.append(info["declared_error"])
    for row in info.get("packages", []):
        if row["required"] and not row["ok"]:
            problems.append(f"{row['package']} {row['declared']} is declared ({row['group']}), installed: {row['installed'] or 'nothing'}")
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
    info["packages"] = package_rows(args.profile, info.pop("declared"))
    problems = check(info, args.profile)
    print(json.dumps({"profile": args.profile, "ok": not problems, "problems": problems, "info": info}, indent=2, sort_keys=True))
    return 0 if not problems else 1

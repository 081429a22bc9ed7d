"""What the controller records (and may require) about the source tree it launches from.

``source_identity`` reports the git commit, branch, and whether the tree is clean; ``check`` applies a policy:
``strict`` refuses a dirty or detached tree, ``record`` (default) only records.  The identity goes into
``controller_identity.json`` of every run so that results can be tied to a commit.

Parity: reference ``glm_tpu/executor/launch_policy.py:129-220`` (clean / branch / origin / pushed policy).
"""

from __future__ import annotations

import subprocess
from pathlib import Path

from glm_tpu_b200.exceptions import ConfigValidationError


def _git(repo: Path, *args: str) -> str | None:
    try:
        done = subprocess.run(["git", "-C", str(repo), *args], capture_output=True, text=True, timeout=20)
    except (OSError, subprocess.TimeoutExpired):
        return None
    return done.stdout.strip() if done.returncode == 0 else None


def source_identity(repo: Path) -> dict:
    repo = Path(repo)
    commit = _git(repo, "rev-parse", "HEAD")
    status = _git(repo, "status", "--porcelain")
    branch = _git(repo, "rev-parse", "--abbrev-ref", "HEAD")
    return {
        "repo": str(repo),
        "git": commit is not None,
        "commit": commit,
        "branch": branch,
        "clean": status == "" if status is not None else None,
        "dirty_files": len(status.splitlines()) if status else 0,
    }


def check(identity: dict, policy: str = "record") -> None:
    if policy not in ("record", "strict"):
        raise ConfigValidationError("launch policy is 'record' or 'strict'")
    if policy == "strict":
        if not identity["git"]:
            raise ConfigValidationError("strict launch policy needs a git checkout")
        if not identity["clean"]:
            raise ConfigValidationError("strict launch policy refuses a tree with uncommitted changes")
        if identity["branch"] in (None, "HEAD"):
            raise ConfigValidationError("strict launch policy refuses a detached HEAD")

"""What the controller records (and may require) about the source tree it launches from.

``source_identity`` describes the checkout: commit, branch, cleanliness, the origin remote and whether the branch head is what
origin has.  ``check`` applies the site's rules to it, in a fixed order, and the first rule that fails refuses the launch:

    clean      no modified, staged or untracked file
    head       HEAD is a commit (a 40-hex pin)
    branch     on a branch (not detached) whose name matches one of ``allowed_branches``
    origin     the ``origin`` remote is the expected one (spelling-normalised; a local path never passes for a remote)
    pushed     ``origin`` has this very commit at ``refs/heads/<branch>``

``policy = "record"`` applies no rule and only records; ``"strict"`` applies clean + head + branch always, origin when
``expected_origin`` is set, pushed when ``require_pushed`` is set.  The identity goes into ``controller_identity.json`` of
every run and, as the source pin, to the workers.

Parity: reference ``glm_tpu/executor/launch_policy.py:129-173`` (rule order clean, HEAD, branch, origin, pushed).
"""

from __future__ import annotations

import fnmatch
import os
import re
import subprocess
from dataclasses import dataclass
from pathlib import Path

from glm_tpu_b200.exceptions import ConfigValidationError

_PIN = re.compile(r"[0-9a-f]{40}")
_SCP = re.compile(r"^(?:[^@/]+@)?([^:/]+):(?!//)(.+)$")
_URL = re.compile(r"^[a-z][a-z0-9+.-]*://(?:[^@/]*@)?([^/:]+)(?::(\d+))?/(.*)$", re.I)
DEFAULT_PORTS = {"22", "443", "80", "9418"}


@dataclass(frozen=True)
class LaunchRules:
    policy: str = "record"
    allowed_branches: tuple = ("main", "release/*")
    expected_origin: str = ""
    require_pushed: bool = False


def _git(repo: Path, *args: str, timeout: float = 20.0) -> str | None:
    try:
        done = subprocess.run(["git", "-C", str(repo), *args], capture_output=True, text=True, timeout=timeout,
                              env=dict(os.environ, GIT_TERMINAL_PROMPT="0"))
    except (OSError, subprocess.TimeoutExpired):
        return None
    return done.stdout.strip() if done.returncode == 0 else None


def normalize_origin(url: str, base: Path | None = None) -> tuple[str, str]:
    """``(kind, spelling)``: kind ``'remote'`` with ``host[:port]/path`` (no credentials, no trailing ``/`` or ``.git``, host in
    lower case) or ``'local'`` with an absolute path.  Two origins are the same only if kind and spelling are equal."""
    url = url.strip()
    m = _URL.match(url)
    if m and not url.lower().startswith("file://"):
        host, port, path = m.group(1).lower(), m.group(2), m.group(3)
        where = host + (f":{port}" if port and port not in DEFAULT_PORTS else "")
        return "remote", where + "/" + re.sub(r"(\.git)?/*$", "", path)
    m = _SCP.match(url)
    if m and not os.path.exists(url):
        return "remote", m.group(1).lower() + "/" + re.sub(r"(\.git)?/*$", "", m.group(2))
    path = url[7:] if url.lower().startswith("file://") else url
    p = Path(path)
    if not p.is_absolute():
        p = Path(base if base is not None else Path.cwd()) / p
    return "local", str(Path(os.path.normpath(p)))


def source_identity(repo: Path) -> dict:
    repo = Path(repo)
    commit = _git(repo, "rev-parse", "--verify", "HEAD^{commit}")
    status = _git(repo, "status", "--porcelain", "--untracked-files=normal")
    branch = _git(repo, "symbolic-ref", "--quiet", "--short", "HEAD")
    origin = _git(repo, "remote", "get-url", "origin")
    return {
        "repo": str(repo),
        "git": commit is not None,
        "commit": commit,
        "branch": branch,
        "clean": status == "" if status is not None else None,
        "dirty_files": len(status.splitlines()) if status else 0,
        "origin": origin,
    }


def origin_head(repo: Path, branch: str, timeout: float = 30.0) -> str | None:
    """The commit ``origin`` has at ``refs/heads/<branch>`` (None: no such ref, no origin, or it could not be asked)."""
    ref = "refs/heads/" + branch
    out = _git(Path(repo), "ls-remote", "--exit-code", "origin", ref, timeout=timeout)
    if out is None:
        return None
    heads = [f[0] for f in (line.split("\t") for line in out.splitlines()) if len(f) == 2 and f[1] == ref]
    return heads[0] if len(heads) == 1 else None


def check(identity: dict, policy: str | LaunchRules = "record", *, remote_head=origin_head) -> None:
    """Apply the rules to ``identity``; raises ``ConfigValidationError`` naming the first rule that fails."""
    rules = policy if isinstance(policy, LaunchRules) else LaunchRules(policy=policy)
    if rules.policy not in ("record", "strict"):
        raise ConfigValidationError("launch policy is 'record' or 'strict'")
    if rules.policy == "record":
        return
    if not identity["git"]:
        raise ConfigValidationError("strict launch policy needs a git checkout")
    if not identity["clean"]:
        raise ConfigValidationError("strict launch policy refuses a tree with uncommitted changes (untracked files included)")
    if not identity["commit"] or not _PIN.fullmatch(identity["commit"]):
        raise ConfigValidationError("HEAD is not a 40-hex commit")
    branch = identity["branch"]
    if branch in (None, "", "HEAD"):
        raise ConfigValidationError("strict launch policy refuses a detached HEAD")
    if not any(fnmatch.fnmatchcase(branch, pattern) for pattern in rules.allowed_branches):
        raise ConfigValidationError(f"branch {branch!r} is not allowed by [launch] allowed_branches")
    if rules.expected_origin or rules.require_pushed:
        if not identity.get("origin"):
            raise ConfigValidationError("the checkout has no 'origin' remote ([launch] expected_origin / require_pushed)")
    if rules.expected_origin:
        repo = Path(identity["repo"])
        if normalize_origin(identity["origin"], repo) != normalize_origin(rules.expected_origin, repo):
            raise ConfigValidationError("origin differs from [launch] expected_origin")
    if rules.require_pushed:
        if remote_head(Path(identity["repo"]), branch) != identity["commit"]:
            raise ConfigValidationError(f"the source must be pushed before a launch: origin refs/heads/{branch} does not name HEAD")

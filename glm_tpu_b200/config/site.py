"""The site file: where this installation keeps its runs, its checkpoint and its pins.

``site.toml`` is read fail-closed: it must be a regular file owned by the user and closed to group and others
(0600), every table must have exactly its known keys, paths must be absolute and plain, pins must be 64 lowercase
hex digits, the box shape must be one the engine supports.  ``resolved_json()`` is the canonical form handed to the
workers, ``sha256`` its digest (workers refuse a site that differs from the controller's).  Precedence everywhere:
CLI flag > ``GLM_B200_*`` environment variable > site file > default.

Tables::

    [box]        gpus = 8                       # 1, 2, 4 or 8 GPUs of one NVLink/NVSwitch box
    [paths]      run_root, model_path, packed_path, state_root
    [checkpoint] manifest_sha256, source_marker_sha256      # optional pins ("" = unpinned)
    [topology]   binding_sha256                              # optional pin of the captured GPU topology
    [launch]     policy = "record" | "strict", master_port, wall_seconds,
                 allowed_branches = ["main", "release/*"], expected_origin = "", require_pushed = false   (rules of "strict")
    [serve]      port

Parity: reference ``glm_tpu/config/site.py:92-684`` (7 tables, exact key sets, 0600, 64-hex pins, resolved JSON + SHA).
"""

from __future__ import annotations

import hashlib
import os
import re
import stat
import tomllib
from dataclasses import asdict, dataclass, field
from pathlib import Path

from glm_tpu_b200.exceptions import ConfigValidationError
from glm_tpu_b200.utils.json_utils import canonical_wire_bytes

_HEX64 = re.compile(r"[0-9a-f]{64}")
_PLAIN = re.compile(r"[A-Za-z0-9_./+@:-]+")
_PLAIN_GLOB = re.compile(r"[A-Za-z0-9_./+@:*?\[\]-]+")
SUPPORTED_GPUS = (1, 2, 4, 8)
TABLE_KEYS = {
    "box": {"gpus"},
    "paths": {"run_root", "model_path", "packed_path", "state_root"},
    "checkpoint": {"manifest_sha256", "source_marker_sha256"},
    "topology": {"binding_sha256"},
    "launch": {"policy", "master_port", "wall_seconds", "allowed_branches", "expected_origin", "require_pushed"},
    "serve": {"port"},
}


@dataclass(frozen=True)
class Paths:
    run_root: Path
    model_path: Path | None = None
    packed_path: Path | None = None
    state_root: Path | None = None


@dataclass(frozen=True)
class SiteConfig:
    gpus: int = 8
    paths: Paths = field(default_factory=lambda: Paths(Path.home() / ".cache" / "glm-b200" / "runs"))
    manifest_sha256: str = ""
    source_marker_sha256: str = ""
    topology_binding_sha256: str = ""
    policy: str = "record"
    allowed_branches: tuple = ("main", "release/*")
    expected_origin: str = ""
    require_pushed: bool = False
    master_port: int = 29577
    wall_seconds: int = 86400
    serve_port: int = 8011
    source: str = "<defaults>"

    # ------------------------------------------------------------------ loading
    @classmethod
    def load(cls, path: Path | None = None, *, required: bool = False) -> "SiteConfig":
        from glm_tpu_b200 import envs

        path = Path(path) if path is not None else envs.GLM_B200_SITE_CONFIG
        if not path.exists():
            if required:
                raise ConfigValidationError(f"site file {path} does not exist")
            return cls()._with_env()
        return cls.parse(path)._with_env()

    @classmethod
    def parse(cls, path: Path) -> "SiteConfig":
        path = Path(path)
        info = os.lstat(path)
        if not stat.S_ISREG(info.st_mode):
            raise ConfigValidationError("the site file must be a regular file (not a symlink)")
        if info.st_uid != os.geteuid() or stat.S_IMODE(info.st_mode) & 0o077:
            raise ConfigValidationError("the site file must be owned by you with mode 0600")
        try:
            doc = tomllib.loads(path.read_text(encoding="utf-8"))
        except tomllib.TOMLDecodeError as exc:
            raise ConfigValidationError(f"the site file is not valid TOML: {exc}") from exc
        return cls.from_document(doc, str(path))

    @classmethod
    def from_document(cls, doc: dict, source: str) -> "SiteConfig":
        """The tables of a site (as parsed TOML, or rebuilt from a resolved site) validated key by key."""
        unknown = set(doc) - set(TABLE_KEYS)
        if unknown:
            raise ConfigValidationError(f"unknown site tables: {sorted(unknown)}")
        for table, keys in TABLE_KEYS.items():
            present = doc.get(table, {})
            if not isinstance(present, dict):
                raise ConfigValidationError(f"[{table}] must be a table")
            extra = set(present) - keys
            if extra:
                raise ConfigValidationError(f"unknown keys in [{table}]: {sorted(extra)}")
        if "paths" not in doc or "run_root" not in doc["paths"]:
            raise ConfigValidationError("[paths] run_root is required")

        def plain(name):
            value = doc["paths"].get(name)
            if value in (None, ""):
                return None
            if type(value) is not str or not os.path.isabs(value) or not _PLAIN.fullmatch(value) or ".." in Path(value).parts:
                raise ConfigValidationError(f"[paths] {name} must be an absolute plain path")
            return Path(value)

        def pin(table, name):
            value = doc.get(table, {}).get(name, "")
            if value != "" and (type(value) is not str or not _HEX64.fullmatch(value)):
                raise ConfigValidationError(f"[{table}] {name} must be 64 lowercase hex digits or empty")
            return value

        def integer(table, name, default, lo, hi):
            value = doc.get(table, {}).get(name, default)
            if type(value) is not int or not lo <= value <= hi:
                raise ConfigValidationError(f"[{table}] {name} must be an integer in [{lo}, {hi}]")
            return value

        gpus = integer("box", "gpus", 8, 1, 8)
        if gpus not in SUPPORTED_GPUS:
            raise ConfigValidationError(f"[box] gpus must be one of {SUPPORTED_GPUS}")
        launch = doc.get("launch", {})
        policy = launch.get("policy", "record")
        if policy not in ("record", "strict"):
            raise ConfigValidationError("[launch] policy must be 'record' or 'strict'")
        branches = launch.get("allowed_branches", ["main", "release/*"])
        if type(branches) is not list or not branches or any(type(b) is not str or not b or not _PLAIN_GLOB.fullmatch(b) for b in branches):
            raise ConfigValidationError("[launch] allowed_branches must be a non-empty list of branch patterns")
        expected_origin = launch.get("expected_origin", "")
        if type(expected_origin) is not str or any(c.isspace() for c in expected_origin):
            raise ConfigValidationError("[launch] expected_origin must be a string without spaces")
        require_pushed = launch.get("require_pushed", False)
        if type(require_pushed) is not bool:
            raise ConfigValidationError("[launch] require_pushed must be true or false")
        return cls(
            gpus=gpus,
            paths=Paths(plain("run_root"), plain("model_path"), plain("packed_path"), plain("state_root")),
            manifest_sha256=pin("checkpoint", "manifest_sha256"),
            source_marker_sha256=pin("checkpoint", "source_marker_sha256"),
            topology_binding_sha256=pin("topology", "binding_sha256"),
            policy=policy,
            allowed_branches=tuple(branches),
            expected_origin=expected_origin,
            require_pushed=require_pushed,
            master_port=integer("launch", "master_port", 29577, 1024, 65535),
            wall_seconds=integer("launch", "wall_seconds", 86400, 1, 30 * 86400),
            serve_port=integer("serve", "port", 8011, 1024, 65535),
            source=source,
        )

    def _with_env(self) -> "SiteConfig":
        from dataclasses import replace

        from glm_tpu_b200 import envs

        paths = self.paths
        if envs.GLM_B200_RUN_ROOT is not None:
            paths = replace(paths, run_root=envs.GLM_B200_RUN_ROOT)
        if envs.GLM_B200_MODEL_PATH is not None:
            paths = replace(paths, model_path=envs.GLM_B200_MODEL_PATH)
        return replace(self, paths=paths)

    # ------------------------------------------------------------------ canonical form
    def resolved(self) -> dict:
        out = asdict(self)
        out["paths"] = {k: (str(v) if v is not None else None) for k, v in out["paths"].items()}
        out["allowed_branches"] = list(self.allowed_branches)
        del out["source"]
        return out

    @classmethod
    def from_staged(cls, path: Path, expected_sha256: str) -> "SiteConfig":
        """The site a controller staged for its workers (``resolved_json`` bytes): refused unless the bytes have the digest the
        controller put on the worker's command line and they parse back to a site with the same canonical form."""
        raw = Path(path).read_bytes()
        if hashlib.sha256(raw).hexdigest() != expected_sha256:
            raise ConfigValidationError("the staged site is not the controller's (digest differs)")
        import json

        try:
            doc = json.loads(raw)
        except ValueError as exc:
            raise ConfigValidationError(f"the staged site is not JSON: {exc}") from exc
        if type(doc) is not dict or set(doc) != set(cls().resolved()) or type(doc["paths"]) is not dict:
            raise ConfigValidationError("the staged site does not have the fields of a resolved site")
        # back into the tables of a site file, so that a staged site passes exactly the checks a site file passes
        tables = {
            "box": {"gpus": doc["gpus"]},
            "paths": {k: v for k, v in doc["paths"].items() if v is not None},
            "checkpoint": {"manifest_sha256": doc["manifest_sha256"], "source_marker_sha256": doc["source_marker_sha256"]},
            "topology": {"binding_sha256": doc["topology_binding_sha256"]},
            "launch": {"policy": doc["policy"], "master_port": doc["master_port"], "wall_seconds": doc["wall_seconds"],
                       "allowed_branches": doc["allowed_branches"], "expected_origin": doc["expected_origin"], "require_pushed": doc["require_pushed"]},
            "serve": {"port": doc["serve_port"]},
        }
        site = cls.from_document(tables, str(path))
        if site.resolved_json() != raw:
            raise ConfigValidationError("the staged site is not in canonical form")
        return site

    @property
    def launch_rules(self):
        from glm_tpu_b200.executor.launch_policy import LaunchRules

        return LaunchRules(self.policy, self.allowed_branches, self.expected_origin, self.require_pushed)

    @property
    def checkpoint_pins(self) -> dict:
        """What a worker hands to the checkpoint loader: an empty pin means unpinned."""
        return {"manifest_sha256": self.manifest_sha256, "source_marker_sha256": self.source_marker_sha256}

    def resolved_json(self) -> bytes:
        return canonical_wire_bytes(self.resolved())

    @property
    def sha256(self) -> str:
        return hashlib.sha256(self.resolved_json()).hexdigest()

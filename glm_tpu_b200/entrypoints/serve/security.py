"""The bearer key of the local ``/v1`` API.

The key lives in one file that only its owner can read.  ``ApiKeyFile.load_or_create`` is the single way in: an existing file is
accepted only if it is a regular, owner-only, non-empty file; a missing one is created exclusively (so two servers starting at once
cannot both mint a key) with 256 bits from the system's random source.  The key is returned to the caller and appears nowhere else:
not in logs, not in reports (the environment registry marks the variable that names the file as secret).

Behaviour parity: reference ``glm_tpu/entrypoints/serve/security.py`` (same messages for a file that is not private or is empty).
"""

from __future__ import annotations

import secrets
import stat
from dataclasses import dataclass
from pathlib import Path

from glm_tpu_b200.utils.io_utils import create_private_exclusive

KEY_BYTES = 32
NOT_PRIVATE = "The API key file must be private (mode 0600)."
EMPTY = "The API key file is empty."


@dataclass(frozen=True)
class ApiKeyFile:
    path: Path

    def _existing(self) -> str | None:
        try:
            facts = self.path.lstat()
        except FileNotFoundError:
            return None
        others_may_touch = stat.S_IMODE(facts.st_mode) & (stat.S_IRWXG | stat.S_IRWXO)
        if not stat.S_ISREG(facts.st_mode) or others_may_touch:  # a link, a directory, or a file open to group / others
            raise ValueError(NOT_PRIVATE)
        key = self.path.read_text(encoding="ascii").strip()
        if not key:
            raise ValueError(EMPTY)
        return key

    def load_or_create(self) -> str:
        key = self._existing()
        if key is not None:
            return key
        key = secrets.token_urlsafe(KEY_BYTES)
        try:
            create_private_exclusive(self.path, (key + "\n").encode("ascii"))
        except FileExistsError:  # another server won the race: its key is the key
            return self._existing() or key
        return key


def api_token(path) -> str:
    """The key in ``path``, minted on first use."""
    return ApiKeyFile(Path(path)).load_or_create()

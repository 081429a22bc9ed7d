"""Documentation stays true to the tree: every repository path and every CLI command the documents mention exists."""

import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
DOCS = [ROOT / "README.md", *sorted((ROOT / "docs").glob("*.md")), *sorted((ROOT / "profiles").glob("*.md"))]
PATH = re.compile(r"`((?:glm_tpu_b200|tests|tools|docs|examples|profiles|csrc)/[A-Za-z0-9_./{},*<>-]+)`")


def _expand(text):
    """`a/{b,c}.py` -> a/b.py, a/c.py; drops wildcard / placeholder paths."""
    m = re.search(r"\{([^{}]*)\}", text)
    if not m:
        return [text]
    return [p for alt in m.group(1).split(",") for p in _expand(text[: m.start()] + alt.strip() + text[m.end():])]


def test_paths_named_in_documents_exist():
    missing = []
    for doc in DOCS:
        for raw in PATH.findall(doc.read_text()):
            for path in _expand(raw):
                if any(ch in path for ch in "*<>"):
                    continue
                path = path.rstrip("/.,:")
                if path.startswith("csrc/"):
                    path = "glm_tpu_b200/" + path
                if not (ROOT / path).exists():
                    missing.append((doc.name, path))
    assert not missing, missing


def test_cli_commands_named_in_documents_parse():
    from glm_tpu_b200.entrypoints.cli.main import build_parser

    parser = build_parser()
    commands = set()
    for doc in DOCS:
        for line in doc.read_text().splitlines():
            m = re.match(r"\s+(?:glm-b200|python -m glm_tpu_b200) ([a-z-]+)", line)
            if m:
                commands.add(m.group(1))
    known = set(parser._subparsers._group_actions[0].choices)
    assert commands and commands <= known, commands - known


def test_example_site_file_parses(tmp_path):
    import os

    from glm_tpu_b200.config.site import SiteConfig

    target = tmp_path / "site.toml"
    target.write_text((ROOT / "examples" / "site.example.toml").read_text())
    os.chmod(target, 0o600)
    site = SiteConfig.parse(target)
    assert site.gpus == 8 and site.policy == "record" and str(site.paths.packed_path) == "/data/GLM-5.3-packed-8"

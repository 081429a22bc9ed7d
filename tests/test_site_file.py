"""The site file, value by value: every key refuses what it cannot mean and names itself when it does; the template that ships
is itself a valid site; the resolved form round-trips through the staged copy a worker reads.

Reference counterpart: ``tests/config/test_site.py``."""

import hashlib
import json
import os
from pathlib import Path

import pytest

from glm_tpu_b200.config.site import SUPPORTED_GPUS, TABLE_KEYS, SiteConfig
from glm_tpu_b200.exceptions import ConfigValidationError

ROOT = Path(__file__).resolve().parents[1]
BASE = {
    "box": {"gpus": 8},
    "paths": {"run_root": "/srv/runs", "model_path": "/data/GLM-5.3", "packed_path": "/data/packed-8", "state_root": "/srv/state"},
    "checkpoint": {"manifest_sha256": "a" * 64, "source_marker_sha256": ""},
    "topology": {"binding_sha256": "b" * 64},
    "launch": {"policy": "strict", "allowed_branches": ["main", "release/*"], "expected_origin": "https://example.org/team/engine",
               "require_pushed": True, "master_port": 29600, "wall_seconds": 3600},
    "serve": {"port": 8011},
}


def toml(doc: dict) -> str:
    def value(v):
        if isinstance(v, bool):
            return "true" if v else "false"
        if isinstance(v, (int, float)):
            return repr(v)
        if isinstance(v, list):
            return "[" + ", ".join(value(x) for x in v) + "]"
        return json.dumps(v)

    return "".join(f"[{table}]\n" + "".join(f"{k} = {value(v)}\n" for k, v in keys.items()) for table, keys in doc.items())


def write(tmp_path, text, mode=0o600, name="site.toml"):
    path = tmp_path / name
    path.write_text(text)
    os.chmod(path, mode)
    return path


def changed(table, key, value):
    doc = {t: dict(k) for t, k in BASE.items()}
    doc[table][key] = value
    return doc


def test_the_full_file_parses_to_what_it_says(tmp_path):
    site = SiteConfig.parse(write(tmp_path, toml(BASE)))
    assert site.gpus == 8 and site.paths.run_root == Path("/srv/runs") and site.paths.state_root == Path("/srv/state")
    assert site.manifest_sha256 == "a" * 64 and site.source_marker_sha256 == "" and site.topology_binding_sha256 == "b" * 64
    assert site.policy == "strict" and site.allowed_branches == ("main", "release/*") and site.require_pushed is True
    assert site.master_port == 29600 and site.wall_seconds == 3600 and site.serve_port == 8011 and site.source.endswith("site.toml")
    rules = site.launch_rules
    assert (rules.policy, rules.allowed_branches, rules.expected_origin, rules.require_pushed) == ("strict", ("main", "release/*"), "https://example.org/team/engine", True)
    assert site.checkpoint_pins == {"manifest_sha256": "a" * 64, "source_marker_sha256": ""}
    assert {t for t in TABLE_KEYS} == set(BASE) and all(set(BASE[t]) == TABLE_KEYS[t] for t in BASE)  # this test covers every key


def test_defaults_fill_what_a_minimal_file_leaves_out(tmp_path):
    site = SiteConfig.parse(write(tmp_path, '[paths]\nrun_root = "/srv/runs"\n'))
    assert site.gpus == 8 and site.policy == "record" and site.manifest_sha256 == "" and site.paths.model_path is None
    assert site.master_port == 29577 and site.wall_seconds == 86400 and site.serve_port == 8011 and site.require_pushed is False
    empty = SiteConfig.parse(write(tmp_path, '[paths]\nrun_root = "/srv/runs"\nmodel_path = ""\n', name="b.toml"))
    assert empty.paths.model_path is None  # an empty path is "not set", like an empty pin


def test_the_shipped_template_is_a_valid_site(tmp_path):
    text = (ROOT / "examples" / "site.example.toml").read_text()
    site = SiteConfig.parse(write(tmp_path, text))
    assert site.gpus == 8 and site.policy == "record" and site.manifest_sha256 == "" and site.serve_port == 8011
    import tomllib

    doc = tomllib.loads(text)
    assert {t: set(k) for t, k in doc.items()} == TABLE_KEYS  # the template shows every key there is, and no other


@pytest.mark.parametrize("table,key,value,match", [
    ("box", "gpus", "8", r"\[box\] gpus must be an integer"),
    ("box", "gpus", 8.0, r"\[box\] gpus must be an integer"),
    ("box", "gpus", True, r"\[box\] gpus must be an integer"),
    ("box", "gpus", 0, r"\[box\] gpus"),
    ("box", "gpus", 16, r"\[box\] gpus"),
    ("box", "gpus", 6, r"\[box\] gpus must be one of"),
    ("paths", "run_root", 7, r"\[paths\] run_root must be an absolute plain path"),
    ("paths", "run_root", "runs", r"\[paths\] run_root"),
    ("paths", "model_path", "/data/with space", r"\[paths\] model_path"),
    ("paths", "model_path", "/data/$HOME", r"\[paths\] model_path"),
    ("paths", "packed_path", "/data/a/../b", r"\[paths\] packed_path"),
    ("paths", "state_root", "~/state", r"\[paths\] state_root"),
    ("checkpoint", "manifest_sha256", "a" * 63, r"\[checkpoint\] manifest_sha256 must be 64 lowercase hex"),
    ("checkpoint", "manifest_sha256", "g" * 64, r"\[checkpoint\] manifest_sha256"),
    ("checkpoint", "source_marker_sha256", 5, r"\[checkpoint\] source_marker_sha256"),
    ("topology", "binding_sha256", "B" * 64, r"\[topology\] binding_sha256"),
    ("launch", "policy", "Strict", r"\[launch\] policy"),
    ("launch", "policy", 1, r"\[launch\] policy"),
    ("launch", "allowed_branches", [], r"\[launch\] allowed_branches"),
    ("launch", "allowed_branches", "main", r"\[launch\] allowed_branches"),
    ("launch", "allowed_branches", ["main", ""], r"\[launch\] allowed_branches"),
    ("launch", "allowed_branches", ["main", 3], r"\[launch\] allowed_branches"),
    ("launch", "allowed_branches", ["ma in"], r"\[launch\] allowed_branches"),
    ("launch", "expected_origin", "https://example.org/a b", r"\[launch\] expected_origin"),
    ("launch", "expected_origin", 3, r"\[launch\] expected_origin"),
    ("launch", "require_pushed", "yes", r"\[launch\] require_pushed"),
    ("launch", "require_pushed", 1, r"\[launch\] require_pushed"),
    ("launch", "master_port", 80, r"\[launch\] master_port must be an integer in \[1024, 65535\]"),
    ("launch", "master_port", 70000, r"\[launch\] master_port"),
    ("launch", "master_port", "29577", r"\[launch\] master_port"),
    ("launch", "wall_seconds", 0, r"\[launch\] wall_seconds"),
    ("launch", "wall_seconds", 31 * 86400, r"\[launch\] wall_seconds"),
    ("serve", "port", 1023, r"\[serve\] port"),
    ("serve", "port", 8011.5, r"\[serve\] port"),
])
def test_every_key_refuses_what_it_cannot_mean_and_names_itself(tmp_path, table, key, value, match):
    with pytest.raises(ConfigValidationError, match=match):
        SiteConfig.parse(write(tmp_path, toml(changed(table, key, value))))


@pytest.mark.parametrize("gpus", SUPPORTED_GPUS)
def test_supported_box_shapes(tmp_path, gpus):
    assert SiteConfig.parse(write(tmp_path, toml(changed("box", "gpus", gpus)))).gpus == gpus


def test_shape_of_the_document(tmp_path):
    with pytest.raises(ConfigValidationError, match=r"\[box\] must be a table"):
        SiteConfig.parse(write(tmp_path, 'box = 3\n[paths]\nrun_root = "/srv/runs"\n'))
    with pytest.raises(ConfigValidationError, match="unknown site tables: \\['fleet'\\]"):
        SiteConfig.parse(write(tmp_path, toml(BASE) + '[fleet]\nhosts = ["a"]\n'))
    with pytest.raises(ConfigValidationError, match=r"unknown keys in \[paths\]: \['cache'\]"):
        SiteConfig.parse(write(tmp_path, toml(changed("paths", "cache", "/x"))))
    with pytest.raises(ConfigValidationError, match="run_root is required"):
        SiteConfig.parse(write(tmp_path, '[paths]\nmodel_path = "/data/m"\n'))
    with pytest.raises(ConfigValidationError, match="not valid TOML"):
        SiteConfig.parse(write(tmp_path, '[paths]\nrun_root = "/srv/runs"\nrun_root = "/srv/other"\n'))  # a key given twice


@pytest.mark.parametrize("mode,ok", [(0o600, True), (0o400, True), (0o640, False), (0o604, False), (0o660, False), (0o666, False), (0o700, True)])
def test_the_file_is_closed_to_everyone_else(tmp_path, mode, ok):
    path = write(tmp_path, toml(BASE), mode)
    if ok:
        SiteConfig.parse(path)
    else:
        with pytest.raises(ConfigValidationError, match="owned by you with mode 0600"):
            SiteConfig.parse(path)


def test_links_and_directories_are_not_site_files(tmp_path):
    real = write(tmp_path, toml(BASE))
    (tmp_path / "link.toml").symlink_to(real)
    with pytest.raises(ConfigValidationError, match="regular file"):
        SiteConfig.parse(tmp_path / "link.toml")
    (tmp_path / "dir.toml").mkdir()
    with pytest.raises(ConfigValidationError, match="regular file"):
        SiteConfig.parse(tmp_path / "dir.toml")
    with pytest.raises(FileNotFoundError):
        SiteConfig.parse(tmp_path / "absent.toml")


def test_where_the_file_is_looked_for(tmp_path, monkeypatch):
    for name in ("GLM_B200_SITE_CONFIG", "GLM_B200_CONFIG_ROOT", "GLM_B200_RUN_ROOT", "GLM_B200_MODEL_PATH"):
        monkeypatch.delenv(name, raising=False)
    root = tmp_path / "config"
    root.mkdir()
    write(root, toml(changed("box", "gpus", 2)))
    monkeypatch.setenv("GLM_B200_CONFIG_ROOT", str(root))
    assert SiteConfig.load().gpus == 2  # <config root>/site.toml
    other = write(tmp_path, toml(changed("box", "gpus", 4)), name="other.toml")
    monkeypatch.setenv("GLM_B200_SITE_CONFIG", str(other))
    assert SiteConfig.load().gpus == 4  # an explicit file wins over the config root
    assert SiteConfig.load(root / "site.toml").gpus == 2  # an argument wins over both
    monkeypatch.setenv("GLM_B200_SITE_CONFIG", str(tmp_path / "nothing.toml"))
    assert SiteConfig.load().source == "<defaults>"
    with pytest.raises(ConfigValidationError, match="does not exist"):
        SiteConfig.load(required=True)
    monkeypatch.setenv("GLM_B200_MODEL_PATH", "/elsewhere/model")
    assert SiteConfig.load(other).paths.model_path == Path("/elsewhere/model") and SiteConfig.load(other).paths.run_root == Path("/srv/runs")
    assert SiteConfig.parse(other).paths.model_path == Path("/data/GLM-5.3")  # parse() is the file alone


def test_resolved_form_is_canonical_and_round_trips_through_the_staged_copy(tmp_path):
    site = SiteConfig.parse(write(tmp_path, toml(BASE)))
    raw = site.resolved_json()
    doc = json.loads(raw)
    assert "source" not in doc and doc["paths"]["run_root"] == "/srv/runs" and doc["allowed_branches"] == ["main", "release/*"]
    assert raw == json.dumps(doc, sort_keys=True, separators=(",", ":"), ensure_ascii=False).encode() and site.sha256 == hashlib.sha256(raw).hexdigest()
    reordered = {t: dict(reversed(list(BASE[t].items()))) for t in reversed(list(BASE))}
    assert SiteConfig.parse(write(tmp_path, toml(reordered), name="r.toml")).sha256 == site.sha256  # the order in the file means nothing
    assert SiteConfig.parse(write(tmp_path, toml(changed("serve", "port", 8012)), name="p.toml")).sha256 != site.sha256

    staged = tmp_path / "site.resolved.json"
    staged.write_bytes(raw)
    back = SiteConfig.from_staged(staged, site.sha256)
    assert back.resolved() == site.resolved() and back.sha256 == site.sha256
    with pytest.raises(ConfigValidationError, match="digest differs"):
        SiteConfig.from_staged(staged, "0" * 64)
    pretty = json.dumps(doc, indent=1).encode()
    staged.write_bytes(pretty)
    with pytest.raises(ConfigValidationError, match="not in canonical form"):
        SiteConfig.from_staged(staged, hashlib.sha256(pretty).hexdigest())
    partial = json.dumps({k: v for k, v in doc.items() if k != "paths"}, sort_keys=True, separators=(",", ":")).encode()
    staged.write_bytes(partial)
    with pytest.raises(ConfigValidationError, match="fields of a resolved site"):
        SiteConfig.from_staged(staged, hashlib.sha256(partial).hexdigest())
    extra = json.dumps(dict(doc, surprise=1), sort_keys=True, separators=(",", ":")).encode()
    staged.write_bytes(extra)
    with pytest.raises(ConfigValidationError, match="fields of a resolved site"):
        SiteConfig.from_staged(staged, hashlib.sha256(extra).hexdigest())


def test_a_staged_site_passes_the_checks_of_a_site_file(tmp_path):
    """The digest binds the staged bytes to the controller; the values are still checked like a file's, so a controller that went
    wrong cannot hand its workers a site no file could express."""
    site = SiteConfig.parse(write(tmp_path, toml(BASE)))
    doc = json.loads(site.resolved_json())
    staged = tmp_path / "site.resolved.json"

    def stage(value) -> str:
        raw = value if isinstance(value, bytes) else json.dumps(value, sort_keys=True, separators=(",", ":")).encode()
        staged.write_bytes(raw)
        return hashlib.sha256(raw).hexdigest()

    for edit, match in ((dict(doc, gpus=3), r"\[box\] gpus"), (dict(doc, manifest_sha256="xyz"), "manifest_sha256"),
                        (dict(doc, policy="lenient"), "policy"), (dict(doc, serve_port=80), r"\[serve\] port"),
                        (dict(doc, paths=dict(doc["paths"], run_root="runs")), "run_root"),
                        (dict(doc, paths=dict(doc["paths"], run_root=None)), "run_root is required"),
                        (dict(doc, paths=dict(doc["paths"], tmp="/x")), r"unknown keys in \[paths\]"),
                        (dict(doc, allowed_branches=[]), "allowed_branches"), (dict(doc, require_pushed="no"), "require_pushed")):
        with pytest.raises(ConfigValidationError, match=match):
            SiteConfig.from_staged(staged, stage(edit))
    for raw, match in ((b"{not json", "not JSON"), (b"[]", "fields of a resolved site"), (b'"site"', "fields of a resolved site"),
                       (json.dumps(dict(doc, paths="/srv")).encode(), "fields of a resolved site")):
        with pytest.raises(ConfigValidationError, match=match):
            SiteConfig.from_staged(staged, stage(raw))
    assert SiteConfig.from_staged(staged, stage(site.resolved_json())).sha256 == site.sha256
    unpinned = SiteConfig.parse(write(tmp_path, '[paths]\nrun_root = "/srv/runs"\n', name="min.toml"))
    assert SiteConfig.from_staged(staged, stage(unpinned.resolved_json())).paths.model_path is None


def test_serve_takes_what_the_command_line_leaves_open_from_the_site(tmp_path, monkeypatch):
    from glm_tpu_b200.entrypoints.cli import main as cli

    for name in ("GLM_B200_SITE_CONFIG", "GLM_B200_CONFIG_ROOT", "GLM_B200_RUN_ROOT", "GLM_B200_MODEL_PATH"):
        monkeypatch.delenv(name, raising=False)
    site = write(tmp_path, toml(changed("serve", "port", 8123)))
    parse = cli.build_parser().parse_args
    assert cli.serve_arguments(parse(["serve", "--run", "/r", "--site", str(site)])) == ["--run", "/r", "--state", "/srv/state", "--port", "8123"]
    explicit = parse(["serve", "--run", "/r", "--state", "/elsewhere", "--port", "9000", "--no-api", "--site", str(site)])
    assert cli.serve_arguments(explicit) == ["--run", "/r", "--state", "/elsewhere", "--port", "9000", "--no-api"]  # the command line wins
    monkeypatch.setenv("GLM_B200_SITE_CONFIG", str(tmp_path / "absent.toml"))
    assert cli.serve_arguments(parse(["serve", "--run", "/r", "--state", "/s"])) == ["--run", "/r", "--state", "/s", "--port", "8011"]
    with pytest.raises(ConfigValidationError, match="--state or \\[paths\\] state_root"):
        cli.serve_arguments(parse(["serve", "--run", "/r"]))

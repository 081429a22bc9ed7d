"""``collect-env`` / ``doctor``: declared requirements against installed distributions, and the profile checks, with fakes for both.

Reference counterpart: ``tests/entrypoints/cli/test_collect_env.py`` (declared pins vs installed versions, per profile)."""

import json
import subprocess
import sys
from importlib import metadata

import pytest

from glm_tpu_b200.entrypoints.cli import collect_env

PROJECT = """
[project]
name = "glm-tpu-b200"
dependencies = ["torch>=2.4", "numpy"]
[project.optional-dependencies]
dev = ["pytest"]
tokenizer = ["tokenizers==0.22.2", "jinja2"]
"""


def fake_installed(table):
    def version(name):
        if name not in table:
            raise metadata.PackageNotFoundError(name)
        return table[name]

    return version


def test_declared_packages_from_a_checkout(tmp_path):
    path = tmp_path / "pyproject.toml"
    path.write_text(PROJECT)
    groups = collect_env.declared_packages(path)
    assert groups == {"core": {"torch": (">=", "2.4"), "numpy": ("", "")}, "dev": {"pytest": ("", "")},
                      "tokenizer": {"tokenizers": ("==", "0.22.2"), "jinja2": ("", "")}}
    # the repository's own file parses and names the packages the report is about
    own = collect_env.declared_packages()
    assert "torch" in own["core"] and set(collect_env.PROFILE_GROUPS["dev"]) <= set(own)


@pytest.mark.parametrize("text,match", [
    ('[project]\nname = "something-else"\ndependencies = []\n', "does not declare"),
    ('[project]\nname = "glm-tpu-b200"\ndependencies = ["torch~=2.4"]\n', "unsupported requirement"),
    ('[project]\nname = "glm-tpu-b200"\ndependencies = ["torch>=2.4,<3"]\n', "unsupported requirement"),
])
def test_declared_packages_refuse_what_they_cannot_check(tmp_path, text, match):
    path = tmp_path / "pyproject.toml"
    path.write_text(text)
    with pytest.raises(ValueError, match=match):
        collect_env.declared_packages(path)


def test_declared_packages_from_distribution_metadata(tmp_path):
    class Dist:
        requires = ["torch>=2.4", "numpy", 'pytest; extra == "dev"', "tokenizers==0.22.2; extra == 'tokenizer'"]

    groups = collect_env.declared_packages(tmp_path / "absent.toml", distribution=Dist())
    assert groups == {"core": {"torch": (">=", "2.4"), "numpy": ("", "")}, "dev": {"pytest": ("", "")}, "tokenizer": {"tokenizers": ("==", "0.22.2")}}

    class Odd:
        requires = ['torch>=2.4; python_version < "3.13"']

    with pytest.raises(ValueError, match="unsupported requirement marker"):
        collect_env.declared_packages(tmp_path / "absent.toml", distribution=Odd())


def test_package_rows_and_profiles(tmp_path):
    path = tmp_path / "pyproject.toml"
    path.write_text(PROJECT)
    groups = collect_env.declared_packages(path)
    have = fake_installed({"torch": "2.11.0+cu128", "numpy": "2.3.5", "tokenizers": "0.22.2+local"})
    rows = {r["package"]: r for r in collect_env.package_rows("dev", groups, have)}
    assert rows["torch"]["ok"] and rows["torch"]["required"] and rows["torch"]["declared"] == ">=2.4"
    assert rows["numpy"]["ok"] and rows["numpy"]["declared"] == "any"
    assert not rows["pytest"]["ok"] and rows["pytest"]["required"] and rows["pytest"]["installed"] is None  # dev needs the dev group
    assert rows["tokenizers"]["ok"] and not rows["tokenizers"]["required"]  # a pin matches the same release with a local label
    assert not rows["jinja2"]["ok"] and not rows["jinja2"]["required"]  # missing, but no profile needs it: listed only
    serve = {r["package"]: r for r in collect_env.package_rows("serve", groups, have)}
    assert not serve["pytest"]["required"]
    old = {r["package"]: r for r in collect_env.package_rows("serve", groups, fake_installed({"torch": "2.3.1", "numpy": "2.0", "tokenizers": "0.21.0"}))}
    assert not old["torch"]["ok"] and not old["tokenizers"]["ok"]


def base_info(**over):
    info = {"python": "3.12.3", "torch": "2.11.0+cu128", "cuda_toolkit": "12.9", "gpus": [{"sm": "10.0"}], "library_built": True,
            "peer_access": True, "packages": []}
    info.update(over)
    return info


def test_check_profiles():
    assert collect_env.check(base_info(), "serve") == []
    assert collect_env.check(base_info(gpus=[], library_built=False), "dev") == []  # the toolchain is enough for dev
    problems = collect_env.check(base_info(gpus=[], library_built=False), "serve")
    assert any("no CUDA GPU" in p for p in problems) and any("not built" in p for p in problems)
    assert any("sm_100a" in p for p in collect_env.check(base_info(gpus=[{"sm": "9.0"}]), "serve"))
    assert any("peer access" in p for p in collect_env.check(base_info(peer_access=False), "serve"))
    assert any("toolkit" in p for p in collect_env.check(base_info(cuda_toolkit="12.4"), "dev"))
    assert any("toolkit" in p for p in collect_env.check(base_info(cuda_toolkit=None), "dev"))
    assert any("torch" in p for p in collect_env.check(base_info(torch=None), "dev"))
    assert any("older" in p for p in collect_env.check(base_info(python="3.9.18"), "dev"))
    row = {"group": "core", "package": "torch", "declared": ">=2.4", "installed": None, "ok": False, "required": True}
    assert any("torch >=2.4 is declared (core), installed: nothing" in p for p in collect_env.check(base_info(packages=[row]), "dev"))
    assert collect_env.check(base_info(packages=[dict(row, required=False)]), "dev") == []
    assert "nothing declares" in collect_env.check(base_info(declared_error="nothing declares the requirements"), "dev")[0]


def test_version_tuple():
    assert collect_env._version_tuple("2.11.0+cu128") == (2, 11, 0)
    assert collect_env._version_tuple("12.9") == (12, 9)
    assert collect_env._version_tuple("3.13.0rc1") == (3, 13)
    assert collect_env._version_tuple("") == ()


@pytest.mark.parametrize("command", ["collect-env", "doctor"])
def test_command_prints_one_json_report(command):
    out = subprocess.run([sys.executable, "-m", "glm_tpu_b200", command, "--profile", "dev"], capture_output=True, text=True, timeout=300)
    report = json.loads(out.stdout)
    assert report["profile"] == "dev" and isinstance(report["problems"], list) and (out.returncode == 0) == report["ok"]
    assert {r["package"] for r in report["info"]["packages"]} >= {"torch", "numpy", "pytest"}
    assert report["info"]["env"]["GLM_B200_API_KEY_FILE"] in ("<unset>", "<set>")  # secrets never appear

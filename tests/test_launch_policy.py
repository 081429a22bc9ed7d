"""Launch policy: every rule on made-up identities (order: clean, HEAD, branch, origin, pushed), the spelling of origins, the
question put to origin, and the identity of real checkouts in odd states (no repository, detached, untracked file).

Reference counterpart: ``tests/executor/test_launch_policy.py``."""

import subprocess
from pathlib import Path

import pytest

from glm_tpu_b200.exceptions import ConfigValidationError
from glm_tpu_b200.executor import launch_policy
from glm_tpu_b200.executor.launch_policy import LaunchRules, check, normalize_origin

COMMIT = "0123456789abcdef0123456789abcdef01234567"


def identity(**over):
    base = {"repo": "/srv/checkout", "git": True, "commit": COMMIT, "branch": "main", "clean": True, "dirty_files": 0,
            "origin": "git@example.org:team/engine.git"}
    base.update(over)
    return base


def refuses(ident, rules, match, **kw):
    with pytest.raises(ConfigValidationError, match=match):
        check(ident, rules, **kw)


def test_record_applies_no_rule_and_unknown_policies_are_refused():
    check(identity(git=False, clean=False, commit=None, branch=None, origin=None), "record")
    check(identity(clean=False), LaunchRules("record", ("nothing",), "elsewhere", True))
    refuses(identity(), "lenient", "'record' or 'strict'")
    refuses(identity(), LaunchRules(policy=""), "'record' or 'strict'")


def test_strict_rules_fail_in_their_order():
    """An identity that breaks every rule is refused for the first one; fixing the rules one by one walks through the order."""
    rules = LaunchRules("strict", ("main", "release/*"), "https://example.org/team/engine", True)
    asked = []

    def head(repo, branch):
        asked.append((str(repo), branch))
        return "f" * 40

    broken = identity(git=False, clean=False, commit="HEAD", branch="topic", origin="git@example.org:other/thing.git")
    refuses(broken, rules, "needs a git checkout", remote_head=head)
    broken["git"] = True
    refuses(broken, rules, "uncommitted changes", remote_head=head)
    broken["clean"] = True
    refuses(broken, rules, "not a 40-hex commit", remote_head=head)
    broken["commit"] = COMMIT
    refuses(broken, rules, "'topic' is not allowed", remote_head=head)
    broken["branch"] = "release/2026.11"
    refuses(broken, rules, "origin differs", remote_head=head)
    broken["origin"] = "ssh://git@example.org/team/engine.git"
    assert asked == []  # origin is asked only when everything before it passed
    refuses(broken, rules, "must be pushed.*refs/heads/release/2026.11", remote_head=head)
    assert asked == [("/srv/checkout", "release/2026.11")]
    check(broken, rules, remote_head=lambda repo, branch: COMMIT)


@pytest.mark.parametrize("over,match", [
    ({"clean": None}, "uncommitted changes"),  # git status could not be asked: not known to be clean
    ({"commit": None}, "not a 40-hex commit"),
    ({"commit": COMMIT.upper()}, "not a 40-hex commit"),
    ({"commit": COMMIT[:39]}, "not a 40-hex commit"),
    ({"branch": None}, "detached HEAD"),
    ({"branch": ""}, "detached HEAD"),
    ({"branch": "HEAD"}, "detached HEAD"),
    ({"branch": "Main"}, "not allowed"),  # patterns are case-sensitive
    ({"branch": "release"}, "not allowed"),
    ({"branch": "xrelease/1"}, "not allowed"),
])
def test_strict_refusals_without_origin_rules(over, match):
    refuses(identity(**over), LaunchRules("strict"), match)


def test_strict_without_origin_rules_never_asks_origin():
    def never(repo, branch):
        raise AssertionError("origin was asked")

    check(identity(origin=None), LaunchRules("strict"), remote_head=never)
    check(identity(branch="release/7", origin=None), "strict", remote_head=never)


def test_origin_rules_need_an_origin():
    refuses(identity(origin=None), LaunchRules("strict", expected_origin="example.org/team/engine"), "no 'origin' remote")
    refuses(identity(origin=""), LaunchRules("strict", require_pushed=True), "no 'origin' remote")
    refuses(identity(), LaunchRules("strict", require_pushed=True), "must be pushed", remote_head=lambda repo, branch: None)


@pytest.mark.parametrize("a,b", [
    ("git@example.org:team/engine.git", "https://example.org/team/engine"),
    ("ssh://git@Example.ORG/team/engine.git/", "example.org:team/engine"),
    ("https://user:secret@example.org:443/team/engine.git", "git://example.org:9418/team/engine"),
    ("ssh://example.org:22/team/engine", "http://example.org:80/team/engine///"),
])
def test_spellings_of_one_remote_are_equal(a, b, tmp_path):
    assert normalize_origin(a, tmp_path) == normalize_origin(b, tmp_path) == ("remote", "example.org/team/engine")


@pytest.mark.parametrize("a,b", [
    ("git@example.org:team/engine.git", "git@example.org:team/engine2.git"),
    ("git@example.org:team/engine.git", "git@example.org:Team/engine.git"),  # only the host is case-insensitive
    ("git@example.org:team/engine.git", "git@example.com:team/engine.git"),
    ("https://example.org:8443/team/engine", "https://example.org/team/engine"),  # a non-default port is part of the name
    ("https://example.org/team/engine", "/example.org/team/engine"),
])
def test_different_origins_stay_different(a, b, tmp_path):
    assert normalize_origin(a, tmp_path) != normalize_origin(b, tmp_path)


def test_local_origins(tmp_path):
    bare = tmp_path / "bare.git"
    bare.mkdir()
    assert normalize_origin(str(bare)) == ("local", str(bare))
    assert normalize_origin("file://" + str(bare)) == ("local", str(bare))
    assert normalize_origin("bare.git", tmp_path) == ("local", str(bare))
    assert normalize_origin("sub/../bare.git/", tmp_path) == ("local", str(bare))
    # a path never passes for a remote of the same spelling, and a host:path spelling that exists on disk is a path
    assert normalize_origin("example.org/team/engine", tmp_path)[0] == "local"
    (tmp_path / "host:dir").mkdir()
    assert normalize_origin(str(tmp_path / "host:dir"))[0] == "local"
    rules = LaunchRules("strict", expected_origin="example.org/team/engine")
    refuses(identity(repo=str(tmp_path)), rules, "origin differs")


def test_origin_head_reads_exactly_one_matching_ref(monkeypatch):
    answers = {}
    monkeypatch.setattr(launch_policy, "_git", lambda repo, *args, timeout=20.0: answers.get(args[-1]))
    answers["refs/heads/main"] = f"{COMMIT}\trefs/heads/main"
    assert launch_policy.origin_head(Path("/x"), "main") == COMMIT
    answers["refs/heads/main"] = f"{COMMIT}\trefs/heads/main\n{'a' * 40}\trefs/heads/main"
    assert launch_policy.origin_head(Path("/x"), "main") is None  # two answers are no answer
    answers["refs/heads/main"] = f"{COMMIT}\trefs/heads/maintenance"
    assert launch_policy.origin_head(Path("/x"), "main") is None  # a ref that only starts the same
    answers["refs/heads/main"] = "garbage without a tab"
    assert launch_policy.origin_head(Path("/x"), "main") is None
    assert launch_policy.origin_head(Path("/x"), "absent") is None  # git failed or timed out


def git(repo, *args):
    env = {"GIT_AUTHOR_NAME": "t", "GIT_AUTHOR_EMAIL": "t@example.org", "GIT_COMMITTER_NAME": "t", "GIT_COMMITTER_EMAIL": "t@example.org",
           "GIT_CONFIG_GLOBAL": "/dev/null", "GIT_CONFIG_SYSTEM": "/dev/null", "PATH": "/usr/bin:/bin:/usr/local/bin", "HOME": str(repo)}
    done = subprocess.run(["git", "-C", str(repo), *args], capture_output=True, text=True, env=env, timeout=60)
    assert done.returncode == 0, done.stderr
    return done.stdout.strip()


def test_identity_of_real_checkouts(tmp_path):
    nothing = tmp_path / "plain"
    nothing.mkdir()
    ident = launch_policy.source_identity(nothing)
    assert ident["git"] is False and ident["commit"] is None and ident["clean"] is None and ident["origin"] is None
    refuses(ident, "strict", "needs a git checkout")

    work = tmp_path / "work"
    work.mkdir()
    git(work, "init", "-q", "-b", "main")
    (work / "a.txt").write_text("a\n")
    git(work, "add", "a.txt")
    git(work, "commit", "-q", "-m", "first")
    ident = launch_policy.source_identity(work)
    assert ident["git"] and ident["clean"] is True and ident["branch"] == "main" and ident["origin"] is None and ident["dirty_files"] == 0
    assert ident["commit"] == git(work, "rev-parse", "HEAD")
    check(ident, "strict")

    (work / "untracked.txt").write_text("x\n")
    ident = launch_policy.source_identity(work)
    assert ident["clean"] is False and ident["dirty_files"] == 1
    refuses(ident, "strict", "untracked files included")
    (work / "untracked.txt").unlink()

    (work / "a.txt").write_text("changed\n")
    git(work, "add", "a.txt")  # staged counts as well
    assert launch_policy.source_identity(work)["clean"] is False
    git(work, "commit", "-q", "-m", "second")

    git(work, "checkout", "-q", "--detach", "HEAD")
    ident = launch_policy.source_identity(work)
    assert ident["branch"] is None and ident["clean"] is True
    refuses(ident, "strict", "detached HEAD")

    git(work, "checkout", "-q", "-b", "topic/x")
    refuses(launch_policy.source_identity(work), "strict", "'topic/x' is not allowed")
    check(launch_policy.source_identity(work), LaunchRules("strict", ("topic/*",)))
    assert launch_policy.origin_head(work, "main") is None  # no origin to ask

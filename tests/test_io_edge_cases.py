"""File discipline at its edges: names taken by things that are not files, FIFOs, links at every level, a file that grows while it
is read, payloads that are not JSON.

Reference counterpart: ``tests/utils_/test_io_utils.py``."""

import json
import os
import stat
import threading

import pytest

from glm_tpu_b200.utils import io_utils


def test_collected_name_taken_by_a_directory_or_a_link(tmp_path):
    divergent: list[str] = []
    (tmp_path / "record.json").mkdir()  # the name is taken by something that is not a file
    io_utils.write_collected(tmp_path, "record.json", b'{"a": 1}', divergent)
    assert divergent == ["record.json"] and (tmp_path / "final" / "record.json").read_bytes() == b'{"a": 1}'
    outside = tmp_path / "outside.json"
    outside.write_bytes(b'{"b": 2}')
    (tmp_path / "linked.json").symlink_to(outside)  # a planted link with the very same content still does not count as filed
    io_utils.write_collected(tmp_path, "linked.json", b'{"b": 2}', divergent)
    assert divergent == ["record.json", "linked.json"] and outside.read_bytes() == b'{"b": 2}'
    assert (tmp_path / "final" / "linked.json").read_bytes() == b'{"b": 2}'
    assert stat.S_IMODE((tmp_path / "final").stat().st_mode) == 0o700


def test_collected_payloads_that_are_not_json(tmp_path):
    divergent: list[str] = []
    io_utils.write_collected(tmp_path, "worker.log", b"line one\n", divergent)
    io_utils.write_collected(tmp_path, "worker.log", b"line one\n", divergent)  # identical bytes: nothing to keep
    assert divergent == []
    io_utils.write_collected(tmp_path, "worker.log", b"line one\nline two\n", divergent)
    assert divergent == ["worker.log"] and (tmp_path / "worker.log").read_bytes() == b"line one\n"
    io_utils.write_collected(tmp_path, "mixed", b'{"a": 1}', divergent)
    io_utils.write_collected(tmp_path, "mixed", b"not json", divergent)  # JSON against text: different
    assert divergent == ["worker.log", "mixed"]
    io_utils.write_collected(tmp_path, "numbers", b"1.0", divergent)
    io_utils.write_collected(tmp_path, "numbers", b"1", divergent)  # equal as JSON values
    assert divergent == ["worker.log", "mixed"]


def test_many_differing_arrivals_each_get_a_place(tmp_path):
    divergent: list[str] = []
    for i in range(5):
        io_utils.write_collected(tmp_path, "r.json", json.dumps({"i": i}).encode(), divergent)
    assert divergent == ["r.json"]
    kept = sorted(p.name for p in (tmp_path / "final").iterdir())
    assert kept == ["r.json", "r.json.1", "r.json.2", "r.json.3"]
    assert [json.loads((tmp_path / "final" / n).read_text())["i"] for n in kept] == [1, 2, 3, 4]
    assert json.loads((tmp_path / "r.json").read_text()) == {"i": 0}


def test_a_fifo_is_refused_without_blocking(tmp_path):
    fifo = tmp_path / "pipe"
    os.mkfifo(fifo)
    done = []

    def read():
        try:
            io_utils.read_bounded(fifo, 100)
        except ValueError as exc:
            done.append(str(exc))

    worker = threading.Thread(target=read, daemon=True)
    worker.start()
    worker.join(5)
    assert done == ["input is not a bounded regular file"]  # opened O_NONBLOCK, refused on its type: nobody had to write to it


def test_a_link_is_refused_wherever_it_sits(tmp_path, monkeypatch):
    real = tmp_path / "real"
    real.mkdir()
    (real / "f").write_bytes(b"data")
    (tmp_path / "to_file").symlink_to(real / "f")
    (tmp_path / "to_dir").symlink_to(real)
    (real / "inner").symlink_to(real / "f")
    for path in (tmp_path / "to_file", tmp_path / "to_dir" / "f", real / "inner"):
        with pytest.raises(ValueError, match="symlink"):
            io_utils.read_bounded(path, 100)
        with pytest.raises(ValueError, match="symlink"):
            io_utils.plain_path(path)
        with pytest.raises(ValueError, match="symlink"):
            io_utils.require_private(path)
    assert io_utils.plain_path(real / "f") == real / "f"
    monkeypatch.chdir(real)
    assert io_utils.plain_path("f") == real / "f"  # made absolute
    with pytest.raises(FileNotFoundError):
        io_utils.read_bounded(real / "absent", 10)


def test_a_file_that_grows_past_its_cap_while_it_is_read(tmp_path, monkeypatch):
    path = tmp_path / "growing"
    path.write_bytes(b"x" * 8)
    real_read = os.read

    def read_and_append(fd, n):
        with open(path, "ab") as extra:  # the writer keeps appending between our size check and our read
            extra.write(b"y" * 8)
        return real_read(fd, n)

    monkeypatch.setattr(os, "read", read_and_append)
    with pytest.raises(ValueError, match="changed beyond its byte cap"):
        io_utils.read_bounded(path, 10)
    monkeypatch.undo()
    assert io_utils.read_bounded(path, 1 << 20).startswith(b"x" * 8)


def test_exactly_at_the_cap_and_one_over(tmp_path):
    path = tmp_path / "edge"
    path.write_bytes(b"z" * 1000)
    assert io_utils.read_bounded(path, 1000) == b"z" * 1000
    with pytest.raises(ValueError, match="bounded regular file"):
        io_utils.read_bounded(path, 999)
    big = tmp_path / "big"
    big.write_bytes(b"q" * ((1 << 20) + 17))  # longer than one read
    assert io_utils.read_bounded(big, 2 << 20) == b"q" * ((1 << 20) + 17)


def test_private_means_owner_only(tmp_path):
    d = tmp_path / "state"
    d.mkdir(mode=0o700)
    io_utils.require_private(d)
    os.chmod(d, 0o750)
    with pytest.raises(ValueError, match="closed to group and others"):
        io_utils.require_private(d)
    f = tmp_path / "key"
    f.write_text("k")
    for mode in (0o640, 0o604, 0o660, 0o601):
        os.chmod(f, mode)
        with pytest.raises(ValueError):
            io_utils.require_private(f)
    for mode in (0o600, 0o400, 0o700):
        os.chmod(f, mode)
        io_utils.require_private(f)


def test_replaced_documents_keep_the_old_one_until_the_new_one_is_whole(tmp_path, monkeypatch):
    path = tmp_path / "state.json"
    io_utils.atomic_json(path, {"v": 1})
    assert stat.S_IMODE(path.stat().st_mode) == 0o600

    class Unserialisable:
        pass

    with pytest.raises(TypeError):
        io_utils.atomic_json(path, {"v": Unserialisable()})
    assert json.loads(path.read_text()) == {"v": 1}  # a failed write never touched the document
    io_utils.atomic_json(path, {"v": 2})
    assert json.loads(path.read_text()) == {"v": 2} and not (tmp_path / "state.json.tmp").exists()
    io_utils.persist_json(path, {"z": 1, "a": [1, 2]})
    assert path.read_text() == '{\n  "a": [\n    1,\n    2\n  ],\n  "z": 1\n}\n'

"""Run the gates against the goldens in ``tests/golden/data`` (see the package docstring)."""

from __future__ import annotations

import json
import sys
from pathlib import Path

DATA = Path(__file__).resolve().parents[2] / "tests" / "golden" / "data"


def gates() -> dict:
    from tools.equivalence import defaults, digests, executed, imports, programs, wire

    return {"g1_launch_programs": programs.collect, "g2_production_defaults": defaults.collect, "g3_oracle_digests": digests.oracle_digests, "g4_checkpoint_identity": digests.checkpoint_identity, "g6_import_closures": imports.collect,
            "g7_executed_functions": executed.collect, "g9_wire_formats": wire.collect}


def load(name: str):
    return json.loads((DATA / f"{name}.json").read_text())


def check(names=None) -> dict:
    from tools.equivalence import executed, imports

    from tools.equivalence import programs

    failures = {}
    for name, fn in gates().items():
        if names and name not in names:
            continue
        if name == "g1_launch_programs" and not programs.available():
            continue  # the launch programs are recorded on a GPU
        current, golden = json.loads(json.dumps(fn())), load(name)
        if name == "g6_import_closures":
            extra = imports.grown(golden, current)
            if extra:
                failures[name] = extra
        elif name == "g7_executed_functions":
            moved = executed.difference(golden, current)
            if moved["no_longer_executed"] or moved["newly_executed"]:
                failures[name] = moved
        elif current != golden:
            failures[name] = {k: {"golden": golden.get(k), "current": current.get(k)} for k in sorted(set(golden) | set(current)) if golden.get(k) != current.get(k)}
    return failures


def update(names=None) -> None:
    DATA.mkdir(parents=True, exist_ok=True)
    from tools.equivalence import programs

    for name, fn in gates().items():
        if names and name not in names:
            continue
        if name == "g1_launch_programs" and not programs.available():
            continue
        (DATA / f"{name}.json").write_text(json.dumps(fn(), indent=1, sort_keys=True) + "\n")


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    command, names = (argv[0] if argv else "check"), set(argv[1:])
    if command == "update":
        update(names)
        return 0
    if command == "selftest":
        from tools.equivalence import selftest

        results = selftest.run()
        print(json.dumps(results, indent=1))
        return 0 if all(results.values()) else 1
    failures = check(names)
    print(json.dumps(failures, indent=1) if failures else "all gates match")
    return 1 if failures else 0


if __name__ == "__main__":
    sys.exit(main())

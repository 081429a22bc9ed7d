"""Token-stream identity of two real runs (e.g. before and after a change, or fused vs NCCL collectives).

    python -m tools.equivalence.compare_run RUN_A RUN_B

Requests are matched by ``request_sha256`` (from ``runner.rank0.json`` of each result directory); for every match the TokenEvent
lines of ``tokens.jsonl`` must be identical.  Exit code 0 = identical, 1 = differences (listed), 2 = nothing to compare.

Parity: reference ``tools/equivalence/compare_run.py:1-60``.
"""

from __future__ import annotations

import json
import sys
from pathlib import Path


def streams(run: Path) -> dict:
    """request_sha256 -> list of (index, token_id, finish_reason) in emission order, over every result directory of ``run``."""
    out: dict = {}
    for record_path in sorted(Path(run).rglob("runner.rank0.json")):
        record = json.loads(record_path.read_text())
        by_id = {r.get("request_id"): r.get("request_sha256") for r in record.get("requests", [])}
        tokens = record_path.parent / "tokens.jsonl"
        if not tokens.exists():
            continue
        for line in tokens.read_text().splitlines():
            event = json.loads(line)
            key = by_id.get(event["request_id"])
            if key:
                out.setdefault(key, []).append((event["index"], event["token_id"], event["finish_reason"]))
    return out


def compare(a: Path, b: Path) -> tuple[int, list]:
    sa, sb = streams(a), streams(b)
    common = sorted(set(sa) & set(sb))
    diffs = []
    for key in common:
        if sa[key] != sb[key]:
            first = next((i for i, (x, y) in enumerate(zip(sa[key], sb[key])) if x != y), min(len(sa[key]), len(sb[key])))
            diffs.append({"request_sha256": key, "first_difference": first, "a_tokens": len(sa[key]), "b_tokens": len(sb[key])})
    return len(common), diffs


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 2:
        print(__doc__)
        return 2
    matched, diffs = compare(Path(argv[0]), Path(argv[1]))
    print(json.dumps({"matched_requests": matched, "differences": diffs}, indent=1))
    return 2 if matched == 0 else (1 if diffs else 0)


if __name__ == "__main__":
    sys.exit(main())

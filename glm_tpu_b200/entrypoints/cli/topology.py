"""``glm-b200 topology capture|bind``.

Parity: reference ``glm_tpu/entrypoints/cli/topology.py``.
"""

from __future__ import annotations

import json


def main(args) -> int:
    from glm_tpu_b200.executor import topology_job

    if args.action == "capture":
        report = topology_job.capture_topology(args.output)
    else:
        report = topology_job.bind_topology(args.capture, args.gpus)
    print(json.dumps(report, indent=2, sort_keys=True))
    return 0

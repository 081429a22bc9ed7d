"""G2: production defaults.  Every limit, cap, default and choice a user or another process relies on without naming it: the
environment registry (kinds, defaults, choices), a site without a file, the request limits and context profiles, the queue and
workspace limits of the serving layer, the body caps and security headers of the HTTP surface, the model names and effort aliases,
the architecture switches the engine assumes, the pack and loader piece size.  A changed default that no test happens to
exercise still changes a digest here; re-record it on purpose with ``python -m tools.equivalence.driver update g2_production_defaults``.
"""

from __future__ import annotations

import dataclasses
from pathlib import Path


def _plain(value):
    if dataclasses.is_dataclass(value) and not isinstance(value, type):
        return {f.name: _plain(getattr(value, f.name)) for f in dataclasses.fields(value)}
    if isinstance(value, dict):
        return {str(k): _plain(v) for k, v in value.items()}
    if isinstance(value, (list, tuple, set, frozenset)):
        items = [_plain(v) for v in value]
        return sorted(items, key=repr) if isinstance(value, (set, frozenset)) else items
    if isinstance(value, Path):
        return "<path>"  # depends on the home directory of whoever runs the gate
    if isinstance(value, bytes):
        return value.decode("latin-1")
    if callable(value):
        return "<computed>"
    return value


def collect() -> dict:
    from glm_tpu_b200 import envs
    from glm_tpu_b200.config import model as model_config
    from glm_tpu_b200.config.site import SUPPORTED_GPUS, TABLE_KEYS, SiteConfig
    from glm_tpu_b200.engine import request as rq
    from glm_tpu_b200.engine import resident_protocol as proto
    from glm_tpu_b200.entrypoints.openai import protocol as api
    from glm_tpu_b200.entrypoints.serve import http_handler, job_queue
    from glm_tpu_b200.entrypoints.ui import conversations
    from glm_tpu_b200.executor.launch_policy import LaunchRules
    from glm_tpu_b200.model_loader.sharded_state import format as fmt

    out: dict = {}
    out["environment"] = {name: {"kind": row.kind, "default": _plain(row.default), "choices": list(row.choices), "secret": row.secret}
                          for name, row in envs.TABLE.items()}
    out["site_without_a_file"] = _plain(SiteConfig())
    out["site_tables"] = {table: sorted(keys) for table, keys in TABLE_KEYS.items()}
    out["supported_gpus"] = list(SUPPORTED_GPUS)
    out["launch_rules"] = _plain(LaunchRules())
    out["request_limits"] = {name: _plain(getattr(rq, name)) for name in (
        "CAPACITY", "CONCURRENT_CAPACITY", "LONG_CAPACITY", "AGENT_CAPACITY", "CAPACITIES", "CONTEXT_ALIASES", "MAX_PROMPT", "PROMPT_LIMITS",
        "CONCURRENT_LIMIT", "QUEUE_LIMIT", "MAX_NEW", "PAYLOAD_CAP", "MESSAGES_CAP", "CHAT_ROLES", "SCHEMA", "BATCH_SCHEMA", "CONCURRENT_SCHEMA")}
    out["glm53_request_profile"] = _plain(rq.GLM53_PROFILE)
    out["model_identity"] = {"model_id": model_config.MODEL_ID, "revision": model_config.MODEL_REVISION, "eos_ids": list(model_config.EOS_IDS),
                             "assumed_switches": _plain(model_config.ASSUMED_SWITCHES)}
    out["serving"] = {"pending": job_queue.PENDING, "api_history": job_queue.API_HISTORY, "busy_poll_seconds": job_queue.BUSY_POLL_SECONDS,
                      "idle_poll_seconds": job_queue.IDLE_POLL_SECONDS, "max_message_bytes": conversations.MAX_MESSAGE_BYTES,
                      "max_title_chars": conversations.MAX_TITLE_CHARS, "auto_title_chars": conversations.AUTO_TITLE_CHARS,
                      "default_title": conversations.DEFAULT_TITLE, "actions": sorted(conversations.ACTIONS)}
    out["http"] = {"ui_body_cap": http_handler.UI_BODY_CAP, "ui_read_seconds": http_handler.UI_READ_SECONDS, "api_read_seconds": http_handler.API_READ_SECONDS,
                   "api_body_cap": api.BODY_CAP, "tools_cap": api.TOOLS_CAP, "security_headers": _plain(http_handler.SECURITY_HEADERS),
                   "pages": _plain(http_handler.UI_PAGES)}
    out["openai_names"] = {"model": api.MODEL_NAME, "aliases": _plain(api.ALIASES), "efforts": list(api.EFFORTS)}
    out["run_directory"] = {name: _plain(getattr(proto, name)) for name in (
        "INBOX_DIR", "STOP_FILE", "STOP_COMMAND", "PRODUCER_LOCK", "READY_FILE", "MEASUREMENT_FILE", "SUMMARY_FILE", "CONTROLLER_IDENTITY_FILE",
        "CONTROLLER_TERMINAL_FILE", "TOKENS_FILE", "ANSWER_FILE", "SEQUENCE_DIGITS", "WORKER_ENV_FLAG", "STDOUT_RUN", "STDOUT_RESIDENT_RESULT")}
    out["checkpoint_format"] = {"version": fmt.FORMAT_VERSION, "piece_bytes": fmt.PIECE_BYTES, "shared_file": fmt.SHARED_FILE, "seal_file": fmt.SEAL_FILE,
                                "manifest_file": fmt.MANIFEST_FILE, "geometry_file": fmt.GEOMETRY_FILE, "expert_file_of_rank_3_of_8": fmt.expert_file(3, 8)}
    return out

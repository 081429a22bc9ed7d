"""G7: the set of functions a fixed scenario executes.

The scenario runs in a fresh interpreter under ``sys.monitoring`` (function-entry events): a question goes through the chat format and
the byte tokenizer into a prepared request, the engine generates six tokens from the tiny model on the CPU oracle runner, the tokens are
written as event lines and split into reasoning and answer, and an OpenAI-style reply is shaped from them.  What is recorded is the set of
``module:qualified name`` of every function of this package that was entered.  The gate compares the set with the golden one and reports
both directions: a function that stopped running (a path silently skipped) and a function that started running (a new dependency of the
serving path) both need a deliberate update of the golden.

Parity: the reference's executed-function gate (``tools/equivalence``, G7) uses the same mechanism on its own scenario.
"""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]

_SCENARIO = r'''
import json, sys
PACKAGE = "glm_tpu_b200"
seen = set()
mon = sys.monitoring
TOOL = mon.COVERAGE_ID
mon.use_tool_id(TOOL, "g7")

def entered(code, offset):
    module = code.co_filename
    at = module.rfind("/" + PACKAGE + "/")
    if at < 0:
        return mon.DISABLE
    name = module[at + 1:-3].replace("/", ".")
    if code.co_name not in ("<module>", "<lambda>", "<genexpr>", "<listcomp>", "<dictcomp>", "<setcomp>"):
        seen.add(name + ":" + code.co_qualname)
    return mon.DISABLE          # one entry per code object is all the gate needs

mon.register_callback(TOOL, mon.events.PY_START, entered)
mon.set_events(TOOL, mon.events.PY_START)

from glm_tpu_b200.config.model import tiny_geometry
from glm_tpu_b200.engine import request as rq
from glm_tpu_b200.engine.llm_engine import LLMEngine
from glm_tpu_b200.engine.outputs import final_channel
from glm_tpu_b200.entrypoints.openai import chat_utils, tool_parser
from glm_tpu_b200.models.glm_moe_dsa.weights import random_checkpoint
from glm_tpu_b200.runner.oracle_runner import OracleRunner
from glm_tpu_b200.tokenizer import load_tokenizer

g = tiny_geometry()
tokenizer = load_tokenizer(None, vocab_size=g.vocab_size, eos_ids=g.eos_ids)
profile = rq.RequestProfile.for_geometry(g, (256,), concurrent_capacity=256)
messages = chat_utils.convert([{"role": "user", "content": "2+2?"}])
prompt = tokenizer.apply_chat_template(messages, reasoning_effort="max")
request = rq.from_token_ids(prompt, request_id="question-01", max_new_tokens=6, context_capacity=256, profile=profile)
rq.validate(request, profile)
runner = OracleRunner(g, random_checkpoint(g, seed=0), context_capacity=256)
events = []
report = LLMEngine(runner, profile=profile).generate(request, events.append)
lines = [json.dumps(e.wire()) for e in events]
thinking, answer = final_channel(tokenizer.decode([e.token_id for e in events]))
tool_parser.parse(answer)
mon.set_events(TOOL, 0)
assert report["emitted"] == 6 and len(lines) == 6
print(json.dumps(sorted(seen)))
'''


def collect() -> dict:
    done = subprocess.run([sys.executable, "-c", _SCENARIO], capture_output=True, text=True, cwd=ROOT, timeout=600)
    if done.returncode != 0:
        raise RuntimeError("the G7 scenario failed:\n" + done.stderr[-3000:])
    return {"functions": json.loads(done.stdout.strip().splitlines()[-1])}


def difference(golden: dict, current: dict) -> dict:
    """``{"no_longer_executed": [...], "newly_executed": [...]}``; both empty when the gate passes."""
    was, now = set(golden.get("functions", [])), set(current.get("functions", []))
    return {"no_longer_executed": sorted(was - now), "newly_executed": sorted(now - was)}

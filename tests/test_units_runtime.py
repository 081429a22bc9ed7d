"""Unit tier for the process-level runtime (no GPU, no model): worker command lines, the idle probe with an injected query, supervision
and cleanup of real child processes, run-directory staging, the API key file, the byte tokenizer and the parallel layout contract.

Mirrors the reference's `tests/executor/test_fleet.py`, `test_staging.py`, `tests/entrypoints/serve/test_security.py` and
`tests/distributed/test_mesh.py` (there the fleet is eight SSH hosts answered by a fake; here it is child processes, so real ones are used).
"""

import json
import os
import stat
import sys
import time

import pytest

from glm_tpu_b200.config.model import glm53_geometry, small_geometry, tiny_geometry
from glm_tpu_b200.config.parallel import ParallelLayout
from glm_tpu_b200.engine import resident_protocol as proto
from glm_tpu_b200.entrypoints.serve.security import api_token
from glm_tpu_b200.exceptions import PlanValidationError
from glm_tpu_b200.executor import fleet, staging
from glm_tpu_b200.tokenizer import ByteTokenizer, load_tokenizer


# ------------------------------------------------------------------------------------------------------- fleet
def test_worker_specs_carry_the_rendezvous_and_the_controller_flag(tmp_path, monkeypatch):
    monkeypatch.delenv("NCCL_NVLS_ENABLE", raising=False)
    specs = fleet.worker_specs(world=4, run_dir=tmp_path, worker_args=["--run", str(tmp_path)], master_port=29123, extra_env={"X_EXTRA": "1"})
    assert [s.rank for s in specs] == [0, 1, 2, 3] and all(s.world == 4 for s in specs)
    for s in specs:
        assert s.argv[:3] == [sys.executable, "-m", proto.WORKER_MODULE] and s.argv[3:] == ["--run", str(tmp_path)]
        assert s.env["RANK"] == s.env["LOCAL_RANK"] == str(s.rank) and s.env["WORLD_SIZE"] == "4"
        assert s.env["MASTER_ADDR"] == "127.0.0.1" and s.env["MASTER_PORT"] == "29123"
        assert s.env[proto.WORKER_ENV_FLAG] == "1" and s.env["X_EXTRA"] == "1"
        assert s.env["NCCL_NVLS_ENABLE"] == "0"  # in-switch reduction stays off unless the operator turns it on
        assert s.log == tmp_path / f"worker.rank{s.rank}.log"
    monkeypatch.setenv("NCCL_NVLS_ENABLE", "1")
    assert fleet.worker_specs(world=1, run_dir=tmp_path, worker_args=[], master_port=1)[0].env["NCCL_NVLS_ENABLE"] == "1"


def test_idle_probe_reports_busy_gpus_and_survives_a_missing_tool():
    idle = fleet.gpu_idle_report(lambda: "\n")
    assert idle == {"available": True, "busy": [], "processes": 0}
    busy = fleet.gpu_idle_report(lambda: "GPU-aaaa, 4242, 1024 MiB\nGPU-bbbb, 4243, 10 MiB\n")
    assert busy["busy"] == ["GPU-aaaa", "GPU-bbbb"] and busy["processes"] == 2

    def broken():
        raise RuntimeError("nvidia-smi failed")

    report = fleet.gpu_idle_report(broken)
    assert report["available"] is False and "nvidia-smi failed" in report["error"] and report["busy"] == []


def _spec(tmp_path, rank, code):
    return fleet.WorkerSpec(rank, 2, [sys.executable, "-c", code], dict(os.environ), tmp_path / f"worker.rank{rank}.log")


def test_supervision_returns_on_the_first_failure_and_cleanup_ends_the_survivor(tmp_path):
    group = fleet.Fleet([_spec(tmp_path, 0, "import time; print('up', flush=True); time.sleep(60)"),
                         _spec(tmp_path, 1, "import sys; print('bye', flush=True); sys.exit(3)")])
    group.start()
    try:
        started = time.monotonic()
        codes = group.wait(deadline=time.monotonic() + 30)
        assert codes[1] == 3 and codes[0] is None and time.monotonic() - started < 20  # one failed: do not wait for the other
    finally:
        final = group.cleanup(grace=5)
    assert final[1] == 3 and final[0] is not None and final[0] != 0  # the sleeper was terminated, not left behind
    assert (tmp_path / "worker.rank1.log").read_text().strip() == "bye"


def test_supervision_honours_the_deadline_and_the_tick_callback(tmp_path):
    group = fleet.Fleet([_spec(tmp_path, 0, "import time; time.sleep(60)")])
    group.start()
    try:
        assert group.wait(deadline=time.monotonic() + 0.5, tick=0.05) == [None]  # deadline passed, still running
        ticks = []
        assert group.wait(deadline=None, on_tick=lambda: ticks.append(1) is None and len(ticks) < 3, tick=0.01) == [None]
        assert len(ticks) == 3
    finally:
        group.cleanup(grace=2)
    assert group.poll()[0] is not None


def test_lines_reach_every_worker_that_keeps_its_stdin(tmp_path):
    code = "import sys; line = sys.stdin.readline(); print(line.strip(), flush=True)"
    group = fleet.Fleet([_spec(tmp_path, 0, code), _spec(tmp_path, 1, code)], keep_stdin=True)
    group.start()
    try:
        group.send_all(b'{"sequence": 1}\n')
        assert group.wait(deadline=time.monotonic() + 30) == [0, 0]
    finally:
        group.cleanup(grace=2)
    assert [json.loads((tmp_path / f"worker.rank{r}.log").read_text()) for r in (0, 1)] == [{"sequence": 1}] * 2


# ------------------------------------------------------------------------------------------------------- staging
def test_run_directories_are_fresh_private_and_never_reused(tmp_path):
    first = staging.new_run_dir(tmp_path / "runs", tag="ask")
    second = staging.new_run_dir(tmp_path / "runs", tag="ask")
    assert first != second and first.name.endswith("-ask") and second.name.endswith("-ask.1")
    for path in (first, second, first / proto.INBOX_DIR):
        assert path.is_dir() and stat.S_IMODE(path.stat().st_mode) == 0o700
    assert staging.stage_request(first, None) is None
    staged = staging.stage_request(first, {"b": 1, "a": "ü"})
    assert staged.read_bytes() == '{"a":"ü","b":1}'.encode("utf-8") and stat.S_IMODE(staged.stat().st_mode) == 0o600
    with pytest.raises(FileExistsError):
        staging.stage_request(first, {"other": True})  # a staged request is never replaced


# ------------------------------------------------------------------------------------------------------- API key
def test_api_key_file_is_created_once_private_and_checked(tmp_path):
    path = tmp_path / "api.key"
    token = api_token(path)
    assert len(token) >= 32 and stat.S_IMODE(path.stat().st_mode) == 0o600 and api_token(path) == token
    os.chmod(path, 0o640)
    with pytest.raises(ValueError, match="private"):
        api_token(path)
    os.chmod(path, 0o600)
    path.write_text("\n")
    with pytest.raises(ValueError, match="empty"):
        api_token(path)
    real = tmp_path / "real.key"
    real.write_text("secret\n")
    os.chmod(real, 0o600)
    (tmp_path / "link.key").symlink_to(real)
    with pytest.raises(ValueError, match="private"):
        api_token(tmp_path / "link.key")


# ------------------------------------------------------------------------------------------------------- tokenizer
def test_byte_tokenizer_specials_unknown_ids_and_limits():
    tok = ByteTokenizer(1024, eos_ids=(1020, 1021))
    text = "<|user|>\nnaïve ✓<|assistant|>"
    ids = tok.encode(text)
    assert tok.decode(ids) == text and ids[0] == tok.special["<|user|>"] and ids[-1] == tok.special["<|assistant|>"]
    assert sum(1 for i in ids if i >= 256) == 2  # specials are single ids, everything else is bytes
    assert tok.decode([72, 105, 1020]) == "Hi<|endoftext|>" and tok.decode([900]) == "<0x384>"
    assert tok.decode([0xE2, 0x9C]) == "�"  # a cut multi-byte character decodes to a replacement, not an exception
    with pytest.raises(ValueError):
        ByteTokenizer(200)
    prompt = tok.apply_chat_template([{"role": "user", "content": "2+2?"}])
    assert tok.decode(prompt).endswith("<|assistant|>") or "<|assistant|>" in tok.decode(prompt)
    assert isinstance(load_tokenizer(None, vocab_size=1024), ByteTokenizer)
    assert isinstance(load_tokenizer("/nonexistent/dir", vocab_size=1024), ByteTokenizer)  # no tokenizer.json there


# ------------------------------------------------------------------------------------------------------- layout contract
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_layout_partitions_heads_experts_columns_and_vocabulary(world):
    g = glm53_geometry()
    layouts = [ParallelLayout(g, world, r) for r in range(world)]
    assert sorted(h for lay in layouts for h in lay.head_range) == list(range(g.attention_heads))
    assert sorted(e for lay in layouts for e in lay.expert_range) == list(range(g.num_routed_experts))
    assert all(lay.expert_owner(e) == lay.rank for lay in layouts for e in lay.expert_range)
    assert sum(lay.vocab_local for lay in layouts) == g.vocab_size
    assert sum(lay.dense_cols_local for lay in layouts) == g.dense_intermediate_size
    assert sum(lay.shared_cols_local for lay in layouts) == g.moe_intermediate_size * g.num_shared_experts
    assert len({lay.layout_hash for lay in layouts}) == 1  # every rank derives the same contract ...
    assert layouts[0].layout_summary()["world"] == world and layouts[0].describe()["experts_local"] == g.num_routed_experts // world


def test_layout_hash_separates_worlds_and_geometries_and_refuses_uneven_splits():
    g = glm53_geometry()
    hashes = {ParallelLayout(g, w, 0).layout_hash for w in (1, 2, 4, 8)} | {ParallelLayout(g.truncated(10), 8, 0).layout_hash}
    assert len(hashes) == 5  # ... and a rank with another world size or another model cannot agree by accident
    with pytest.raises(PlanValidationError, match="not divisible"):
        ParallelLayout(g, 3, 0)
    with pytest.raises(PlanValidationError, match="rank"):
        ParallelLayout(tiny_geometry(), 2, 2)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sliced_experts_partition_the_columns_of_every_expert(world, monkeypatch):
    import torch

    from glm_tpu_b200.config.parallel import default_expert_split
    from glm_tpu_b200.models.glm_moe_dsa.weights import cut_routed, routed_shape

    g = glm53_geometry()
    monkeypatch.delenv("GLM_B200_EXPERT_SPLIT", raising=False)
    assert default_expert_split(g, world) == "sliced" and default_expert_split(g, 1) == "whole"
    monkeypatch.setenv("GLM_B200_EXPERT_SPLIT", "whole")
    assert default_expert_split(g, world) == "whole"
    layouts = [ParallelLayout(g, world, r, "sliced") for r in range(world)]
    cols = g.moe_intermediate_size // world
    assert all(lay.experts_resident == g.num_routed_experts and lay.expert_base == 0 and lay.moe_cols_local == cols for lay in layouts)
    assert sorted(c for lay in layouts for c in lay.moe_col_range) == list(range(g.moe_intermediate_size))
    assert routed_shape(layouts[0], "gate_proj") == (g.num_routed_experts, cols, g.hidden_size)
    assert routed_shape(layouts[0], "down_proj") == (g.num_routed_experts, g.hidden_size, cols)
    assert ParallelLayout(g, world, 0, "sliced").layout_hash != ParallelLayout(g, world, 0, "whole").layout_hash  # the ranks must agree on the split
    # the cuts of a small stacked table put every weight and every block scale on exactly one GPU
    import dataclasses

    small = dataclasses.replace(small_geometry(4), moe_intermediate_size=128 * world)  # 8 heads, 16 experts: divisible by 8
    E, I, H = small.num_routed_experts, small.moe_intermediate_size, small.hidden_size
    bits_up = torch.arange(E * I * H, dtype=torch.int64).reshape(E, I, H)
    scale_up = torch.arange(E * (I // 128) * -(-H // 128), dtype=torch.float32).reshape(E, I // 128, -(-H // 128))
    bits_down = torch.arange(E * H * I, dtype=torch.int64).reshape(E, H, I)
    scale_down = torch.arange(E * -(-H // 128) * (I // 128), dtype=torch.float32).reshape(E, -(-H // 128), I // 128)
    ups = [cut_routed(bits_up, scale_up, "up_proj", ParallelLayout(small, world, r, "sliced")) for r in range(world)]
    downs = [cut_routed(bits_down, scale_down, "down_proj", ParallelLayout(small, world, r, "sliced")) for r in range(world)]
    assert torch.equal(torch.cat([b for b, _ in ups], dim=1), bits_up) and torch.equal(torch.cat([s for _, s in ups], dim=1), scale_up)
    assert torch.equal(torch.cat([b for b, _ in downs], dim=2), bits_down) and torch.equal(torch.cat([s for _, s in downs], dim=2), scale_down)
    with pytest.raises(PlanValidationError, match="FP8 block"):
        ParallelLayout(dataclasses.replace(small_geometry(4), moe_intermediate_size=64 * world), world, 0, "sliced")  # half a block per GPU


def test_checkpoint_tokenizer_json_and_template_file_are_used_and_pinned(tmp_path):
    """A checkpoint directory with a real ``tokenizer.json`` (a small BPE model trained here, with the chat format's special
    tokens) and a ``chat_template.jinja``: ``load_tokenizer`` uses the fast tokenizer, renders the checkpoint's own template, and
    reports the digests of the files it read (they are pinned into every prepared request)."""
    import hashlib

    tokenizers = pytest.importorskip("tokenizers")
    pytest.importorskip("jinja2")
    from tokenizers import models, pre_tokenizers, trainers

    from glm_tpu_b200.tokenizer import SPECIAL_TOKENS, HfTokenizer, chat_template

    tok = tokenizers.Tokenizer(models.BPE(unk_token=None))
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = tokenizers.decoders.ByteLevel()
    corpus = ["Why is the sky blue?", "Name three prime numbers.", "the quick brown fox jumps over the lazy dog"] * 20
    tok.train_from_iterator(corpus, trainers.BpeTrainer(vocab_size=400, special_tokens=list(SPECIAL_TOKENS),
                                                        initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
    tok.save(str(tmp_path / "tokenizer.json"))
    (tmp_path / "tokenizer_config.json").write_text('{"model_max_length": 202752}')
    template = "[gMASK]<sop>{% for m in messages %}<|{{ m['role'] }}|>{{ m['content'] }}{% endfor %}{% if add_generation_prompt %}<|assistant|>{% endif %}"
    (tmp_path / "chat_template.jinja").write_text(template)

    loaded = load_tokenizer(tmp_path, vocab_size=1024)
    assert isinstance(loaded, HfTokenizer) and loaded.vocab_size == tok.get_vocab_size()
    text = "Why is the sky blue?"
    ids = loaded.encode(text)
    assert ids and loaded.decode(ids) == text and len(ids) < len(text.encode())  # merges learned: fewer tokens than bytes
    assert loaded.files == {name: hashlib.sha256((tmp_path / name).read_bytes()).hexdigest() for name in ("tokenizer.json", "tokenizer_config.json")}
    assert loaded.template_sha256 == hashlib.sha256(template.encode()).hexdigest()
    prompt = loaded.apply_chat_template([{"role": "user", "content": text}])
    user, assistant, gmask = (tok.token_to_id(t) for t in ("<|user|>", "<|assistant|>", "[gMASK]"))
    assert prompt[0] == gmask and user in prompt and prompt[-1] == assistant  # the checkpoint's template, special tokens as single ids
    assert loaded.decode(prompt) == "[gMASK]<sop><|user|>" + text + "<|assistant|>"
    # without the template file the built-in chat format is rendered, and its digest is the pinned one
    (tmp_path / "chat_template.jinja").unlink()
    plain = load_tokenizer(tmp_path)
    assert plain.template_sha256 == hashlib.sha256(open(chat_template.__file__, "rb").read()).hexdigest()
    assert plain.decode(plain.apply_chat_template([{"role": "user", "content": text}])) == chat_template.render(
        [{"role": "user", "content": text}], tools=None, reasoning_effort=None, add_generation_prompt=True)

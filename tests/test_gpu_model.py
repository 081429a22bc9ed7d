"""End-to-end: prefill + greedy decode on one B200 against the CPU contract reference.

Router and DSA top-k decisions sit on near-ties (margins of 1e-5 are common with random weights), so a raw token
comparison between two correct implementations is ill-conditioned.  The comparison therefore imposes the engine's
discrete decisions (attended positions of every full layer, routed experts of every sparse layer) on the oracle,
checks that only a small fraction of them differ from the oracle's own, and then requires every generated token
to be the oracle's greedy choice up to a bf16 near-tie in the logits.
"""

import pytest
import torch

from glm_tpu_b200.config.model import small_geometry, tiny_geometry
from glm_tpu_b200.models.glm_moe_dsa.weights import random_checkpoint
from glm_tpu_b200.oracle import contract

pytestmark = pytest.mark.gpu


def _run_engine(g, ckpt, prompt, new_tokens, capacity, stripe, use_graphs, prefill_chunk=32, record=False):
    from glm_tpu_b200.runner.gpu_runner import build_runner

    runner = build_runner(g, checkpoint=ckpt, context_capacity=capacity, lanes=1, stripe=stripe, use_graphs=use_graphs,
                          prefill_chunk=prefill_chunk)
    decisions = {"selected": {i: [] for i in g.full_layers}, "experts": {i: [] for i in g.sparse_layers}}
    if record:
        assert not use_graphs
        inner = runner.model.run_rows

        def recording(*a, **k):
            runner.model.trace = {}
            out = inner(*a, **k)
            t = runner.model.trace
            for layer in g.full_layers:
                for row in t["sel_global"][layer].cpu():
                    decisions["selected"][layer].append(row[row >= 0].long())
            for layer in g.sparse_layers:
                decisions["experts"][layer].append(t["topk_ids"][layer].cpu().long())
            runner.model.trace = None
            return out

        runner.model.run_rows = recording
    first = runner.prefill(0, prompt)
    runner.build_decode_program()
    if record:  # the warm-up launch of build_decode_program ran one inactive row: drop its record
        for layer in g.full_layers:
            decisions["selected"][layer].pop()
        for layer in g.sparse_layers:
            decisions["experts"][layer].pop()
    out = [first]
    for step in range(new_tokens - 1):
        runner.decode_step()
        out.append(runner.read_step_tokens(step)[0])
    runner.peer.check_status()
    runner.close()
    if record:
        decisions["experts"] = {k: torch.cat(v) for k, v in decisions["experts"].items()}
    return out, decisions


def _bad_tokens(g, ckpt, prompt, generated, capacity, decisions=None):
    w = contract.OracleWeights.from_checkpoint(g, ckpt)
    seq = list(prompt) + list(generated[:-1])
    kwargs = {}
    if decisions is not None:
        kwargs = {"selected": {k: v[: len(seq)] for k, v in decisions["selected"].items()},
                  "expert_ids": {k: v[: len(seq)] for k, v in decisions["experts"].items()}}
    trace = contract.forward(w, seq, capacity=capacity, **kwargs)
    bad = []
    for i, tok in enumerate(generated):
        row = trace.logits[len(prompt) - 1 + i]
        gap = float(row.max() - row[tok])
        if gap > 2 * 2**-7 * float(row.abs().max()) + 1e-6:
            bad.append((i, tok, int(trace.tokens[len(prompt) - 1 + i]), gap))
    return bad, trace


def _decision_drift(g, ckpt, seq, decisions, capacity):
    """Fraction of rows whose imposed decision differs from the oracle's own (run with the decisions imposed upstream)."""
    w = contract.OracleWeights.from_checkpoint(g, ckpt)
    free = contract.forward(w, seq, capacity=capacity)
    rows = len(seq)
    sel_diff = sum(
        int(not torch.equal(decisions["selected"][layer][r], free.selected[layer][r])) for layer in g.full_layers for r in range(rows)
    )
    exp_diff = sum(
        int((decisions["experts"][layer][:rows].sort(-1).values != free.expert_ids[layer].sort(-1).values).any(-1).sum())
        for layer in g.sparse_layers
    )
    return sel_diff / max(1, rows * len(g.full_layers)), exp_diff / max(1, rows * len(g.sparse_layers))


def test_tiny_fixture_tokens_match_oracle(native_lib):
    g = tiny_geometry()
    ckpt = random_checkpoint(g, seed=0)
    torch.manual_seed(0)
    prompt = torch.randint(0, g.vocab_size, (32,)).tolist()
    out, decisions = _run_engine(g, ckpt, prompt, 16, capacity=64, stripe=8, use_graphs=False, record=True)
    assert len(out) == 16 and all(0 <= t < g.vocab_size for t in out)
    bad, _ = _bad_tokens(g, ckpt, prompt, out, 64, decisions)
    assert not bad, bad
    graph_out, _ = _run_engine(g, ckpt, prompt, 16, capacity=64, stripe=8, use_graphs=True)
    assert graph_out == out  # the CUDA-graph replay runs the same kernels in the same order


def test_small_fixture_index_share_and_chunked_prefill(native_lib):
    g = small_geometry(4)
    ckpt = random_checkpoint(g, seed=3)
    torch.manual_seed(3)
    prompt = torch.randint(0, g.vocab_size, (75,)).tolist()  # > top_k 32, not a multiple of the chunk
    out, decisions = _run_engine(g, ckpt, prompt, 12, capacity=128, stripe=16, use_graphs=False, prefill_chunk=32, record=True)
    bad, _ = _bad_tokens(g, ckpt, prompt, out, 128, decisions)
    assert not bad, bad
    sel_drift, exp_drift = _decision_drift(g, ckpt, list(prompt) + out[:-1], decisions, 128)
    assert sel_drift < 0.2 and exp_drift < 0.2, (sel_drift, exp_drift)
    graph_out, _ = _run_engine(g, ckpt, prompt, 12, capacity=128, stripe=16, use_graphs=True, prefill_chunk=32)
    assert graph_out == out


def test_prefill_partition(native_lib):
    g = small_geometry(2)
    ckpt = random_checkpoint(g, seed=4)
    torch.manual_seed(4)
    prompt = torch.randint(0, g.vocab_size, (50,)).tolist()
    for chunk in (64, 16):
        out, decisions = _run_engine(g, ckpt, prompt, 6, capacity=128, stripe=16, use_graphs=False, prefill_chunk=chunk, record=True)
        bad, _ = _bad_tokens(g, ckpt, prompt, out, 128, decisions)
        assert not bad, (chunk, bad)


def test_decode_is_deterministic(native_lib):
    g = tiny_geometry()
    ckpt = random_checkpoint(g, seed=1)
    prompt = list(range(5, 25))
    a, _ = _run_engine(g, ckpt, prompt, 10, capacity=64, stripe=8, use_graphs=True)
    b, _ = _run_engine(g, ckpt, prompt, 10, capacity=64, stripe=8, use_graphs=True)
    assert a == b


def test_lanes_are_isolated_bitwise(native_lib):
    """Batched decode: a lane's tokens and cached rows do not change when the OTHER lane's conversation changes
    (reference ``tests/models/glm_moe_dsa/test_model.py:88-99``: bitwise isolation under perturbation of one lane)."""
    from glm_tpu_b200.runner.gpu_runner import build_runner

    g = small_geometry(4)
    ckpt = random_checkpoint(g, seed=11)
    gen = torch.Generator().manual_seed(11)
    mine = torch.randint(0, g.vocab_size, (45,), generator=gen).tolist()
    others = [torch.randint(0, g.vocab_size, (n,), generator=gen).tolist() for n in (30, 61)]
    results = []
    for other in others:
        runner = build_runner(g, checkpoint=ckpt, context_capacity=128, lanes=2, stripe=16, use_graphs=True, prefill_chunk=32)
        first = runner.prefill(0, mine)
        runner.prefill(1, other)
        runner.build_decode_program()
        toks = [first]
        for step in range(8):
            runner.decode_step()
            toks.append(runner.read_step_tokens(step)[0])
        torch.cuda.synchronize()
        rows = len(mine) + 8
        results.append((toks, runner.state.kv_cache[0, :, :rows].clone().cpu(), runner.state.index_cache[0, :, :rows].clone().cpu()))
        runner.peer.check_status()
        runner.close()
    assert results[0][0] == results[1][0]
    assert torch.equal(results[0][1].view(torch.int16), results[1][1].view(torch.int16))
    assert torch.equal(results[0][2].view(torch.int16), results[1][2].view(torch.int16))


def test_inactive_lane_is_frozen(native_lib):
    """A deactivated lane neither advances nor writes its cache while the other lane keeps decoding."""
    from glm_tpu_b200.runner.gpu_runner import build_runner

    g = tiny_geometry()
    ckpt = random_checkpoint(g, seed=2)
    runner = build_runner(g, checkpoint=ckpt, context_capacity=64, lanes=2, stripe=16, use_graphs=True, prefill_chunk=16)
    runner.prefill(0, list(range(3, 20)))
    runner.prefill(1, list(range(40, 52)))
    runner.build_decode_program()
    runner.decode_step()
    runner.deactivate(1)
    torch.cuda.synchronize()
    before = (runner.state.kv_cache[1].clone(), int(runner.state.positions[1]), int(runner.state.tokens[1]))
    for step in range(1, 5):
        runner.decode_step()
        assert runner.read_step_tokens(step)[1] == -1
    torch.cuda.synchronize()
    assert int(runner.state.positions[1]) == before[1] and int(runner.state.tokens[1]) == before[2]
    assert torch.equal(runner.state.kv_cache[1].view(torch.int16), before[0].view(torch.int16))
    assert int(runner.state.positions[0]) == 17 + 5
    runner.peer.check_status()
    runner.close()


def test_bad_cache_metadata_is_reported_and_leaves_the_caches_unchanged(native_lib):
    """A position outside the context (corrupted device metadata): the step reports BAD_INDEX, stores nothing into the KV and
    index caches, faults nothing, and the engine refuses to go on (the status word fails the validity vote)."""
    from glm_tpu_b200.engine import request as rq
    from glm_tpu_b200.engine.llm_engine import LLMEngine
    from glm_tpu_b200.exceptions import EngineFailure
    from glm_tpu_b200.ops import native
    from glm_tpu_b200.runner.gpu_runner import build_runner

    g = tiny_geometry()
    ckpt = random_checkpoint(g, seed=2)
    for graphs in (False, True):
        runner = build_runner(g, checkpoint=ckpt, context_capacity=64, lanes=2, stripe=16, use_graphs=graphs, prefill_chunk=16)
        runner.prefill(0, list(range(3, 20)))
        runner.prefill(1, list(range(40, 52)))
        runner.build_decode_program()
        runner.decode_step()
        torch.cuda.synchronize()
        assert runner.peer.read_status() == 0
        runner.state.positions[1] = 64 + 9  # beyond the 64-slot context
        kv, idx = runner.state.kv_cache.clone(), runner.state.index_cache.clone()
        runner.decode_step()
        torch.cuda.synchronize()
        assert runner.peer.read_status() & native.STATUS_BAD_INDEX
        assert torch.equal(runner.state.kv_cache[1].view(torch.int16), kv[1].view(torch.int16))  # the bad lane stored nothing
        assert torch.equal(runner.state.index_cache[1].view(torch.int16), idx[1].view(torch.int16))
        assert not torch.equal(runner.state.kv_cache[0].view(torch.int16), kv[0].view(torch.int16))  # the healthy lane did
        runner.close()
    # through the engine: the same corruption in the middle of a request poisons it
    runner = build_runner(g, checkpoint=ckpt, context_capacity=64, lanes=1, stripe=16, use_graphs=True, prefill_chunk=16)
    profile = rq.RequestProfile(vocab_size=g.vocab_size, eos_ids=tuple(g.eos_ids), capacities=(64,), prompt_limits={64: 32},
                                concurrent_capacity=64, max_new=32)
    engine = LLMEngine(runner, profile=profile)
    inner, calls = runner.decode_step, [0]

    def corrupting():
        calls[0] += 1
        if calls[0] == 3:
            runner.state.positions[0] = -5
        inner()

    runner.decode_step = corrupting
    request = rq.from_token_ids(list(range(3, 12)), request_id="r", max_new_tokens=10, context_capacity=64, profile=profile)
    with pytest.raises(EngineFailure):
        engine.generate(request)
    assert engine.poisoned
    runner.close()


def test_packed_checkpoint_streams_to_the_device_and_decodes_like_the_arrays_it_came_from(native_lib, tmp_path, monkeypatch):
    """export -> pack -> load on the GPU: tensors travel file -> pinned staging -> device in bounded pieces, digests are checked on
    the way, and the resident weights equal those cut from the in-memory checkpoint; the runner built from them decodes the same tokens."""
    from glm_tpu_b200.config.parallel import ParallelLayout
    from glm_tpu_b200.executor.pack_job import pack_checkpoint
    from glm_tpu_b200.model_loader import export, source_marker
    from glm_tpu_b200.model_loader.sharded_state import format as fmt
    from glm_tpu_b200.model_loader.sharded_state import loader
    from glm_tpu_b200.models.glm_moe_dsa.weights import shard_checkpoint
    from glm_tpu_b200.runner.gpu_runner import build_runner

    g = tiny_geometry()
    ckpt = random_checkpoint(g, seed=6)
    export.export_source(ckpt, g, tmp_path / "src", shards=2)
    source_marker.mark_source(tmp_path / "src")
    pack_checkpoint(tmp_path / "src", tmp_path / "packed", 1, jobs=1)
    monkeypatch.setattr(fmt, "PIECE_BYTES", 8192)  # many pieces per tensor through one small pinned buffer
    streamed = loader.load_rank_checkpoint(tmp_path / "packed", 0, 1, device="cuda:0")
    layout = ParallelLayout(g, 1, 0)
    got = shard_checkpoint(streamed, layout, "cuda:0")
    want = shard_checkpoint(ckpt, layout, "cuda:0")
    stats = streamed.io_stats()
    assert 0 < stats["largest_piece"] <= 8192 and stats["bytes_read"] > 0
    assert torch.equal(got.embed, want.embed) and torch.equal(got.lm_head, want.lm_head)
    for lw, lg in zip(want.layers, got.layers):
        for key, value in vars(lw).items():
            if isinstance(value, torch.Tensor):
                assert torch.equal(getattr(lg, key), value), key
    prompt = list(range(5, 25))
    tokens = []
    for arrays in (loader.load_rank_checkpoint(tmp_path / "packed", 0, 1, device="cuda:0"), ckpt):
        runner = build_runner(g, checkpoint=arrays, context_capacity=64, lanes=1, stripe=16, use_graphs=True, prefill_chunk=16)
        out = [runner.prefill(0, prompt)]
        runner.build_decode_program()
        for step in range(5):
            runner.decode_step()
            out.append(runner.read_step_tokens(step)[0])
        runner.peer.check_status()
        runner.close()
        tokens.append(out)
    assert tokens[0] == tokens[1]


def test_glm53_dimensions_match_the_oracle(native_lib):
    """The flagship's tensor shapes end to end against the CPU oracle: hidden 6144, 64 heads, MLA ranks 2048 / 512 + 64, the 32 x 128
    indexer with top-2048, 12,288-wide dense MLPs, 2,048-wide FP8 experts in 128 x 128 blocks -- the first four layers of the
    architecture (three dense, one MoE; three with their own indexer, one sharing), with 16 routed experts and an 8,192-token
    vocabulary so that the oracle stays affordable on the CPU.  Tokens are compared under the engine's own discrete decisions."""
    import dataclasses

    from glm_tpu_b200.config.model import glm53_geometry

    g = dataclasses.replace(glm53_geometry().truncated(4), num_routed_experts=16, vocab_size=8192, eos_ids=(8189, 8190, 8191))
    ckpt = random_checkpoint(g, seed=11)
    torch.manual_seed(11)
    prompt = torch.randint(0, g.vocab_size - 8, (45,)).tolist()
    out, decisions = _run_engine(g, ckpt, prompt, 6, capacity=256, stripe=64, use_graphs=False, prefill_chunk=32, record=True)
    assert len(out) == 6 and all(0 <= t < g.vocab_size for t in out)
    bad, _ = _bad_tokens(g, ckpt, prompt, out, 256, decisions)
    assert not bad, bad
    graph_out, _ = _run_engine(g, ckpt, prompt, 6, capacity=256, stripe=64, use_graphs=True, prefill_chunk=32)
    assert graph_out == out

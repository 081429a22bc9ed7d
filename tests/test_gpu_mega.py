"""The fused decode phases against the per-kernel decode path (one B200).

The phases run either as kernels of their own (``decode_path="phases"``) or as stretches of one persistent cooperative kernel
(``"mega"``).  Both share their inner functions with the per-kernel path; with the compatible split of K over warps all three
must agree bit for bit: the same tokens, the same layer outputs, the same cache rows.  The default (balanced) split adds the
same products in another order, so it is compared with a tolerance.
"""

import pytest
import torch

from glm_tpu_b200.config.model import glm53_geometry, small_geometry, tiny_geometry
from glm_tpu_b200.models.glm_moe_dsa.weights import random_checkpoint

pytestmark = pytest.mark.gpu


def _runner(g, ckpt, *, path, lanes=1, capacity=256, stripe=8, graphs=False, compat=True, chunk=32, seed=0):
    from glm_tpu_b200.runner.gpu_runner import build_runner

    return build_runner(g, checkpoint=ckpt, seed=seed, context_capacity=capacity, lanes=lanes, stripe=stripe, use_graphs=graphs,
                        prefill_chunk=chunk, decode_path=path, mega_compat_ksplit=compat)


def _decode(runner, prompts, steps):
    first = [runner.prefill(lane, p) for lane, p in enumerate(prompts)]
    runner.build_decode_program()
    tokens, updates = [first], []
    for step in range(steps):
        runner.decode_step()
        tokens.append(runner.read_step_tokens(step))
        updates.append(runner.decode_ws.update.clone())
    runner.peer.check_status()
    return tokens, updates


def _prompts(g, lengths, seed=3):
    gen = torch.Generator().manual_seed(seed)
    return [torch.randint(0, g.vocab_size, (n,), generator=gen).tolist() for n in lengths]


@pytest.mark.parametrize("path", ["phases", "mega"])
@pytest.mark.parametrize("geometry,lengths", [
    ("tiny", (20,)), ("small", (40,)), ("small", (17, 33, 5, 40)), ("small8", (9, 30)),
])
def test_mega_is_bit_identical_to_the_kernel_path(geometry, lengths, path):
    g = {"tiny": tiny_geometry(), "small": small_geometry(4), "small8": small_geometry(8)}[geometry]
    ckpt = random_checkpoint(g, seed=11)
    prompts = _prompts(g, lengths)
    ref = _runner(g, ckpt, path="kernels", lanes=len(lengths))
    mega = _runner(g, ckpt, path=path, lanes=len(lengths))
    assert mega.decode_path == path and ref.decode_path == "kernels"
    steps = 12
    t_ref, u_ref = _decode(ref, prompts, steps)
    t_mega, u_mega = _decode(mega, prompts, steps)
    assert t_mega == t_ref
    for a, b in zip(u_ref, u_mega):
        assert torch.equal(a, b)
    assert torch.equal(ref.state.kv_cache, mega.state.kv_cache)
    assert torch.equal(ref.state.index_cache, mega.state.index_cache)
    assert torch.equal(ref.state.positions, mega.state.positions)
    if path == "mega":  # a few dozen launches instead of ~17 per layer
        assert mega.decode_launches <= 4 * len(g.full_layers) + 1
    else:
        assert mega.decode_launches <= 11 * g.num_layers + 3 * len(g.full_layers) + 2
    ref.close()
    mega.close()


@pytest.mark.parametrize("path", ["phases", "mega"])
def test_mega_at_glm53_shapes_is_bit_identical(path):
    """Five layers of the GLM-5.3 geometry (3 dense + 2 MoE with all 256 FP8 experts, three layers with their own indexer)."""
    g = glm53_geometry().truncated(5)
    prompts = _prompts(g, (48,))
    ref = _runner(g, None, path="kernels", capacity=2048, stripe=64, chunk=64)
    mega = _runner(g, None, path=path, capacity=2048, stripe=64, chunk=64)
    t_ref, u_ref = _decode(ref, prompts, 6)
    t_mega, u_mega = _decode(mega, prompts, 6)
    assert t_mega == t_ref
    for a, b in zip(u_ref, u_mega):
        assert torch.equal(a, b)
    assert torch.equal(ref.state.kv_cache[:, :, :64], mega.state.kv_cache[:, :, :64])
    ref.close()
    mega.close()


@pytest.mark.parametrize("path", ["phases", "mega"])
def test_mega_four_lanes_at_glm53_shapes_is_bit_identical(path):
    g = glm53_geometry().truncated(4)
    prompts = _prompts(g, (30, 41, 12, 25))
    ref = _runner(g, None, path="kernels", lanes=4, capacity=1024, stripe=64, chunk=64)
    mega = _runner(g, None, path=path, lanes=4, capacity=1024, stripe=64, chunk=64)
    t_ref, u_ref = _decode(ref, prompts, 4)
    t_mega, u_mega = _decode(mega, prompts, 4)
    assert t_mega == t_ref
    for a, b in zip(u_ref, u_mega):
        assert torch.equal(a, b)
    ref.close()
    mega.close()


@pytest.mark.parametrize("path", ["phases", "mega"])
def test_mega_graph_replay_equals_eager_and_frozen_lane_stays_put(path):
    g = small_geometry(4)
    ckpt = random_checkpoint(g, seed=5)
    prompts = _prompts(g, (21, 34))
    eager = _runner(g, ckpt, path=path, lanes=2, graphs=False)
    graph = _runner(g, ckpt, path=path, lanes=2, graphs=True)
    t_e, _ = _decode(eager, prompts, 10)
    t_g, _ = _decode(graph, prompts, 10)
    assert t_e == t_g
    assert graph.report.programs[-1].kind == "cuda_graph"
    # freeze lane 1: its position, token register and cache stay as they are, lane 0 goes on
    graph.deactivate(1)
    pos = graph.state.positions.clone()
    cache1 = graph.state.kv_cache[1].clone()
    graph.decode_step()
    out = graph.read_last_tokens()
    assert out[1] == -1 and out[0] >= 0
    assert int(graph.state.positions[1]) == int(pos[1]) and int(graph.state.positions[0]) == int(pos[0]) + 1
    assert torch.equal(graph.state.kv_cache[1], cache1)
    graph.peer.check_status()
    eager.close()
    graph.close()


@pytest.mark.parametrize("path", ["phases", "mega"])
def test_mega_balanced_split_stays_close_to_the_compatible_one(path):
    """The balanced K split changes only the order of fp32 additions: one step from the same state gives layer outputs within
    bf16 rounding of the compatible split's (a step later the discrete choices may differ, so one step is what is compared)."""
    g = small_geometry(4)
    ckpt = random_checkpoint(g, seed=7)
    prompts = _prompts(g, (37,))
    a = _runner(g, ckpt, path=path, compat=True)
    b = _runner(g, ckpt, path=path, compat=False)
    _, ua = _decode(a, prompts, 1)
    _, ub = _decode(b, prompts, 1)
    x, y = ua[0].float(), ub[0].float()
    assert torch.allclose(x, y, rtol=2**-6, atol=2**-6 * float(x.abs().max()))
    a.close()
    b.close()


def test_mega_refuses_what_it_does_not_take():
    from glm_tpu_b200.runner.gpu_runner import build_runner

    g = small_geometry(4)
    ckpt = random_checkpoint(g, seed=1)
    with pytest.raises(ValueError):
        # nine lanes are more rows than the skinny phases take
        build_runner(g, checkpoint=ckpt, context_capacity=128, lanes=9, stripe=8, decode_path="mega")

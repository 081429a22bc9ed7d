"""Property-based checks (hypothesis) of the pieces whose contract is a total rule rather than an example: the exact top-k, the cache
striping, canonical JSON and the route grouping that the expert sort must reproduce."""

import json
import struct

import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from glm_tpu_b200.config.cache import CacheConfig
from glm_tpu_b200.config.model import tiny_geometry
from glm_tpu_b200.oracle import contract
from glm_tpu_b200.utils import json_utils

finite32 = st.floats(width=32, allow_nan=False, allow_infinity=False)


def _bits(x: float) -> int:
    """Total order of fp32 values as the kernels see it: sign-magnitude bits mapped to an unsigned key (-0 below +0)."""
    b = struct.unpack("<I", struct.pack("<f", x))[0]
    return 0xFFFFFFFF - b if b >> 31 else b + 0x80000000


@settings(max_examples=200, deadline=None)
@given(st.lists(st.one_of(finite32, st.sampled_from([0.0, -0.0, 1.0, 1.0, -2.5])), min_size=1, max_size=300), st.integers(1, 64), st.data())
def test_top_k_is_the_k_largest_by_bit_order_with_ties_to_the_lowest_position(values, k, data):
    n = data.draw(st.integers(1, len(values)))
    got = contract.top_k_positions(torch.tensor(values, dtype=torch.float32), n, k).tolist()
    want = sorted(sorted(range(n), key=lambda i: (-_bits(values[i]), i))[: min(k, n)])
    assert got == want


@settings(max_examples=100, deadline=None)
@given(st.sampled_from([1, 2, 4, 8]), st.sampled_from([1, 8, 64]), st.integers(1, 6), st.data())
def test_striping_round_trips_for_any_layout(world, stripe, pages, data):
    cache = CacheConfig(tiny_geometry(), context_capacity=world * stripe * pages, world=world, stripe=stripe)
    pos = data.draw(st.integers(0, cache.context_capacity - 1))
    rank, row = cache.owner(pos), cache.local_row(pos)
    assert cache.global_position(rank, row) == pos and 0 <= row < cache.local_capacity
    ctx = data.draw(st.integers(0, cache.context_capacity))
    assert sum(cache.owned_count(r, ctx) for r in range(world)) == ctx
    assert (row < cache.owned_count(rank, ctx)) == (pos < ctx)  # a position is below the context exactly when its row is among the owned ones


json_values = st.recursive(st.one_of(st.none(), st.booleans(), st.integers(-2**53, 2**53), st.text(max_size=8)),
                           lambda inner: st.one_of(st.lists(inner, max_size=4), st.dictionaries(st.text(max_size=6), inner, max_size=4)), max_leaves=12)


@settings(max_examples=150, deadline=None)
@given(st.dictionaries(st.text(max_size=6), json_values, max_size=5), st.randoms())
def test_canonical_json_ignores_key_order_and_round_trips(value, rng):
    items = list(value.items())
    rng.shuffle(items)
    shuffled = dict(items)
    assert json_utils.canonical_wire_bytes(value) == json_utils.canonical_wire_bytes(shuffled)
    assert json_utils.fingerprint(value) == json_utils.fingerprint(shuffled)
    assert json.loads(json_utils.canonical_wire_bytes(value).decode("utf-8")) == value
    assert json.loads(json_utils.canonical_hash_bytes(value).decode("ascii")) == value
    assert json_utils.canonical_hash_bytes(value).isascii()


@settings(max_examples=100, deadline=None)
@given(st.integers(1, 40), st.integers(1, 4), st.integers(1, 12), st.data())
def test_route_grouping_is_lossless_and_stable(rows, tk, experts, data):
    """The grouping the expert sort must reproduce: every local route appears once, experts ascending, route order kept inside an
    expert, tiles of at most 128 routes that never straddle two experts."""
    from glm_tpu_b200.models.glm_moe_dsa.model import GlmMoeDsaModel

    el = data.draw(st.integers(1, experts))
    ebase = data.draw(st.integers(0, experts - el))
    ids = torch.tensor(data.draw(st.lists(st.lists(st.integers(0, experts - 1), min_size=tk, max_size=tk), min_size=rows, max_size=rows)), dtype=torch.int32)
    tiles, n_tiles, perm = GlmMoeDsaModel._route_tiles128(None, ids, ebase, el)
    flat = ids.reshape(-1).tolist()
    local = [i for i, e in enumerate(flat) if ebase <= e < ebase + el]
    placed = [p for p in perm.tolist() if p >= 0]
    assert sorted(placed) == local and perm.tolist()[len(local):] == [-1] * (len(flat) - len(local))
    assert placed == sorted(local, key=lambda i: (flat[i], i))
    covered = []
    for row0, row_end, expert, _ in tiles[: int(n_tiles.item())].tolist():
        stop = min(row_end, row0 + 128)
        assert 0 <= expert < el and row0 < row_end
        assert all(flat[placed[j]] - ebase == expert for j in range(row0, stop))
        covered += list(range(row0, stop))
    assert covered == list(range(len(local)))

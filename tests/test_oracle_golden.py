"""Pin the CPU oracle: reference known answers + fixtures generated from the reference."""

from __future__ import annotations

from types import SimpleNamespace

import numpy as np
import pytest
import torch

from community_kv_b200.state import DecodeDeltaChunks, MutableGraphState, PrefillCSR
from oracle import decode_oracle as oracle


def _bits(values) -> np.ndarray:
    return np.asarray(values, dtype=np.float32).astype(np.float16).view(np.uint16)


def _takes(selection: oracle.Selection) -> list[tuple[int, int]]:
    ends = selection.cumulative_ends.tolist()
    starts = [0] + ends[:-1]
    return [(int(c), e - s) for c, s, e in zip(selection.communities.tolist(), starts, ends)]


# ---- known answers held by the reference's own unit tests ----------------------------------
def test_ordered_keys_preserve_numeric_order():
    # reference tests/community_kv/attention/kernels/test_centroid_selection.py:69-75
    keys = oracle.ordered_fp16_keys(_bits([-np.inf, -2.0, -0.0, 0.0, 1.0, np.inf])).astype(np.int64)
    assert np.all(keys[1:] >= keys[:-1])


def test_selection_truncates_last_community():
    # test_centroid_selection.py:78-88 -> (1, 7), (2, 3)
    picked = oracle.select_descriptors(_bits([0.1, 0.9, 0.5]), np.array([4, 7, 5], np.int32), 3, 10)
    assert sorted(_takes(picked)) == [(1, 7), (2, 3)]
    assert int(picked.cumulative_ends[-1]) == 10


def test_selection_breaks_fp16_ties_by_community_id():
    # test_centroid_selection.py:91-99 -> [0, 1]
    picked = oracle.select_descriptors(
        _bits([1.0001, 1.0002, 1.0001]), np.array([1, 1, 1], np.int32), 3, 2
    )
    assert picked.communities.tolist() == [0, 1]


def test_selection_ignores_empty_and_inactive():
    # test_centroid_selection.py:102-111 -> [(0, 2)]
    picked = oracle.select_descriptors(
        _bits([2.0, 3.0, 100.0, 200.0]), np.array([2, 0, 9, 9], np.int32), 2, 4
    )
    assert _takes(picked) == [(0, 2)]


def test_tile_starts_known_answers():
    # reference test_packed_segments.py:103-149
    assert oracle.tile_start_descriptors(np.array([20, 90, 117]), 3, 2, 10).tolist() == [0, 1]
    assert oracle.tile_start_descriptors(np.array([54, 117]), 2, 2, 10).tolist() == [0, 1]
    singles = np.arange(1, 128)
    assert oracle.tile_start_descriptors(singles, 127, 2, 0).tolist() == [0, 64]


def _reference_csr() -> PrefillCSR:
    return PrefillCSR(
        member_offsets=torch.tensor([[0, 2, 3, 6]], dtype=torch.int32),
        member_positions=torch.tensor([[4, 9, 2, 0, 6, 8]], dtype=torch.int32),
        community_counts=torch.tensor([3], dtype=torch.int32),
    )


def test_positions_read_deltas_newest_first_then_prefill():
    # reference tests/community_kv/graph/test_state.py:160-175 -> [11, 10, 4, 9, 0]
    csr = _reference_csr()
    deltas = DecodeDeltaChunks.allocate(graph_count=1, community_capacity=4, max_decode_tokens=8)
    deltas.append(0, 0, 10)
    deltas.append(0, 0, 11)
    positions = oracle.resolve_positions(
        graph=0,
        csr=csr,
        deltas=deltas,
        communities=np.array([0, 2], np.int32),
        cumulative_ends=np.array([4, 5], np.int32),
        count=2,
        sink_positions=np.zeros(0, np.int32),
        current_position=99,
        token_budget=64,
        num_sink=0,
    )
    assert positions[:5].tolist() == [11, 10, 4, 9, 0]
    assert positions[63] == 99 and np.all(positions[5:63] == -1)


def _small_state(capacity=8, dim=128, decode=16, sequence=70_000) -> MutableGraphState:
    state = MutableGraphState(
        centroids=torch.zeros((1, capacity, dim), dtype=torch.float8_e4m3fn),
        community_sizes=torch.zeros((1, capacity), dtype=torch.int32),
        community_counts=torch.full((1,), 2, dtype=torch.int32),
        community_weight=torch.zeros((1, capacity), dtype=torch.float32),
        total_weight=torch.ones((1,), dtype=torch.float32),
        token_communities=torch.full((1, sequence), -1, dtype=torch.int32),
        deltas=DecodeDeltaChunks.allocate(
            graph_count=1, community_capacity=capacity, max_decode_tokens=decode
        ),
        retrieval_to_graph=torch.zeros(1, dtype=torch.int32),
        retrieval_to_kv=torch.zeros(1, dtype=torch.int32),
    )
    state.community_sizes[:, :2] = torch.tensor([2, 1], dtype=torch.int32)
    state.centroids[:, 0] = 1.0
    state.centroids[:, 1] = -1.0
    state.token_communities[:, 10:12] = 0
    state.token_communities[:, 12:13] = 1
    state.token_communities[:, 4:5] = 0
    state.token_communities[:, 5:6] = 1
    return state


def _run_update(state, scores, positions, lse, key_row, current, lam, forced=-1):
    cache = torch.zeros((1, state.token_communities.shape[1], key_row.shape[-1]), dtype=torch.bfloat16)
    cache[0, current] = key_row
    cursor = torch.tensor([current], dtype=torch.int32)
    assigned = torch.zeros(1, dtype=torch.int32)
    overflow = torch.zeros(1, dtype=torch.int32)
    padded_scores = np.full(8, -np.inf, np.float32)
    padded_positions = np.full(8, -1, np.int32)
    padded_scores[: len(scores)] = scores
    padded_positions[: len(positions)] = positions
    oracle.online_update(
        state=state,
        retrieval_head=0,
        graph=0,
        kv_head=0,
        topk_scores=padded_scores,
        topk_positions=padded_positions,
        representative_lse=np.float32(lse),
        key_cache=cache,
        current_position=cursor,
        lam=lam,
        assigned_out=assigned,
        overflow_out=overflow,
        forced_community=forced,
    )
    return int(assigned[0]), int(overflow[0]), int(cursor[0])


def test_online_update_joins_best_weighted_neighbour():
    # reference test_state.py:239-267
    state = _small_state()
    state.community_weight[0, :2] = torch.tensor([0.2, 0.8])
    key = torch.zeros(128, dtype=torch.bfloat16)
    key[:4] = torch.tensor([3.0, 5.0, 7.0, 9.0], dtype=torch.bfloat16)
    assigned, overflow, cursor = _run_update(
        state, [2.0, 1.5, 0.5, -1.0], [10, 11, 12, 13], 2.5, key, 20, 0.5
    )
    assert (assigned, overflow, cursor) == (0, 0, 21)
    assert state.community_counts.tolist() == [2]
    assert state.community_sizes[0, :2].tolist() == [3, 1]
    assert state.deltas.members(0, 0).tolist() == [20]
    expected = torch.tensor([5 / 3, 7 / 3, 3.0, 11 / 3]).to(torch.float8_e4m3fn).float()
    assert torch.equal(state.centroids[0, 0, :4].float(), expected)
    probabilities = np.exp(np.array([2.0, 1.5, 0.5, -1.0], np.float32) - np.float32(2.5))
    want = 0.2 + (probabilities[0] + probabilities[1]) * 0.25 + probabilities.sum() * 0.25
    assert abs(float(state.community_weight[0, 0]) - want) < 1e-6


def test_online_update_creates_singleton_without_positive_gain():
    # reference test_state.py:270-287
    state = _small_state()
    state.community_weight[0, :2] = 100.0
    key = torch.zeros(128, dtype=torch.bfloat16)
    key[:4] = torch.tensor([2.0, 4.0, 6.0, 8.0], dtype=torch.bfloat16)
    assigned, _, _ = _run_update(state, [1.0, 0.5], [4, 5], 2.0, key, 21, 1.0)
    assert assigned == 2
    assert state.community_counts.tolist() == [3]
    assert int(state.community_sizes[0, 2]) == 1
    assert state.centroids[0, 2, :4].float().tolist() == [2.0, 4.0, 6.0, 8.0]
    assert state.deltas.members(0, 2).tolist() == [21]


def test_online_update_with_a_forced_community():
    """The nearest-centroid variant hands the update the community to join (no reference counterpart):
    a live community replaces the rule's choice, anything else leaves the rule in charge."""

    key = torch.zeros(128, dtype=torch.bfloat16)
    key[:4] = torch.tensor([2.0, 4.0, 6.0, 8.0], dtype=torch.bfloat16)
    # the rule alone would open community 2 (no positive gain): forced into community 1 instead
    state = _small_state()
    state.community_weight[0, :2] = 100.0
    sizes_before = state.community_sizes[0, :2].tolist()
    assigned, overflow, cursor = _run_update(state, [1.0, 0.5], [4, 5], 2.0, key, 21, 1.0, forced=1)
    assert (assigned, overflow, cursor) == (1, 0, 22)
    assert state.community_counts.tolist() == [2]
    assert state.community_sizes[0, :2].tolist() == [sizes_before[0], sizes_before[1] + 1]
    assert state.deltas.members(0, 1).tolist()[0] == 21
    assert int(state.token_communities[0, 21]) == 1
    # a community that is not live (or -1) is ignored
    for forced in (2, 7, -1):
        state = _small_state()
        state.community_weight[0, :2] = 100.0
        assigned, _, _ = _run_update(state, [1.0, 0.5], [4, 5], 2.0, key, 21, 1.0, forced=forced)
        assert assigned == 2 and state.community_counts.tolist() == [3]


def test_online_update_survives_many_appends():
    # reference test_state.py:290-313 (scaled down for speed: 512 appends)
    steps = 512
    state = _small_state(capacity=steps + 2, decode=steps)
    state.community_weight[0, :2] = 100.0
    for step in range(steps):
        key = torch.full((128,), float(step % 200), dtype=torch.bfloat16)
        assigned, overflow, _ = _run_update(state, [1.0], [step], 1.5, key, 64_000 + step, 0.5)
        assert assigned == step + 2 and overflow == 0
    assert state.community_counts.tolist() == [steps + 2]
    assert int(state.deltas.next_free_chunk[0]) == steps
    assert int(state.deltas.next_free_position[0]) == steps
    assert state.deltas.members(0, steps + 1).tolist() == [64_000 + steps - 1]


# ---- fixtures generated from the reference (tests/golden/make_golden.py) ---------------------
def test_selection_matches_reference_helper(golden_dir):
    data = np.load(golden_dir / "selection.npz")
    assert np.array_equal(
        oracle.ordered_fp16_keys(data["key_probe"].astype(np.float16).view(np.uint16)).astype(np.int32),
        data["key_probe_keys"],
    )
    for case in data["cases"]:
        active, budget, filled = data[f"meta_{case}"].tolist()
        picked = oracle.select_descriptors(
            data[f"scores_{case}"], data[f"sizes_{case}"], active, budget
        )
        want = sorted(zip(data[f"ids_{case}"].tolist(), data[f"takes_{case}"].tolist()))
        got = _takes(picked)
        # same communities and take counts; the kernels emit them in index order
        # within the above-threshold and at-threshold classes
        assert sorted(got) == want, case
        assert int(picked.cumulative_ends[-1]) == filled
        keys = oracle.ordered_fp16_keys(data[f"scores_{case}"]).astype(np.int64)
        above = [c for c, _ in got if keys[c] > picked.threshold_key]
        equal = [c for c, _ in got if keys[c] == picked.threshold_key]
        assert above == sorted(above) and equal == sorted(equal)
        assert [c for c, _ in got] == above + equal


def test_tile_starts_match_reference_helper(golden_dir):
    data = np.load(golden_dir / "packing.npz")
    for case in data["cases"]:
        budget, sink = data[f"meta_{case}"].tolist()
        ends = data[f"ends_{case}"]
        counts = data[f"counts_{case}"]
        tiles = data[f"tiles_{case}"]
        for head in range(ends.shape[0]):
            got = oracle.tile_start_descriptors(ends[head], int(counts[head]), budget // 64, sink)
            assert got.tolist() == tiles[head].tolist(), (case, head)


def _delta_store(data, prefix: str) -> SimpleNamespace:
    names = (
        "positions", "chunk_start", "chunk_capacity", "chunk_size", "chunk_next",
        "chunk_previous", "community_head", "community_tail", "community_sizes",
        "next_free_chunk", "next_free_position",
    )
    return SimpleNamespace(**{name: torch.from_numpy(data[f"{prefix}{name}"]) for name in names})


def test_positions_match_reference_materialisation(golden_dir):
    data = np.load(golden_dir / "positions.npz")
    csr = SimpleNamespace(
        member_offsets=torch.from_numpy(data["offsets"]),
        member_positions=torch.from_numpy(data["member_positions"]),
    )
    deltas = _delta_store(data, "delta_")
    # our append() must rebuild the very same chunk pools
    graphs = int(data["meta"][0])
    mine = DecodeDeltaChunks.allocate(
        graph_count=graphs,
        community_capacity=deltas.community_head.shape[1],
        max_decode_tokens=deltas.chunk_start.shape[1],
    )
    for graph, community, position in data["appended"].tolist():
        mine.append(graph, community, position)
    for name in vars(deltas):
        assert torch.equal(getattr(mine, name), getattr(deltas, name)), name
    for query in data["queries"]:
        spec = data[f"query_{query}"]
        graph = int(spec[0, 0])
        communities = spec[1:, 0].astype(np.int32)
        ends = np.cumsum(spec[1:, 1]).astype(np.int32)
        total = int(ends[-1])
        budget = -(-(total + 1) // 64) * 64
        positions = oracle.resolve_positions(
            graph=graph,
            csr=csr,
            deltas=deltas,
            communities=communities,
            cumulative_ends=ends,
            count=len(communities),
            sink_positions=np.zeros(0, np.int32),
            current_position=7,
            token_budget=budget,
            num_sink=0,
        )
        assert positions[:total].tolist() == data[f"result_{query}"].tolist(), query


def test_online_update_matches_reference_helper(golden_dir):
    data = np.load(golden_dir / "online_update.npz")
    capacity, length, steps, dim, _ = data["meta"].tolist()
    state = MutableGraphState(
        centroids=torch.from_numpy(data["initial_centroids"].copy()).view(torch.float8_e4m3fn),
        community_sizes=torch.from_numpy(data["initial_sizes"].copy()),
        community_counts=torch.tensor([int(data["meta"][4])], dtype=torch.int32),
        community_weight=torch.from_numpy(data["initial_weight"].copy()),
        total_weight=torch.from_numpy(data["initial_total"].copy()),
        token_communities=torch.from_numpy(data["initial_labels"].copy()),
        deltas=DecodeDeltaChunks.allocate(
            graph_count=1, community_capacity=capacity, max_decode_tokens=steps
        ),
        retrieval_to_graph=torch.zeros(1, dtype=torch.int32),
        retrieval_to_kv=torch.zeros(1, dtype=torch.int32),
    )
    cache = torch.zeros((1, length + steps, dim), dtype=torch.bfloat16)
    cursor = torch.tensor([length], dtype=torch.int32)
    assigned = torch.zeros(1, dtype=torch.int32)
    overflow = torch.zeros(1, dtype=torch.int32)
    for step in range(steps):
        lse, lam = data[f"scalars_{step}"].tolist()
        cache[0, length + step] = torch.from_numpy(data[f"key_{step}"][0]).to(torch.bfloat16)
        # the generator perturbs the weights before some steps; replay that
        state.community_weight.copy_(torch.from_numpy(data[f"weight_before_{step}"]))
        oracle.online_update(
            state=state,
            retrieval_head=0,
            graph=0,
            kv_head=0,
            topk_scores=data[f"scores_{step}"],
            topk_positions=data[f"positions_{step}"],
            representative_lse=np.float32(lse),
            key_cache=cache,
            current_position=cursor,
            lam=float(lam),
            assigned_out=assigned,
            overflow_out=overflow,
        )
        assert assigned.tolist() == data[f"assigned_{step}"].tolist(), step
        assert int(overflow[0]) == 0 and int(cursor[0]) == length + step + 1
        assert state.community_counts.tolist() == data[f"counts_{step}"].tolist()
        assert np.array_equal(state.community_sizes.numpy(), data[f"sizes_{step}"])
        assert np.array_equal(state.token_communities.numpy(), data[f"labels_{step}"])
        assert np.array_equal(state.centroids.view(torch.uint8).numpy(), data[f"centroids_{step}"]), step
        np.testing.assert_allclose(state.community_weight.numpy(), data[f"weight_{step}"], rtol=2e-6, atol=1e-7)
        np.testing.assert_allclose(state.total_weight.numpy(), data[f"total_{step}"], rtol=2e-6)
    final = _delta_store(data, "final_delta_")
    for name in vars(final):
        assert torch.equal(getattr(state.deltas, name), getattr(final, name)), name


# ---- internal consistency of the floating-point half ---------------------------------------
def test_fixed_dot_is_close_to_float64_and_order_stable():
    rng = np.random.default_rng(3)
    left = torch.from_numpy(rng.normal(size=(5, 128)).astype(np.float32)).to(torch.bfloat16).float().numpy()
    right = torch.from_numpy(rng.normal(size=(7, 128)).astype(np.float32)).to(torch.bfloat16).float().numpy()
    got = oracle.fixed_dot(left[:, None, :], right[None, :, :])
    want = left.astype(np.float64) @ right.astype(np.float64).T
    np.testing.assert_allclose(got, want, rtol=0, atol=2e-5)
    assert got.dtype == np.float32
    exact = oracle.fixed_dot(np.ones((1, 128), np.float32), np.arange(128, dtype=np.float32)[None])
    assert float(exact[0]) == 127 * 64


def test_attention_unit_matches_dense_softmax():
    rng = np.random.default_rng(4)
    tokens, group = 256, 4
    q = torch.from_numpy(rng.normal(size=(group, 128)).astype(np.float32)).to(torch.bfloat16).float().numpy()
    k = torch.from_numpy((rng.normal(size=(tokens, 128)) / 11.3).astype(np.float32)).to(torch.bfloat16).float().numpy()
    v = torch.from_numpy((rng.normal(size=(tokens, 128)) / 11.3).astype(np.float32)).to(torch.bfloat16).float().numpy()
    valid = np.ones(tokens, bool)
    valid[100:130] = False
    out, lse, scores = oracle.attention_unit(
        query_group=q, key_rows=k, value_rows=v, valid=valid, softmax_scale=0.088
    )
    dense = (q.astype(np.float64) @ k.astype(np.float64).T) * 0.088
    dense[:, ~valid] = -np.inf
    weights = np.exp(dense - dense.max(axis=1, keepdims=True))
    want = (weights / weights.sum(axis=1, keepdims=True)) @ v.astype(np.float64)
    np.testing.assert_allclose(out, want, atol=2e-3)
    np.testing.assert_allclose(lse, np.log(weights.sum(axis=1)) + dense.max(axis=1), atol=1e-4)
    top_scores, top_positions = oracle.global_topk(
        scores[0], np.where(valid, np.arange(tokens) * 3, -1).astype(np.int32), np.arange(tokens) < 5
    )
    order = np.argsort(-np.where(valid & (np.arange(tokens) >= 5), scores[0], -np.inf), kind="stable")[:8]
    assert top_positions.tolist() == (order * 3).tolist()
    assert np.array_equal(top_scores, scores[0][order])


# ---- edge list -> adjacency ---------------------------------------------------------------------
def test_adjacency_oracle_known_answers_of_the_reference_tests():
    """tests/community_kv/graph/test_partition.py:212-248 of the reference."""

    from oracle.adjacency_oracle import build_adjacency

    indices = np.array([[[1, 2], [2, 1]]], dtype=np.int32)
    source, destination, weight = build_adjacency(indices, np.ones_like(indices, dtype=np.float32),
                                                  np.array([[2, 3]]), seq_len=4, lam=1.0)
    assert {(int(a), int(b)): float(w) for a, b, w in zip(source, destination, weight)} == {
        (1, 2): 0.5, (2, 2): 0.5, (1, 3): 0.5, (2, 3): 0.5}
    indices = np.array([[[1, 4], [-1, 5]]], dtype=np.int32)
    source, destination, weight = build_adjacency(indices, np.ones_like(indices, dtype=np.float32),
                                                  np.array([[2, 3]]), seq_len=4, lam=0.5)
    assert {(int(a), int(b)): float(w) for a, b, w in zip(source, destination, weight)} == {
        (1, 1): 0.5, (1, 2): 0.25}


def test_adjacency_oracle_matches_reference_fixture(golden_dir):
    from community_kv_b200.assembly import reshape_by_aggregation
    from oracle.adjacency_oracle import build_adjacency

    data = np.load(golden_dir / "adjacency.npz")
    for case in data["cases"].tolist():
        length, lam = int(data[f"scalars_{case}"][0]), float(data[f"scalars_{case}"][1])
        source, destination, weight = build_adjacency(data[f"indices_{case}"], data[f"scores_{case}"],
                                                      data[f"positions_{case}"], seq_len=length, lam=lam)
        assert np.array_equal(source, data[f"source_{case}"]), case
        assert np.array_equal(destination, data[f"destination_{case}"]), case
        assert np.array_equal(weight.view(np.int32), data[f"weight_{case}"].view(np.int32)), case
    heads, kv_heads, rows, kappa, sink = data["reshape_meta"].tolist()
    indices = torch.from_numpy(data["reshape_inputs_indices"])
    scores = torch.from_numpy(data["reshape_inputs_scores"])
    for index, mode in enumerate(("per_query_head", "query_group", "layer_wise")):
        shaped = reshape_by_aggregation(indices, scores, aggregation=mode, num_kv_heads=kv_heads, num_sink=sink)
        assert np.array_equal(shaped[0].numpy(), data[f"reshape_indices_{index}"]), mode
        assert np.array_equal(shaped[1].numpy(), data[f"reshape_scores_{index}"]), mode
        assert np.array_equal(shaped[2].numpy(), data[f"reshape_positions_{index}"]), mode

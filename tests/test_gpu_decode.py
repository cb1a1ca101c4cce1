"""Parity of the CUDA decode path (through the C ABI) against the CPU oracle."""

from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

from community_kv_b200 import native, ops
from community_kv_b200.batched import BatchedDecodeRuntime
from community_kv_b200.config import CommunityKVConfig, GraphAggregation
from community_kv_b200.runtime import DecodeRuntime, convert_prefill_tensors
from community_kv_b200.state import DecodeLayerWorkspace
from community_kv_b200.synthetic import make_layer, make_query
from tests.helpers import OracleLayer, assert_state_equal, assert_step_equal, fp16_ulp_distance

pytestmark = pytest.mark.gpu
SCALE = 128 ** -0.5


def _cover(converted):
    capacity = converted.mutable.community_capacity
    return [min(capacity, c + converted.decode_capacity) for c in converted.initial_community_counts]


def _run_sequence(layer, config, steps, *, seed, integer=False, splits=None, defer_update=False,
                  exact_scores=False, max_communities=0):

    device = torch.device("cuda", 0)
    runtime = DecodeRuntime(config, splits=splits, defer_update=defer_update, max_communities=max_communities)
    state = runtime.prepare_layer(0, **layer.to(device).prepare_kwargs())
    twin = OracleLayer(
        state.converted.csr,
        state.converted.mutable,
        state.converted.current_position,
        token_budget=state.workspace.selection.token_budget,
        num_sink=config.num_sink,
        cover=_cover(state.converted),
        max_communities=max_communities,
    )
    key = layer.key.to(device)[None]
    value = layer.value.to(device)[None]
    for step in range(steps):
        query = make_query(seed=seed + step, query_heads=layer.query_heads, integer_valued=integer)
        out = runtime.decode(
            layer_idx=0,
            query=query.to(device)[None, :, None, :],
            key=key,
            value=value,
            softmax_scale=SCALE,
        )
        assert out.shape == (1, 1, layer.query_heads, 128)
        runtime.synchronize_updates()
        where = f"step {step}"
        if exact_scores:  # the device scores themselves, bit for bit, where the scan covers them
            cover = torch.as_tensor(twin.cover)[:, None]
            covered = torch.arange(twin.scores.shape[1])[None, :] < cover
            want_scores = twin.exact_scores(query)
            got_scores = state.workspace.selection.scores.cpu()
            assert torch.equal(got_scores.view(torch.int16)[covered], want_scores.view(torch.int16)[covered]), where
        want = twin.step(query=query, key=layer.key, value=layer.value, softmax_scale=SCALE, lam=config.lam,
                         device_scores=state.workspace.selection.scores, assignment=config.online_assignment)
        assert_step_equal(
            selection=state.workspace.selection,
            attention=state.workspace.attention,
            update=state.workspace.update,
            result=want,
            where=where,
        )
        assert_state_equal(state.converted.mutable, twin.state, where)
        assert torch.equal(state.converted.current_position.cpu(), twin.current), where
    runtime.assert_no_overflow()
    return state, twin


@pytest.mark.parametrize(
    "aggregation", [GraphAggregation.QUERY_GROUP, GraphAggregation.PER_QUERY_HEAD, GraphAggregation.LAYER_WISE]
)
def test_single_layer_config0_parity(aggregation):
    """Single-layer configuration: ctx 8192, 32/8 heads, 64 planted clusters, budget 1024."""

    layer = make_layer(seed=0, seq_len=8192, communities=64, max_decode_tokens=8, aggregation=aggregation)
    config = CommunityKVConfig(token_budget=1024, num_sink=10, lam=0.5, aggregation=aggregation)
    _run_sequence(layer, config, steps=4, seed=100)


def test_unfused_kernels_give_the_same_result(monkeypatch):
    """The four stand-alone kernels and the single cluster launch are the same path."""

    monkeypatch.setenv("CKV_UNFUSED", "1")
    layer = make_layer(seed=0, seq_len=8192, communities=64, max_decode_tokens=8, aggregation="query_group")
    config = CommunityKVConfig(token_budget=1024, num_sink=10, lam=0.5, aggregation="query_group")
    _run_sequence(layer, config, steps=4, seed=100)


@pytest.mark.parametrize("unfused", [False, True])
def test_fixed_order_scores_are_bit_exact(monkeypatch, unfused):
    """``CKV_TENSOR_SCORES=0``: the CUDA-core scoring path sums in the fixed order the CPU restatement
    reproduces, so the fp16 scores themselves (and with them everything else) match bit for bit."""

    monkeypatch.setenv("CKV_TENSOR_SCORES", "0")
    assert not ops.tensor_scores_enabled()
    if unfused:
        monkeypatch.setenv("CKV_UNFUSED", "1")
    layer = make_layer(seed=13, seq_len=16384, communities=700, max_decode_tokens=8, zipf_exponent=1.1)
    config = CommunityKVConfig(token_budget=1024, num_sink=10, lam=0.5, aggregation="query_group")
    _run_sequence(layer, config, steps=6, seed=1300)
    layer = make_layer(seed=0, seq_len=8192, communities=64, max_decode_tokens=8, aggregation="per_query_head")
    config = CommunityKVConfig(token_budget=1024, num_sink=10, lam=0.5, aggregation="per_query_head")
    _run_sequence(layer, config, steps=3, seed=100)


@pytest.mark.parametrize("unfused", [False, True])
def test_tensor_core_scores(monkeypatch, unfused):
    """Scoring on the tensor cores (single cluster launch and the stand-alone kernels): scores within one
    fp16 unit in the last place of the fixed-order ones, the rest of the step exact given those scores."""

    monkeypatch.setenv("CKV_TENSOR_SCORES", "1")
    assert ops.tensor_scores_enabled()
    if unfused:
        monkeypatch.setenv("CKV_UNFUSED", "1")
    layer = make_layer(seed=11, seq_len=16384, communities=700, max_decode_tokens=8, zipf_exponent=1.1)
    config = CommunityKVConfig(token_budget=1024, num_sink=10, lam=0.5, aggregation="query_group")
    _run_sequence(layer, config, steps=6, seed=1100)
    layer = make_layer(seed=12, kv_heads=2, group_size=8, seq_len=4096, communities=100, max_decode_tokens=4)
    config = CommunityKVConfig(token_budget=512, num_sink=4, lam=0.5, aggregation="query_group")
    _run_sequence(layer, config, steps=3, seed=1200, splits=3)


@pytest.mark.parametrize("aggregation", [GraphAggregation.QUERY_GROUP, GraphAggregation.LAYER_WISE])
def test_deferred_update_gives_the_same_result(aggregation):
    """Attention on the caller's stream, online assignment on a second stream: same step, same state."""

    layer = make_layer(seed=21, seq_len=8192, communities=200, max_decode_tokens=10, aggregation=aggregation,
                       zipf_exponent=1.1)
    config = CommunityKVConfig(token_budget=1024, num_sink=10, lam=0.5, aggregation=aggregation)
    _run_sequence(layer, config, steps=8, seed=2100, defer_update=True)


@pytest.mark.parametrize(
    "aggregation,defer", [(GraphAggregation.QUERY_GROUP, False), (GraphAggregation.QUERY_GROUP, True),
                          (GraphAggregation.PER_QUERY_HEAD, False), (GraphAggregation.LAYER_WISE, False)]
)
def test_nearest_centroid_assignment_variant(aggregation, defer):
    """Not in the reference: every decoded token joins the community whose centroid is nearest to its key
    (largest inner product, first maximum).  State and outputs against the CPU restatement, bit for bit;
    the variant never opens a community, and its choices differ from the modularity rule's."""

    layer = make_layer(seed=23, seq_len=8192, communities=96, max_decode_tokens=12, aggregation=aggregation,
                       zipf_exponent=1.1)
    config = CommunityKVConfig(token_budget=1024, num_sink=10, lam=0.5, aggregation=aggregation,
                               online_assignment="nearest_centroid")
    before = layer.to(torch.device("cuda", 0)).prepare_kwargs()["num_communities"].clone()
    state, twin = _run_sequence(layer, config, steps=10, seed=2300, defer_update=defer)
    counts = state.converted.mutable.community_counts
    assert int(counts.max()) == int(before.max()) and int(counts.min()) == int(before.min())
    with pytest.raises(ValueError):
        CommunityKVConfig(online_assignment="nearest")


@pytest.mark.parametrize("aggregation", [GraphAggregation.QUERY_GROUP, GraphAggregation.LAYER_WISE])
def test_fp32_centroid_table(aggregation):
    """Not the reference's layout: the centroid table in fp32.  The scores (fixed-order sum of products
    rounded one by one), everything downstream and the unquantised running mean against the CPU
    restatement, bit for bit; the call runs the four stand-alone kernels."""

    layer = make_layer(seed=29, seq_len=8192, communities=80, max_decode_tokens=10, aggregation=aggregation)
    table = layer.assembled.centroids.float()
    generator = torch.Generator().manual_seed(291)
    layer.assembled.centroids = table * 1.0009765625 + 1e-3 * torch.randn(table.shape, generator=generator)
    config = CommunityKVConfig(token_budget=1024, num_sink=10, lam=0.5, aggregation=aggregation,
                               centroid_dtype="fp32")
    with pytest.raises(TypeError, match="FP8"):  # the reference's layout unless asked otherwise
        convert_prefill_tensors(**layer.prepare_kwargs())
    state, twin = _run_sequence(layer, config, steps=8, seed=2900, exact_scores=True)
    assert state.converted.mutable.centroids.dtype == torch.float32
    assert native.library().ckv_decode_layer_kernels(ctypes.byref(state.args)) >= 4


def test_single_layer_configuration_as_worded():
    """The single-layer configuration to the letter: ctx 8192, 32 / 8 heads, 64 planted clusters, the
    centroids the per-community mean keys in fp32, the eight best communities per KV head, budget 1024.
    Scores, selection, attention output, neighbour candidates and the online update against the CPU
    restatement (scores and state bit for bit)."""

    layer = make_layer(seed=0, seq_len=8192, communities=64, max_decode_tokens=8, aggregation="query_group")
    assembled = layer.assembled
    heads, capacity, _ = assembled.centroids.shape
    labels = assembled.token_communities[:, : layer.prefill_seq_len].long()  # [graphs, S]
    means = torch.zeros((heads, capacity, 128), dtype=torch.float32)
    for head in range(heads):
        graph, kv = int(assembled.retrieval_to_graph[head]), int(assembled.retrieval_to_kv[head])
        keep = torch.arange(layer.prefill_seq_len) >= 10  # the ten sink positions are not members
        means[head].index_add_(0, labels[graph][keep], layer.key[kv, : layer.prefill_seq_len][keep].float())
        sizes = assembled.community_sizes[head].clamp(min=1).float()
        means[head] /= sizes[:, None]
    assembled.centroids = means
    config = CommunityKVConfig(token_budget=1024, num_sink=10, lam=0.5, aggregation="query_group",
                               centroid_dtype="fp32")
    state, _ = _run_sequence(layer, config, steps=4, seed=100, exact_scores=True, max_communities=8)
    assert int(state.workspace.selection.descriptor_counts.max()) <= 8


def test_many_small_communities_and_delta_chains():
    """Mean community size ~16 (the tuned regime): many descriptors, decode deltas get re-selected."""

    layer = make_layer(seed=1, kv_heads=2, seq_len=4096, communities=256, max_decode_tokens=24)
    config = CommunityKVConfig(token_budget=512, num_sink=4, lam=0.5, aggregation="query_group")
    state, twin = _run_sequence(layer, config, steps=24, seed=200, splits=4)
    assert int(state.converted.mutable.deltas.community_sizes.sum()) == 24 * 2


def test_integer_fixture_is_exact_end_to_end():
    """Small-integer operands: every fp32 sum is exact, so even the bf16 output must match closely."""

    layer = make_layer(seed=2, kv_heads=2, seq_len=2048, communities=32, max_decode_tokens=6, integer_valued=True)
    config = CommunityKVConfig(token_budget=256, num_sink=2, lam=0.25, aggregation="query_group")
    _run_sequence(layer, config, steps=6, seed=300, integer=True, splits=2)


@pytest.mark.parametrize("group_size,kv_heads", [(1, 4), (2, 4), (5, 2), (8, 2), (12, 1), (16, 1)])
def test_group_sizes(group_size, kv_heads):
    layer = make_layer(seed=3 + group_size, kv_heads=kv_heads, group_size=group_size, seq_len=2048,
                       communities=48, max_decode_tokens=4)
    config = CommunityKVConfig(token_budget=256, num_sink=3, lam=0.5, aggregation="query_group")
    _run_sequence(layer, config, steps=2, seed=400 + group_size, splits=1)


def test_zipf_communities_full_context_unit():
    """One (sequence, layer) of the batched long-context configuration: ctx 131072, 4096 Zipf communities, budget 2048."""

    layer = make_layer(seed=5, seq_len=131072, communities=4096, max_decode_tokens=4, zipf_exponent=1.1)
    config = CommunityKVConfig(token_budget=2048, num_sink=10, lam=0.5, aggregation="query_group")
    _run_sequence(layer, config, steps=2, seed=500)


def test_config3_layer_with_online_assignment():
    """One layer of the whole-model configuration: ctx 32768, 512 Zipf(1.1) communities per KV head,
    budget 2048, every decoded token assigned online (eight steps)."""

    layer = make_layer(seed=7, seq_len=32768, communities=512, max_decode_tokens=12, zipf_exponent=1.1)
    config = CommunityKVConfig(token_budget=2048, num_sink=10, lam=0.5, aggregation="query_group")
    _run_sequence(layer, config, steps=8, seed=700)


def test_batched_sequences_match_per_sequence_oracle():
    device = torch.device("cuda", 0)
    config = CommunityKVConfig(token_budget=512, num_sink=10, lam=0.5, aggregation="query_group")
    layers = [
        make_layer(seed=10 + b, kv_heads=4, seq_len=4096, communities=96 + 16 * b, max_decode_tokens=6,
                   zipf_exponent=1.1 if b % 2 else None)
        for b in range(3)
    ]
    runtime = BatchedDecodeRuntime(config, splits=2)
    converted = [convert_prefill_tensors(**layer.to(device).prepare_kwargs()) for layer in layers]
    state = runtime.prepare_layer(0, converted)
    twins = []
    for b in range(3):
        csr, mutable, current = state.sequence_view(b)
        twins.append(
            OracleLayer(csr, mutable, current, token_budget=state.token_budget, num_sink=config.num_sink,
                        cover=state.workspace.selection.score_cover[b].cpu().tolist())
        )
    key = torch.stack([layer.key for layer in layers]).to(device)
    value = torch.stack([layer.value for layer in layers]).to(device)
    for step in range(5):
        queries = torch.stack([make_query(seed=600 + 10 * step + b, query_heads=16) for b in range(3)])
        out = runtime.decode(layer_idx=0, query=queries.to(device), key=key, value=value, softmax_scale=SCALE)
        assert out.shape == (3, 16, 128)
        for b in range(3):
            want = twins[b].step(query=queries[b], key=layers[b].key, value=layers[b].value,
                                 softmax_scale=SCALE, lam=config.lam,
                                 device_scores=state.workspace.selection.scores[b])
            ws = state.workspace
            view = lambda obj, names: type("V", (), {n: getattr(obj, n)[b] for n in names})
            assert_step_equal(
                selection=view(ws.selection, ["scores", "descriptor_counts", "communities", "cumulative_ends",
                                               "tile_descriptors", "positions"]),
                attention=view(ws.attention, ["output", "lse", "topk_positions", "topk_scores"]),
                update=view(ws.update, ["assigned_communities", "overflow"]),
                result=want,
                where=f"step {step} seq {b}",
            )
            _, mutable, current = state.sequence_view(b)
            assert_state_equal(mutable, twins[b].state, f"step {step} seq {b}")
            assert torch.equal(current.cpu(), twins[b].current)
    runtime.assert_no_overflow()


def test_standalone_entry_points_and_skip_update():
    """score -> select -> attention as three separate C-ABI calls, without the online update."""

    device = torch.device("cuda", 0)
    layer = make_layer(seed=20, kv_heads=2, seq_len=2048, communities=40, max_decode_tokens=4)
    config = CommunityKVConfig(token_budget=256, num_sink=5, lam=0.5, aggregation="query_group")
    converted = convert_prefill_tensors(**layer.to(device).prepare_kwargs())
    ws = DecodeLayerWorkspace.allocate(
        retrieval_head_count=2, graph_count=2, group_size=4, community_capacity=converted.mutable.community_capacity,
        token_budget=256, num_sink=5, dtype=torch.bfloat16, device=device, splits=2,
    )
    sinks = torch.arange(5, dtype=torch.int32, device=device)
    twin = OracleLayer(converted.csr, converted.mutable, converted.current_position, token_budget=256,
                       num_sink=5, cover=None)
    query = make_query(seed=21, query_heads=8)
    mutable = converted.mutable
    ops.score_centroids(query=query.to(device), centroids=mutable.centroids,
                        community_sizes=mutable.community_sizes, community_counts=mutable.community_counts,
                        workspace=ws.selection)
    segments = ops.select_weighted_descriptors_auto(
        community_sizes=mutable.community_sizes, community_counts=mutable.community_counts,
        workspace=ws.selection, csr=converted.csr, state=mutable, sink_positions=sinks,
        current_position=converted.current_position)
    ws.selection.positions.fill_(-7)  # the attention entry point must resolve positions itself
    ops.segmented_attention(
        query=query.to(device), key=layer.key.to(device), value=layer.value.to(device), csr=converted.csr,
        deltas=mutable.deltas, segments=segments, sink_positions=sinks,
        current_position=converted.current_position, softmax_scale=SCALE, workspace=ws.attention,
        update_state=mutable, update_workspace=None, update_lam=0.5, positions=ws.selection.positions)
    want = twin.step(query=query, key=layer.key, value=layer.value, softmax_scale=SCALE, lam=0.5, update=False,
                     device_scores=ws.selection.scores)
    assert_step_equal(selection=ws.selection, attention=ws.attention, update=ws.update, result=want,
                      check_update=False)
    assert_state_equal(mutable, twin.state, "skip-update leaves the state untouched")
    assert int(converted.current_position[0]) == 2048


def test_topk_communities_mode_and_underfill():
    """Extension (top-k communities under a token budget): at most k communities; unfilled slots are masked."""

    device = torch.device("cuda", 0)
    config = CommunityKVConfig(token_budget=1024, num_sink=10, lam=0.5, aggregation="query_group")
    layer = make_layer(seed=30, kv_heads=4, seq_len=8192, communities=64, max_decode_tokens=4)
    converted = [convert_prefill_tensors(**layer.to(device).prepare_kwargs())]
    runtime = BatchedDecodeRuntime(config)
    state = runtime.prepare_layer(0, converted, max_communities=5)
    csr, mutable, current = state.sequence_view(0)
    twin = OracleLayer(csr, mutable, current, token_budget=1024, num_sink=10,
                       cover=state.workspace.selection.score_cover[0].cpu().tolist(), max_communities=5)
    key = layer.key.to(device)[None]
    value = layer.value.to(device)[None]
    for step in range(3):
        query = make_query(seed=700 + step, query_heads=16)
        runtime.decode(layer_idx=0, query=query.to(device)[None], key=key, value=value, softmax_scale=SCALE)
        want = twin.step(query=query, key=layer.key, value=layer.value, softmax_scale=SCALE, lam=0.5,
                         device_scores=state.workspace.selection.scores[0])
        ws = state.workspace
        view = lambda obj, names: type("V", (), {n: getattr(obj, n)[0] for n in names})
        assert int(ws.selection.descriptor_counts.max()) <= 5
        assert int((ws.selection.positions == -1).sum()) > 0  # 5 of 64 clusters cannot fill 1013 slots
        assert_step_equal(
            selection=view(ws.selection, ["scores", "descriptor_counts", "communities", "cumulative_ends",
                                           "tile_descriptors", "positions"]),
            attention=view(ws.attention, ["output", "lse", "topk_positions", "topk_scores"]),
            update=view(ws.update, ["assigned_communities", "overflow"]),
            result=want, where=f"step {step}")
        assert_state_equal(state.sequence_view(0)[1], twin.state, f"step {step}")


def test_overflow_flags_stop_the_cursor():
    """Exhaust the decode-delta pools on purpose: flags are raised, the cursor stops, nothing faults."""

    layer = make_layer(seed=40, kv_heads=1, seq_len=1024, communities=16, max_decode_tokens=2)
    config = CommunityKVConfig(token_budget=128, num_sink=2, lam=0.5, aggregation="query_group")
    device = torch.device("cuda", 0)
    runtime = DecodeRuntime(config, splits=1)
    state = runtime.prepare_layer(0, **layer.to(device).prepare_kwargs())
    twin = OracleLayer(state.converted.csr, state.converted.mutable, state.converted.current_position,
                       token_budget=128, num_sink=2, cover=_cover(state.converted))
    key, value = layer.key.to(device)[None], layer.value.to(device)[None]
    for step in range(4):
        query = make_query(seed=800 + step, query_heads=4)
        runtime.decode(layer_idx=0, query=query.to(device)[None, :, None, :], key=key, value=value,
                       softmax_scale=SCALE)
        want = twin.step(query=query, key=layer.key, value=layer.value, softmax_scale=SCALE, lam=0.5,
                         device_scores=state.workspace.selection.scores)
        assert torch.equal(state.workspace.update.overflow.cpu(), want.overflow), step
        assert_state_equal(state.converted.mutable, twin.state, f"step {step}")
        assert torch.equal(state.converted.current_position.cpu(), twin.current)
    with pytest.raises(RuntimeError, match="overflow"):
        runtime.assert_no_overflow()


def test_full_cache_masks_the_cursor_row():
    """Once the cache is full the cursor equals its capacity: the update reports it (overflow bit 8) and
    the attention treats that slot as masked instead of reading one row past the head's slice."""

    device = torch.device("cuda", 0)
    layer = make_layer(seed=41, kv_heads=2, seq_len=1024, communities=16, max_decode_tokens=3).to(device)
    config = CommunityKVConfig(token_budget=128, num_sink=2, lam=0.5, aggregation="query_group")
    runtime = DecodeRuntime(config, splits=2)
    state = runtime.prepare_layer(0, **layer.prepare_kwargs())
    rows = 1024 + 2  # a cache that ends two rows after the prompt
    key = layer.key[:, :rows].contiguous()[None]
    value = layer.value[:, :rows].contiguous()[None]
    # poison what lies right behind the last head's slice: it must never be read
    for step in range(4):
        query = make_query(seed=810 + step, query_heads=8).to(device)
        out = runtime.decode(layer_idx=0, query=query[None, :, None, :], key=key, value=value, softmax_scale=SCALE)
        assert torch.isfinite(out.float()).all(), step
        flags = state.workspace.update.overflow.cpu()
        cursor = state.converted.current_position.cpu()
        if step < 2:
            assert int(flags.max()) == 0 and int(cursor.min()) == 1024 + step + 1
        else:
            assert bool(((flags & 8) == 8).all()) and int(cursor.max()) == rows
            # every slot of the budget is a cached row or masked, never the row at the capacity
            assert int(state.workspace.selection.positions.max()) <= rows
    with pytest.raises(RuntimeError, match="overflow"):
        runtime.assert_no_overflow()


def test_shape_errors_are_reported_before_launch():
    device = torch.device("cuda", 0)
    layer = make_layer(seed=50, kv_heads=1, seq_len=1024, communities=16, max_decode_tokens=2)
    config = CommunityKVConfig(token_budget=128, num_sink=2)
    runtime = DecodeRuntime(config)
    runtime.prepare_layer(0, **layer.to(device).prepare_kwargs())
    with pytest.raises(ValueError, match="query shape"):
        runtime.decode(layer_idx=0, query=torch.zeros((1, 4, 2, 128), device=device, dtype=torch.bfloat16),
                       key=layer.key.to(device)[None], value=layer.value.to(device)[None], softmax_scale=SCALE)
    with pytest.raises(RuntimeError, match="not prepared"):
        runtime.decode(layer_idx=3, query=torch.zeros((1, 4, 1, 128), device=device, dtype=torch.bfloat16),
                       key=layer.key.to(device)[None], value=layer.value.to(device)[None], softmax_scale=SCALE)


def test_append_kv_rows():
    """ckv_append_kv: one row per (sequence, head) into both caches, scalar and per-unit index."""

    device = torch.device("cuda", 0)
    torch.manual_seed(5)
    key = torch.randn((3, 2, 40, 128), device=device).to(torch.bfloat16)
    value = torch.randn_like(key)
    new_key = torch.randn((3, 2, 128), device=device).to(torch.bfloat16)
    new_value = torch.randn_like(new_key)
    want_key, want_value = key.clone(), value.clone()
    want_key[:, :, 17] = new_key
    want_value[:, :, 17] = new_value
    ops.append_kv(key, value, new_key, new_value, 17)
    assert torch.equal(key, want_key) and torch.equal(value, want_value)
    rows = torch.tensor([0, 39, -1, 5, 5, 12], dtype=torch.int32, device=device)
    for unit, row in enumerate(rows.tolist()):
        if row >= 0:
            want_key.view(6, 40, 128)[unit, row] = new_key.view(6, 128)[unit]
            want_value.view(6, 40, 128)[unit, row] = new_value.view(6, 128)[unit]
    ops.append_kv(key, value, new_key, new_value, rows)
    assert torch.equal(key, want_key) and torch.equal(value, want_value)
    with pytest.raises(ValueError):
        ops.append_kv(key, value, new_key, new_value, 40)


def test_full_size_batch_one_launch_equals_four_kernels():
    """The batched long-context configuration as far as one layer goes (8 sequences x 8 KV heads at ctx 131072,
    1024-4096 Zipf communities, budget 2048): the single cluster launch and the four
    stand-alone kernels, fed the same inputs for three steps, leave bit-identical
    workspaces and graph state (one unit of this size is checked against the CPU oracle
    by ``test_zipf_communities_full_context_unit``)."""

    from dataclasses import fields

    from community_kv_b200 import native
    from community_kv_b200.workload import build_decode_workload

    device = torch.device("cuda", 0)

    def build():
        return build_decode_workload(
            layers=1, batch=8, kv_heads=8, group_size=4, seq_len=131072, communities=(1024, 4096),
            token_budget=2048, num_sink=10, max_decode_tokens=8, device=device, seed=3, zipf_exponent=1.1)

    fused, plain = build(), build()
    generator = torch.Generator(device=device).manual_seed(1)
    stream = native.current_stream(device)

    def tensors(obj):
        found = {}
        for item in fields(obj):
            value = getattr(obj, item.name)
            if isinstance(value, torch.Tensor):
                found[item.name] = value
            elif hasattr(value, "__dataclass_fields__"):
                found.update({f"{item.name}.{k}": v for k, v in tensors(value).items()})
        return found

    for step in range(3):
        query = torch.randn((8, 32, 128), generator=generator, device=device).to(torch.bfloat16)
        for work, flag in ((fused, 0), (plain, native.FLAG_UNFUSED)):
            args = work.runtime.pack(0, query=query, key=work.key[0], value=work.value[0], softmax_scale=SCALE)
            args.flags = (args.flags & ~native.FLAG_UNFUSED) | flag
            assert native.library().ckv_decode_layer_kernels(args) == (4 if flag else 1)
            native.call("ckv_decode_layer", args, stream)
        torch.cuda.synchronize()
        left, right = fused.state(0), plain.state(0)
        for name, a in {**tensors(left.workspace), **tensors(left.mutable)}.items():
            b = {**tensors(right.workspace), **tensors(right.mutable)}[name]
            if name.endswith(("partials", "partial_topk_packed", "score_cover")) or not a.numel():
                continue
            same = torch.equal(a.view(torch.uint8) if a.dtype == torch.float8_e4m3fn else a, b.view(torch.uint8) if b.dtype == torch.float8_e4m3fn else b)
            if not same and a.is_floating_point():  # NaN-free by construction; compare bits
                same = torch.equal(a.contiguous().view(torch.int16 if a.element_size() == 2 else torch.int32),
                                   b.contiguous().view(torch.int16 if b.element_size() == 2 else torch.int32))
            assert same, f"step {step}: {name} differs between the two paths"
        assert torch.equal(left.current_position, right.current_position)
    fused.runtime.assert_no_overflow()

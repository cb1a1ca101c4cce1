"""The allocation-free attention entry point against the regular one.

Collected last on purpose (file name): if it fails, a run that stops at the
first failure has already exercised every other test.

Who needs this entry point: hosts that are not allowed to call the device
allocator - their memory was handed out at start-up, or they run inside memory
that belongs to another component - so they cannot supply the scratch tensors
the regular call takes.  The check: same inputs, two calls in a row with
different queries, outputs of both entry points must be identical.
"""

from __future__ import annotations

import pytest
import torch

from community_kv_b200 import native, ops
from community_kv_b200.runtime import convert_prefill_tensors
from community_kv_b200.state import DecodeLayerWorkspace
from community_kv_b200.synthetic import make_layer, make_query

pytestmark = pytest.mark.gpu


def test_static_scratch_entry_point_matches_the_regular_one():
    device = torch.device("cuda", 0)
    budget, sinks = 512, 6
    layer = make_layer(seed=77, kv_heads=4, seq_len=4096, communities=80, max_decode_tokens=4)
    converted = convert_prefill_tensors(**layer.to(device).prepare_kwargs())
    state = converted.mutable

    def workspace():
        return DecodeLayerWorkspace.allocate(
            retrieval_head_count=4, graph_count=4, group_size=4,
            community_capacity=state.community_capacity, token_budget=budget, num_sink=sinks,
            dtype=torch.bfloat16, device=device, splits=4,
        )

    regular, static = workspace(), workspace()
    assert regular.attention.splits <= native.STATIC_MAX_SPLITS
    sink_positions = torch.arange(sinks, dtype=torch.int32, device=device)
    key, value = layer.key.to(device), layer.value.to(device)
    common = dict(
        key=key, value=value, csr=converted.csr, deltas=state.deltas, sink_positions=sink_positions,
        current_position=converted.current_position, softmax_scale=128**-0.5,
        update_state=state, update_workspace=None, update_lam=0.5,
    )
    for call in range(2):
        query = make_query(seed=900 + call, query_heads=16).to(device)
        segments = ops.score_and_select(
            query=query, centroids=state.centroids, community_sizes=state.community_sizes,
            community_counts=state.community_counts, workspace=regular.selection, csr=converted.csr,
            state=state, sink_positions=sink_positions, current_position=converted.current_position,
        )
        ops.segmented_attention(
            query=query, segments=segments, workspace=regular.attention,
            positions=regular.selection.positions, **common,
        )
        # poison the outputs of the second workspace so that a no-op cannot pass
        static.attention.output.fill_(float("nan"))
        static.attention.topk_positions.fill_(-5)
        ops.segmented_attention_static(
            query=query, segments=segments, workspace=static.attention, **common
        )
        torch.cuda.synchronize()
        where = f"call {call}"
        # same kernels, same inputs: the tolerance of the other attention tests (2e-2) is
        # met with zero difference
        assert torch.equal(static.attention.output, regular.attention.output), where
        assert torch.equal(static.attention.lse, regular.attention.lse), where
        assert torch.equal(static.attention.topk_positions, regular.attention.topk_positions), where
        assert torch.equal(static.attention.topk_scores, regular.attention.topk_scores), where
        assert not torch.isnan(static.attention.output.float()).any()


def test_static_scratch_entry_point_updates_the_graph_like_the_regular_one():
    """With the online update enabled the merge reads its neighbour candidates from the
    built-in array: both entry points must leave identical graph state, three steps in a row."""

    from tests.helpers import assert_state_equal, cpu_clone

    device = torch.device("cuda", 0)
    budget, sinks = 512, 6
    layer = make_layer(seed=79, kv_heads=4, seq_len=4096, communities=80, max_decode_tokens=6).to(device)
    sink_positions = torch.arange(sinks, dtype=torch.int32, device=device)
    sides = []
    for _ in range(2):
        # conversion keeps some of the tensors it is given: each side gets its own copies
        converted = convert_prefill_tensors(
            **{k: (v.clone() if torch.is_tensor(v) else v) for k, v in layer.prepare_kwargs().items()}
        )
        workspace = DecodeLayerWorkspace.allocate(
            retrieval_head_count=4, graph_count=4, group_size=4,
            community_capacity=converted.mutable.community_capacity, token_budget=budget, num_sink=sinks,
            dtype=torch.bfloat16, device=device, splits=4,
        )
        sides.append((converted, workspace))
    for step in range(3):
        query = make_query(seed=950 + step, query_heads=16).to(device)
        for index, (converted, workspace) in enumerate(sides):
            state = converted.mutable
            segments = ops.score_and_select(
                query=query, centroids=state.centroids, community_sizes=state.community_sizes,
                community_counts=state.community_counts, workspace=workspace.selection, csr=converted.csr,
                state=state, sink_positions=sink_positions, current_position=converted.current_position,
            )
            call = ops.segmented_attention_static if index else ops.segmented_attention
            call(
                query=query, key=layer.key, value=layer.value, csr=converted.csr, deltas=state.deltas,
                segments=segments, sink_positions=sink_positions, current_position=converted.current_position,
                softmax_scale=128**-0.5, workspace=workspace.attention, update_state=state,
                update_workspace=workspace.update, update_lam=0.5,
            )
        torch.cuda.synchronize()
        (regular, regular_ws), (static, static_ws) = sides
        where = f"step {step}"
        assert torch.equal(static_ws.attention.output, regular_ws.attention.output), where
        assert torch.equal(static_ws.update.assigned_communities, regular_ws.update.assigned_communities), where
        assert torch.equal(static_ws.update.overflow, regular_ws.update.overflow), where
        assert int(regular_ws.update.overflow.max()) == 0
        _, want, current = cpu_clone(regular.csr, regular.mutable, regular.current_position)
        assert_state_equal(static.mutable, want, where)
        assert torch.equal(static.current_position.cpu(), current), where


def test_static_scratch_entry_point_rejects_oversized_requests():
    device = torch.device("cuda", 0)
    layer = make_layer(seed=78, kv_heads=2, seq_len=2048, communities=40, max_decode_tokens=2)
    converted = convert_prefill_tensors(**layer.to(device).prepare_kwargs())
    state = converted.mutable
    ws = DecodeLayerWorkspace.allocate(
        retrieval_head_count=2, graph_count=2, group_size=4,
        community_capacity=state.community_capacity, token_budget=256, num_sink=2,
        dtype=torch.bfloat16, device=device, splits=native.STATIC_MAX_SPLITS + 1,
    )
    sinks = torch.arange(2, dtype=torch.int32, device=device)
    query = make_query(seed=1, query_heads=8).to(device)
    segments = ops.score_and_select(
        query=query, centroids=state.centroids, community_sizes=state.community_sizes,
        community_counts=state.community_counts, workspace=ws.selection, csr=converted.csr,
        state=state, sink_positions=sinks, current_position=converted.current_position,
    )
    with pytest.raises(native.NativeError, match="maximum"):
        ops.segmented_attention_static(
            query=query, key=layer.key.to(device), value=layer.value.to(device), csr=converted.csr,
            deltas=state.deltas, segments=segments, sink_positions=sinks,
            current_position=converted.current_position, softmax_scale=128**-0.5,
            workspace=ws.attention, update_state=state, update_workspace=None, update_lam=0.5,
        )

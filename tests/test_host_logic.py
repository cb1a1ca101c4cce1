"""Host-side logic on CPU: configuration, state layout, assembly, conversion, and the C ABI surface."""

from __future__ import annotations

import ctypes
import re
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

import community_kv_b200 as ckv
from community_kv_b200 import native, ops
from community_kv_b200.assembly import aggregation_mappings, build_member_csr, compute_centroids
from community_kv_b200.batched import stack_sequences
from community_kv_b200.config import CommunityKVConfig, GraphAggregation, PartitionConfig
from community_kv_b200.runtime import (
    CommunityKVRuntime,
    DecodeRuntime,
    _effective_token_budget,
    convert_prefill_tensors,
)
from community_kv_b200.state import (
    CentroidSelectionWorkspace,
    DecodeDeltaChunks,
    DecodeLayerWorkspace,
    choose_splits,
)
from community_kv_b200.synthetic import make_layer

ROOT = Path(__file__).resolve().parents[1]


# ---- public surface (reference tests/community_kv/test_init.py:18-32) -----------------------
def test_root_exports_match_the_reference_names():
    for name in (
        "ATTENTION_IMPLEMENTATION", "CommunityKVAttention", "CommunityKVConfig", "CommunityKVRuntime",
        "GraphAggregation", "HuggingFaceAttention", "PartitionConfig",
    ):
        assert hasattr(ckv, name), name
    assert ckv.ATTENTION_IMPLEMENTATION == "community_kv"


# ---- configuration (reference community_kv/config.py:33-70) ----------------------------------
def test_config_validation():
    assert CommunityKVConfig().token_budget == 4096
    assert CommunityKVConfig(aggregation="query_group").aggregation is GraphAggregation.QUERY_GROUP
    for bad in (dict(token_budget=96), dict(token_budget=0), dict(num_sink=-1),
                dict(token_budget=64, num_sink=63), dict(lam=1.5), dict(leiden_resolution=0.0)):
        with pytest.raises(ValueError):
            CommunityKVConfig(**bad)
    with pytest.raises(ValueError):
        PartitionConfig(workers_per_device=0)
    assert GraphAggregation.PER_QUERY_HEAD.graph_count(query_heads=32, kv_heads=8) == 32
    assert GraphAggregation.QUERY_GROUP.graph_count(query_heads=32, kv_heads=8) == 8
    assert GraphAggregation.LAYER_WISE.retrieval_head_count(query_heads=32, kv_heads=8) == 8
    with pytest.raises(ValueError):
        GraphAggregation.QUERY_GROUP.graph_count(query_heads=30, kv_heads=8)


def test_effective_budget_known_answers(golden_dir):
    # reference tests/community_kv/test_runtime.py:48-66
    assert _effective_token_budget(configured_budget=4096, prefill_seq_len=3806, num_sink=10) == 3776
    assert _effective_token_budget(configured_budget=4096, prefill_seq_len=4095, num_sink=10) == 4096
    assert _effective_token_budget(configured_budget=2048, prefill_seq_len=8192, num_sink=10) == 2048
    data = np.load(golden_dir / "assembly.npz")
    for (budget, length, sink), want in zip(data["budget_cases"].tolist(), data["budget_results"].tolist()):
        assert _effective_token_budget(configured_budget=budget, prefill_seq_len=length, num_sink=sink) == want
    with pytest.raises(ValueError):
        _effective_token_budget(configured_budget=128, prefill_seq_len=10, num_sink=10)


# ---- workspaces (reference test_centroid_selection.py:131-152) --------------------------------
def test_selection_workspace_contract():
    ws = CentroidSelectionWorkspace.allocate(
        kv_heads=2, community_capacity=32, token_budget=128, num_sink=10,
        score_community_counts=(8, 12), score_headroom=2, device="cpu",
    )
    assert ws.scores.shape == (2, 32) and ws.scores.dtype == torch.float16
    assert ws.selected_budget == 117
    assert ws.score_cover.tolist() == [10, 14]
    assert ws.packed_segments().tile_descriptors.shape == (2, 2)
    assert ws.communities.shape == (2, 117) and int(ws.communities[0, 0]) == -1
    with pytest.raises(ValueError, match="multiple of 64"):
        CentroidSelectionWorkspace.allocate(
            kv_heads=1, community_capacity=8, token_budget=96, num_sink=1, device="cpu"
        )
    batched = DecodeLayerWorkspace.allocate(
        retrieval_head_count=2, graph_count=2, group_size=4, community_capacity=32, token_budget=128,
        num_sink=10, dtype=torch.bfloat16, device="cpu", batch=3,
    )
    assert batched.selection.scores.shape == (3, 2, 32)
    assert batched.attention.output.shape == (3, 8, 128)
    assert batched.attention.partials.shape[-1] == native.PARTIAL_STRIDE
    assert choose_splits(2048, 64) == 6 and choose_splits(64, 8, 9) == 4
    # few units: eight (one cluster launch) unless a split would exceed 512 tokens
    assert choose_splits(2048, 1) == 8 and choose_splits(8192, 8) == 32 and choose_splits(2048, 1, 32) == 32


def test_operators_validate_before_launch_and_refuse_cpu():
    ws = CentroidSelectionWorkspace.allocate(
        kv_heads=2, community_capacity=32, token_budget=128, num_sink=10, device="cpu"
    )
    sizes = torch.ones((2, 32), dtype=torch.int32)
    counts = torch.tensor([8, 12], dtype=torch.int32)
    with pytest.raises(ValueError, match="query heads"):   # reference test_centroid_selection.py:228-238
        ops.score_centroids(query=torch.empty((3, 64), dtype=torch.bfloat16),
                            centroids=torch.empty((2, 32, 128), dtype=torch.float8_e4m3fn),
                            community_sizes=sizes, community_counts=counts, workspace=ws)
    with pytest.raises(TypeError, match="FP8 E4M3"):        # reference :241-251
        ops.score_centroids(query=torch.empty((8, 128), dtype=torch.bfloat16),
                            centroids=torch.empty((2, 32, 128), dtype=torch.bfloat16),
                            community_sizes=sizes, community_counts=counts, workspace=ws)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.score_centroids(query=torch.zeros((8, 128), dtype=torch.bfloat16),
                            centroids=torch.zeros((2, 32, 128), dtype=torch.float8_e4m3fn),
                            community_sizes=sizes, community_counts=counts, workspace=ws)


# ---- state assembly against fixtures generated from the reference ------------------------------
def test_assembly_matches_reference_builders(golden_dir):
    data = np.load(golden_dir / "assembly.npz")
    kv_heads, query_heads, length, sink, headroom = data["meta"].tolist()
    keys = torch.from_numpy(data["keys"]).to(torch.bfloat16)
    for index, mode in enumerate(("per_query_head", "query_group", "layer_wise")):
        to_graph, to_kv = aggregation_mappings(mode, query_heads=query_heads, kv_heads=kv_heads)
        assert to_graph.tolist() == data[f"to_graph_{index}"].tolist()
        assert to_kv.tolist() == data[f"to_kv_{index}"].tolist()
        labels = torch.from_numpy(data[f"labels_{index}"])
        counts = (labels.amax(dim=1) + 1).to(torch.int32)
        centroids, sizes = compute_centroids(labels, counts, keys, retrieval_to_graph=to_graph,
                                             retrieval_to_kv=to_kv, num_sink=sink, max_decode_tokens=headroom)
        assert np.array_equal(centroids.view(torch.uint8).numpy(), data[f"centroids_{index}"])
        assert np.array_equal(sizes.numpy(), data[f"sizes_{index}"])
        offsets, positions = build_member_csr(labels, counts, num_sink=sink)
        assert np.array_equal(offsets.numpy(), data[f"offsets_{index}"])
        assert np.array_equal(positions.numpy(), data[f"positions_{index}"])
    # reference tests/community_kv/graph/test_partition.py:81-93
    offsets, positions = build_member_csr(torch.tensor([[0, 1, 1, 0, 1, 0]], dtype=torch.int32),
                                          torch.tensor([2], dtype=torch.int32), num_sink=1)
    assert offsets.tolist() == [[0, 2, 5]] and positions.tolist() == [[5, 3, 4, 2, 1]]


def test_delta_chunks_grow_geometrically():
    # reference tests/community_kv/graph/test_state.py:145-157
    chunks = DecodeDeltaChunks.allocate(graph_count=1, community_capacity=4, max_decode_tokens=8)
    for position in (10, 11, 12):
        chunks.append(0, 1, position)
    chunks.append(0, 2, 13)
    assert chunks.members(0, 1).tolist() == [10, 11, 12]
    assert chunks.members(0, 2).tolist() == [13]
    assert chunks.chunk_capacity[0, :3].tolist() == [1, 2, 1]
    assert int(chunks.next_free_position[0]) == 4
    chunks.validate()
    small = DecodeDeltaChunks.allocate(graph_count=1, community_capacity=2, max_decode_tokens=1)
    small.append(0, 0, 5)
    with pytest.raises(RuntimeError, match="exhausted"):
        small.append(0, 1, 6)


# ---- conversion and runtime bookkeeping (reference test_runtime.py:205-319) --------------------
def test_convert_prefill_tensors_pads_offsets_and_validates():
    layer = make_layer(seed=1, kv_heads=2, seq_len=512, communities=12, max_decode_tokens=6)
    kwargs = layer.prepare_kwargs()
    converted = convert_prefill_tensors(**kwargs)
    capacity = converted.mutable.community_capacity
    assert converted.csr.member_offsets.shape == (2, capacity + 1)
    assert torch.all(converted.csr.member_offsets[:, 13:] == converted.csr.member_offsets[:, 12:13])
    assert converted.current_position.tolist() == [512, 512]
    assert converted.initial_community_counts == (12, 12)
    assert converted.mutable.deltas.positions.shape == (2, 12)
    bad = dict(kwargs)
    bad["centroids"] = kwargs["centroids"].view(torch.uint8).float()
    with pytest.raises(TypeError, match="FP8"):
        convert_prefill_tensors(**bad)
    bad = dict(kwargs)
    bad["token_communities"] = kwargs["token_communities"][:, :514]
    with pytest.raises(ValueError, match="headroom"):
        convert_prefill_tensors(**bad)
    shared = make_layer(seed=2, kv_heads=2, seq_len=512, communities=12, max_decode_tokens=6,
                        aggregation="layer_wise")
    converted = convert_prefill_tensors(**shared.prepare_kwargs())
    assert converted.mutable.graph_count == 1 and converted.mutable.retrieval_head_count == 2
    assert converted.initial_community_counts == (12, 12)


def test_runtime_lifecycle_without_a_gpu():
    config = CommunityKVConfig(token_budget=128, num_sink=4)
    runtime = DecodeRuntime(config)
    layer = make_layer(seed=3, kv_heads=2, seq_len=512, communities=12, max_decode_tokens=6)
    state = runtime.prepare_layer(0, **layer.prepare_kwargs())
    assert state.workspace.selection.token_budget == 128
    with pytest.raises(ValueError, match="already prepared"):
        runtime.prepare_layer(0, **layer.prepare_kwargs())
    with pytest.raises(RuntimeError, match="not prepared"):
        runtime.decode(layer_idx=1, query=torch.zeros(1, 8, 1, 128), key=torch.zeros(1, 2, 8, 128),
                       value=torch.zeros(1, 2, 8, 128), softmax_scale=1.0)
    with pytest.raises(ValueError, match="query shape"):
        runtime.decode(layer_idx=0, query=torch.zeros(2, 8, 1, 128), key=torch.zeros(1, 2, 8, 128),
                       value=torch.zeros(1, 2, 8, 128), softmax_scale=1.0)
    runtime.assert_no_overflow()
    state.workspace.update.overflow[0] = 2
    with pytest.raises(RuntimeError, match="overflow"):
        runtime.assert_no_overflow()

    seen = []

    def partitioner(**kwargs):
        seen.append(kwargs["layer_idx"])
        raise KeyError("stop")

    with CommunityKVRuntime(config=config, partition=PartitionConfig(), num_layers=2,
                            max_decode_tokens=4, partitioner=partitioner) as full:
        full.start_request(resolutions=[1.0, 2.0])
        assert full.resolutions == {0: 1.0, 1: 2.0}
        with pytest.raises(ValueError, match="one value per layer"):
            full.start_request(resolutions=[1.0])
        with pytest.raises(KeyError):
            full.submit_prefill_layer(layer_idx=1, topk_indices=None, topk_scores=None, keys=None,
                                      completion_event=None)
        assert seen == [1]
        with pytest.raises(RuntimeError, match="incomplete"):
            full.finish_prefill()
    with pytest.raises(RuntimeError, match="no partitioner"):
        CommunityKVRuntime(config=config, partition=PartitionConfig(), num_layers=1,
                           max_decode_tokens=4).submit_prefill_layer(
            layer_idx=0, topk_indices=None, topk_scores=None, keys=None, completion_event=None)


def test_batched_stack_pads_and_views():
    config = CommunityKVConfig(token_budget=128, num_sink=4, aggregation="query_group")
    layers = [make_layer(seed=5 + b, kv_heads=2, seq_len=512, communities=10 + 3 * b, max_decode_tokens=4)
              for b in range(3)]
    converted = [convert_prefill_tensors(**layer.prepare_kwargs()) for layer in layers]
    state = stack_sequences(converted, config=config)
    assert state.mutable.centroids.shape[:2] == (3, 2)
    capacity = state.mutable.centroids.shape[2]
    assert capacity == 16 + 4
    for b in range(3):
        csr, mutable, current = state.sequence_view(b)
        have = converted[b].mutable.community_capacity
        assert torch.equal(mutable.centroids[:, :have].view(torch.uint8),
                           converted[b].mutable.centroids.view(torch.uint8))
        assert torch.equal(csr.member_offsets[:, : have + 1], converted[b].csr.member_offsets)
        assert torch.all(csr.member_offsets[:, have:] == csr.member_offsets[:, have : have + 1])
        assert int(current[0]) == 512
        mutable.community_counts[0] += 1          # a view: writes land in the stacked tensor
        assert int(state.mutable.community_counts[b, 0]) == converted[b].initial_community_counts[0] + 1


# ---- the C ABI surface ---------------------------------------------------------------------
def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "ckv_b200.h").read_text()
    declared = set(re.findall(r"^(?:int|int64_t|const char\*)\s+(ckv_\w+)\s*\(", header, flags=re.M))
    assert declared == set(native.ENTRY_POINTS)
    lib = native.library()
    for name in declared:
        assert getattr(lib, name) is not None
    assert lib.ckv_version() >= 100
    assert b"null" in lib.ckv_status_string(-1)
    assert lib.ckv_attention_smem_bytes(4) > 60_000


def test_ctypes_struct_matches_the_header(tmp_path):
    source = tmp_path / "layout.c"
    fields = [name for name, _ in native.LayerArgs._fields_]
    probes = "\n".join(f'  printf("%zu\\n", offsetof(ckv_layer_args, {name}));' for name in fields)
    source.write_text(
        '#include <stdio.h>\n#include <stddef.h>\n#include "ckv_b200.h"\nint main(void) {\n'
        '  printf("%zu\\n", sizeof(ckv_layer_args));\n' + probes + "\n  return 0;\n}\n"
    )
    binary = tmp_path / "layout"
    subprocess.run(["gcc", "-I", str(ROOT / "include"), str(source), "-o", str(binary)], check=True)
    numbers = [int(x) for x in subprocess.run([str(binary)], capture_output=True, text=True, check=True).stdout.split()]
    assert numbers[0] == ctypes.sizeof(native.LayerArgs)
    for name, offset in zip(fields, numbers[1:]):
        assert getattr(native.LayerArgs, name).offset == offset, name


def test_prefill_struct_matches_the_header(tmp_path):
    source = tmp_path / "layout.c"
    fields = [name for name, _ in native.PrefillArgs._fields_]
    probes = "\n".join(f'  printf("%zu\\n", offsetof(ckv_prefill_args, {name}));' for name in fields)
    source.write_text(
        '#include <stdio.h>\n#include <stddef.h>\n#include "ckv_b200.h"\nint main(void) {\n'
        '  printf("%zu\\n", sizeof(ckv_prefill_args));\n' + probes + "\n  return 0;\n}\n"
    )
    binary = tmp_path / "layout"
    subprocess.run(["gcc", "-I", str(ROOT / "include"), str(source), "-o", str(binary)], check=True)
    numbers = [int(x) for x in subprocess.run([str(binary)], capture_output=True, text=True, check=True).stdout.split()]
    assert numbers[0] == ctypes.sizeof(native.PrefillArgs)
    for name, offset in zip(fields, numbers[1:]):
        assert getattr(native.PrefillArgs, name).offset == offset, name
    lib = native.library()
    args = native.PrefillArgs()
    assert lib.ckv_prefill_topk(None, None) == -1
    assert lib.ckv_prefill_topk(ctypes.byref(args), None) == -2
    native.fill(args, batch=1, seq_len=64, query_heads=6, kv_heads=2)
    assert lib.ckv_prefill_topk(ctypes.byref(args), None) == -6   # group size 3 is not supported


def test_argument_errors_come_back_as_status_codes():
    """Host-side validation only: no kernel is launched for a rejected argument block."""

    lib = native.library()
    args = native.LayerArgs()
    for entry in ("ckv_score_centroids", "ckv_select_descriptors", "ckv_segmented_attention",
                  "ckv_decode_layer", "ckv_segmented_attention_static"):
        assert getattr(lib, entry)(ctypes.byref(args), None) < 0
        assert getattr(lib, entry)(None, None) == -1
    native.fill(args, batch=1, retrieval_heads=1, graphs=1, group_size=17, community_capacity=4,
                token_budget=128, num_sink=1)
    assert lib.ckv_score_centroids(ctypes.byref(args), None) == -2
    with pytest.raises(native.NativeError, match="status -2"):
        native.call("ckv_decode_layer", args, 0)


def test_static_entry_point_applies_the_shared_validation():
    """The allocation-free entry point rejects what the regular one rejects, before any CUDA call:
    a peer count beyond CKV_MAX_PEERS would otherwise index past the peer pointer arrays."""

    lib = native.library()
    keep = (ctypes.c_int32 * 4)()
    address = ctypes.addressof(keep)
    for entry in ("ckv_segmented_attention", "ckv_segmented_attention_static"):
        args = native.LayerArgs()
        native.fill(args, batch=1, retrieval_heads=1, graphs=1, group_size=4, community_capacity=4,
                    token_budget=128, num_sink=1, splits=1, retrieval_to_graph=address,
                    retrieval_to_kv=address, peer_count=native.MAX_PEERS + 1)
        assert getattr(lib, entry)(ctypes.byref(args), None) == -2, entry
        args.peer_count = 1  # in range, but the peer's pointers are missing
        assert getattr(lib, entry)(ctypes.byref(args), None) == -1, entry
    args = native.LayerArgs()
    native.fill(args, batch=65, retrieval_heads=1, graphs=1, group_size=4, community_capacity=4,
                token_budget=128, num_sink=1, splits=1)
    assert lib.ckv_segmented_attention_static(ctypes.byref(args), None) == -7

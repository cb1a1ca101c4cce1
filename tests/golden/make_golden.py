"""Generate the golden fixtures in this directory from the reference project.

Run from anywhere, in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/reference [group ...]

It imports the reference package (``community_kv``) and the semantic helpers
that live in the reference's own unit tests, feeds them seeded random inputs and
stores inputs and outputs as ``*.npz`` files.  The fixtures travel with the
repository; the reference does not.  ``tests/test_oracle_golden.py`` checks the
CPU oracle against them.
"""

from __future__ import annotations

import copy
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
if len(sys.argv) < 2:
    raise SystemExit("usage: make_golden.py <path to a checkout of the reference project>")
REFERENCE = Path(sys.argv[1])
sys.path.insert(0, str(REFERENCE))

from community_kv.graph.partition import (  # noqa: E402
    _reshape_by_aggregation,
    aggregation_mappings,
    build_adjacency,
    build_member_csr,
    compute_centroids,
)
from community_kv.graph.state import (  # noqa: E402
    DecodeDeltaChunks,
    MutableGraphState,
    PrefillCSR,
)
from community_kv.runtime import _effective_token_budget, convert_prefill_tensors  # noqa: E402
from tests.community_kv.attention.kernels.test_centroid_selection import (  # noqa: E402
    _ordered_fp16_keys,
    _weighted_prefix_select,
)
from tests.community_kv.attention.kernels.test_packed_segments import (  # noqa: E402
    _pack_segments,
    _selection,
)
from tests.community_kv.graph.test_state import (  # noqa: E402
    _materialize_positions,
    _online_assign_and_update,
)


def selection_cases(rng: np.random.Generator) -> dict[str, np.ndarray]:
    out: dict[str, np.ndarray] = {}
    cases = []
    for case in range(48):
        capacity = int(rng.integers(4, 400))
        active = int(rng.integers(1, capacity + 1))
        coarse = case % 3 == 0
        scores = rng.normal(size=capacity).astype(np.float32)
        if coarse:  # many fp16 ties
            scores = np.round(scores * 4) / 4
        scores16 = scores.astype(np.float16)
        sizes = rng.integers(0, 40, size=capacity).astype(np.int32)
        sizes[rng.random(capacity) < 0.15] = 0
        total = int(sizes[:active].sum())
        if total < 2:
            sizes[0] = 5
            total = int(sizes[:active].sum())
        budget = int(rng.integers(1, total + 1))
        picked = _weighted_prefix_select(
            torch.from_numpy(scores16.astype(np.float32)),
            torch.from_numpy(sizes),
            budget,
            active_communities=active,
        )
        ids = np.array([d.community_id for d in picked.descriptors], dtype=np.int32)
        takes = np.array([d.take_count for d in picked.descriptors], dtype=np.int32)
        out[f"scores_{case}"] = scores16.view(np.uint16)
        out[f"sizes_{case}"] = sizes
        out[f"meta_{case}"] = np.array([active, budget, picked.token_count], dtype=np.int64)
        out[f"ids_{case}"] = ids
        out[f"takes_{case}"] = takes
        cases.append(case)
    probe = np.array([-np.inf, -65504.0, -2.0, -1e-7, -0.0, 0.0, 1e-7, 1.0, 65504.0, np.inf], dtype=np.float32)
    out["key_probe"] = probe
    out["key_probe_keys"] = _ordered_fp16_keys(torch.from_numpy(probe)).numpy().astype(np.int32)
    out["cases"] = np.array(cases)
    return out


def packing_cases(rng: np.random.Generator) -> dict[str, np.ndarray]:
    out: dict[str, np.ndarray] = {}
    count = 0
    for budget, sink in ((128, 10), (128, 0), (256, 3), (512, 10), (64, 1), (1024, 62)):
        selected = budget - sink - 1
        heads = []
        for _ in range(3):
            takes = []
            left = selected
            while left > 0:
                take = int(min(left, rng.integers(1, 90)))
                takes.append(take)
                left -= take
            communities = rng.permutation(10_000)[: len(takes)]
            heads.append(_selection(*zip(communities.tolist(), takes)))
        heads.append(_selection(*((c, 1) for c in range(selected))))
        packed = _pack_segments(tuple(heads), token_budget=budget, num_sink=sink)
        out[f"meta_{count}"] = np.array([budget, sink], dtype=np.int64)
        out[f"communities_{count}"] = packed.communities.numpy()
        out[f"ends_{count}"] = packed.cumulative_ends.numpy()
        out[f"counts_{count}"] = packed.descriptor_counts.numpy()
        out[f"tiles_{count}"] = packed.tile_descriptors.numpy()
        count += 1
    out["cases"] = np.arange(count)
    return out


def _random_partition(rng: np.random.Generator, graphs: int, length: int, communities: int, sink: int):
    labels = rng.integers(0, communities, size=(graphs, length)).astype(np.int32)
    labels[:, :communities] = np.arange(communities, dtype=np.int32)  # every id occurs
    return torch.from_numpy(labels)


def position_cases(rng: np.random.Generator) -> dict[str, np.ndarray]:
    out: dict[str, np.ndarray] = {}
    graphs, length, communities, sink = 2, 300, 12, 4
    labels = _random_partition(rng, graphs, length, communities, sink)
    counts = torch.full((graphs,), communities, dtype=torch.int32)
    offsets, positions = build_member_csr(labels, counts, num_sink=sink)
    csr = PrefillCSR(member_offsets=offsets, member_positions=positions, community_counts=counts)
    csr.validate()
    deltas = DecodeDeltaChunks.allocate(
        graph_count=graphs, community_capacity=communities + 40, max_decode_tokens=40
    )
    appended = []
    for step in range(40):
        for graph in range(graphs):
            community = int(rng.integers(0, communities))
            deltas.append(graph, community, length + step)
            appended.append((graph, community, length + step))
    out["labels"] = labels.numpy()
    out["offsets"] = offsets.numpy()
    out["member_positions"] = positions.numpy()
    out["appended"] = np.array(appended, dtype=np.int32)
    for name in (
        "positions", "chunk_start", "chunk_capacity", "chunk_size", "chunk_next",
        "chunk_previous", "community_head", "community_tail", "community_sizes",
        "next_free_chunk", "next_free_position",
    ):
        out[f"delta_{name}"] = getattr(deltas, name).numpy()
    queries = 0
    for graph in range(graphs):
        for _ in range(6):
            picked = rng.permutation(communities)[: int(rng.integers(1, 6))]
            descriptors = []
            for community in picked.tolist():
                size = int(offsets[graph, community + 1] - offsets[graph, community]) + int(
                    deltas.community_sizes[graph, community]
                )
                descriptors.append((community, int(rng.integers(1, size + 1))))
            result = _materialize_positions(
                csr=csr, deltas=deltas, graph=graph, descriptors=tuple(descriptors)
            )
            out[f"query_{queries}"] = np.array([[graph, 0]] + descriptors, dtype=np.int32)
            out[f"result_{queries}"] = result.numpy().astype(np.int32)
            queries += 1
    out["queries"] = np.arange(queries)
    out["meta"] = np.array([graphs, length, communities, sink], dtype=np.int64)
    return out


def assembly_cases(rng: np.random.Generator) -> dict[str, np.ndarray]:
    out: dict[str, np.ndarray] = {}
    kv_heads, query_heads, length, sink, headroom = 2, 4, 160, 3, 5
    keys = torch.from_numpy(rng.normal(size=(kv_heads, length, 128)).astype(np.float32)).to(
        torch.bfloat16
    )
    out["keys"] = keys.float().numpy()
    for index, mode in enumerate(("per_query_head", "query_group", "layer_wise")):
        to_graph, to_kv = aggregation_mappings(
            __import__("community_kv").GraphAggregation(mode),
            query_heads=query_heads,
            kv_heads=kv_heads,
            device="cpu",
        )
        graphs = int(to_graph.max()) + 1
        labels = _random_partition(rng, graphs, length, 9 + index, sink)
        counts = (labels.amax(dim=1) + 1).to(torch.int32)
        centroids, sizes = compute_centroids(
            labels, counts, keys, retrieval_to_graph=to_graph, retrieval_to_kv=to_kv,
            num_sink=sink, max_decode_tokens=headroom,
        )
        offsets, positions = build_member_csr(labels, counts, num_sink=sink)
        out[f"labels_{index}"] = labels.numpy()
        out[f"to_graph_{index}"] = to_graph.numpy()
        out[f"to_kv_{index}"] = to_kv.numpy()
        out[f"centroids_{index}"] = centroids.view(torch.uint8).numpy()
        out[f"sizes_{index}"] = sizes.numpy()
        out[f"offsets_{index}"] = offsets.numpy()
        out[f"positions_{index}"] = positions.numpy()
    out["meta"] = np.array([kv_heads, query_heads, length, sink, headroom], dtype=np.int64)
    budgets = [(4096, 3806, 10), (4096, 4095, 10), (2048, 8192, 10), (1024, 100, 2), (128, 127, 0)]
    out["budget_cases"] = np.array(budgets, dtype=np.int64)
    out["budget_results"] = np.array(
        [
            _effective_token_budget(configured_budget=b, prefill_seq_len=s, num_sink=n)
            for b, s, n in budgets
        ],
        dtype=np.int64,
    )
    return out


def online_update_cases(rng: np.random.Generator) -> dict[str, np.ndarray]:
    """Several consecutive online assignments on one graph, recorded step by step."""

    out: dict[str, np.ndarray] = {}
    capacity, length, steps, dim = 40, 400, 24, 128
    communities = 10
    labels = _random_partition(rng, 1, length, communities, 0)
    token_communities = torch.full((1, length + steps), -1, dtype=torch.int32)
    token_communities[:, :length] = labels
    sizes = torch.zeros((1, capacity), dtype=torch.int32)
    sizes[0, :communities] = torch.bincount(labels[0].long(), minlength=communities).to(torch.int32)
    centroids = torch.from_numpy(rng.normal(size=(1, capacity, dim)).astype(np.float32)).to(
        torch.float8_e4m3fn
    )
    weight = torch.zeros((1, capacity), dtype=torch.float32)
    weight[0, :communities] = torch.from_numpy(rng.uniform(0.05, 3.0, size=communities).astype(np.float32))
    state = MutableGraphState(
        centroids=centroids,
        community_sizes=sizes,
        community_counts=torch.tensor([communities], dtype=torch.int32),
        community_weight=weight,
        total_weight=torch.tensor([float(weight.sum()) * 0.5], dtype=torch.float32),
        token_communities=token_communities,
        deltas=DecodeDeltaChunks.allocate(
            graph_count=1, community_capacity=capacity, max_decode_tokens=steps
        ),
        retrieval_to_graph=torch.zeros(1, dtype=torch.int32),
        retrieval_to_kv=torch.zeros(1, dtype=torch.int32),
    )
    state.validate()
    out["initial_centroids"] = state.centroids.view(torch.uint8).numpy().copy()
    out["initial_sizes"] = state.community_sizes.numpy().copy()
    out["initial_weight"] = state.community_weight.numpy().copy()
    out["initial_total"] = state.total_weight.numpy().copy()
    out["initial_labels"] = state.token_communities.numpy().copy()
    out["meta"] = np.array([capacity, length, steps, dim, communities], dtype=np.int64)
    for step in range(steps):
        known = length + step
        scores = np.sort(rng.normal(size=8).astype(np.float32))[::-1].copy()
        positions = rng.permutation(known)[:8].astype(np.int32)
        if step % 5 == 4:
            positions[6:] = -1
        lse = np.float32(scores.max() + rng.uniform(0.1, 2.0))
        lam = float(rng.choice([0.0, 0.25, 0.5, 1.0]))
        key = torch.from_numpy(rng.normal(size=(1, dim)).astype(np.float32)).to(torch.bfloat16)
        if step % 7 == 3:  # force a fresh singleton community
            state.community_weight[0, : int(state.community_counts[0])] += 1000.0
        weight_before = state.community_weight.numpy().copy()
        result = _online_assign_and_update(
            state=state,
            topk_scores=torch.from_numpy(scores).unsqueeze(0),
            topk_positions=torch.from_numpy(positions).unsqueeze(0),
            representative_lse=torch.tensor([lse]),
            current_key=key,
            current_position=known,
            lam=lam,
        )
        out[f"scores_{step}"] = scores
        out[f"positions_{step}"] = positions
        out[f"scalars_{step}"] = np.array([lse, lam], dtype=np.float32)
        out[f"key_{step}"] = key.float().numpy()
        out[f"weight_before_{step}"] = weight_before
        out[f"assigned_{step}"] = result.assigned_communities.numpy().copy()
        out[f"counts_{step}"] = state.community_counts.numpy().copy()
        out[f"sizes_{step}"] = state.community_sizes.numpy().copy()
        out[f"centroids_{step}"] = state.centroids.view(torch.uint8).numpy().copy()
        out[f"weight_{step}"] = state.community_weight.numpy().copy()
        out[f"total_{step}"] = state.total_weight.numpy().copy()
        out[f"labels_{step}"] = state.token_communities.numpy().copy()
    for name in (
        "positions", "chunk_start", "chunk_capacity", "chunk_size", "chunk_next",
        "chunk_previous", "community_head", "community_tail", "community_sizes",
        "next_free_chunk", "next_free_position",
    ):
        out[f"final_delta_{name}"] = getattr(state.deltas, name).numpy().copy()
    return out


def adjacency_cases(rng: np.random.Generator) -> dict[str, np.ndarray]:
    """Prefill edges -> coalesced adjacency (build_adjacency) and the per-graph reshaping of the edges."""

    out: dict[str, np.ndarray] = {}
    shapes = [(1, 2, 2, 4, 1.0), (1, 2, 2, 4, 0.5), (3, 40, 8, 64, 0.5), (2, 75, 8, 90, 0.0),
              (4, 60, 5, 33, 0.25), (8, 128, 8, 200, 0.7), (2, 300, 8, 310, 1.0)]
    for case, (graphs, rows, kappa, length, lam) in enumerate(shapes):
        indices = rng.integers(-2, length + 3, size=(graphs, rows, kappa)).astype(np.int32)
        if case % 2:
            indices[:, :, 1] = indices[:, :, 0]  # duplicated neighbours inside a row
        scores = rng.uniform(0.0, 1.0, size=(graphs, rows, kappa)).astype(np.float32)
        positions = rng.integers(0, length, size=(graphs, rows)).astype(np.int64)
        source, destination, weight = build_adjacency(
            torch.from_numpy(indices), torch.from_numpy(scores), torch.from_numpy(positions),
            seq_len=length, lam=lam,
        )
        out[f"indices_{case}"] = indices
        out[f"scores_{case}"] = scores
        out[f"positions_{case}"] = positions
        out[f"scalars_{case}"] = np.array([length, lam], dtype=np.float64)
        out[f"source_{case}"] = source.numpy()
        out[f"destination_{case}"] = destination.numpy()
        out[f"weight_{case}"] = weight.numpy()
    out["cases"] = np.arange(len(shapes))
    heads, kv_heads, rows, kappa, sink = 8, 2, 21, 8, 3
    indices = torch.from_numpy(rng.integers(0, 40, size=(heads, rows, kappa)).astype(np.int32))
    scores = torch.from_numpy(rng.uniform(size=(heads, rows, kappa)).astype(np.float32))
    for index, mode in enumerate(("per_query_head", "query_group", "layer_wise")):
        shaped = _reshape_by_aggregation(
            indices, scores, aggregation=__import__("community_kv").GraphAggregation(mode),
            num_kv_heads=kv_heads, num_sink=sink,
        )
        out[f"reshape_indices_{index}"] = shaped[0].numpy()
        out[f"reshape_scores_{index}"] = shaped[1].numpy()
        out[f"reshape_positions_{index}"] = shaped[2].numpy()
    out["reshape_inputs_indices"] = indices.numpy()
    out["reshape_inputs_scores"] = scores.numpy()
    out["reshape_meta"] = np.array([heads, kv_heads, rows, kappa, sink], dtype=np.int64)
    return out


def main() -> None:
    groups = {
        "selection": selection_cases,
        "packing": packing_cases,
        "positions": position_cases,
        "assembly": assembly_cases,
        "online_update": online_update_cases,
        "adjacency": adjacency_cases,
    }
    wanted = set(sys.argv[2:])
    for seed, (name, builder) in enumerate(groups.items()):
        if wanted and name not in wanted:
            continue
        arrays = builder(np.random.default_rng(1000 + seed))
        np.savez_compressed(HERE / f"{name}.npz", **arrays)
        print(name, len(arrays), "arrays")


if __name__ == "__main__":
    main()

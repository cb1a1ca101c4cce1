"""Decode-state assembly kernels (``ckv_assemble_*``) against the host restatement of the reference's
builders (community_kv/graph/partition.py:382-535), which ``tests/test_host_logic.py`` pins on fixtures
generated from the reference itself."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from community_kv_b200.assembly import (
    aggregation_mappings,
    assemble_layer,
    build_member_csr,
    compute_centroids,
    init_modularity_state,
)
from community_kv_b200.synthetic import zipf_sizes

pytestmark = pytest.mark.gpu


def _labels(graphs, length, communities, seed, zipf=None):
    generator = torch.Generator().manual_seed(seed)
    rows = []
    for _ in range(graphs):
        if zipf is None:
            ids = torch.randint(0, communities, (length,), generator=generator)
            ids[:communities] = torch.randperm(communities, generator=generator)
        else:
            sizes = zipf_sizes(length, communities, zipf, generator)
            ids = torch.repeat_interleave(torch.arange(communities), sizes)[torch.randperm(length, generator=generator)]
        rows.append(ids)
    return torch.stack(rows).to(torch.int32)


@pytest.mark.parametrize(
    "graphs,kv_heads,query_heads,aggregation,length,communities,zipf",
    [
        (2, 2, 8, "query_group", 3000, 37, None),
        (8, 2, 8, "per_query_head", 1000, 11, None),
        (1, 4, 16, "layer_wise", 5000, 130, 1.1),
        (8, 8, 32, "query_group", 32768, 512, 1.1),      # one layer of the whole-model configuration
        (2, 2, 8, "query_group", 131072, 4096, 1.1),     # long-context sizes
    ],
)
def test_member_lists_and_centroids_match_the_host_builders(graphs, kv_heads, query_heads, aggregation, length,
                                                            communities, zipf):
    device = torch.device("cuda", 0)
    sinks, decode = 10, 7
    labels = _labels(graphs, length, communities, seed=length + graphs, zipf=zipf)
    generator = torch.Generator().manual_seed(5)
    keys = (torch.randn((kv_heads, length, 128), generator=generator) / 128**0.5).to(torch.bfloat16)
    counts = (labels.amax(dim=1) + 1).to(torch.int32)
    to_graph, to_kv = aggregation_mappings(aggregation, query_heads=query_heads, kv_heads=kv_heads)

    want_offsets, want_positions = build_member_csr(labels, counts, num_sink=sinks)
    want_centroids, want_sizes = compute_centroids(labels, counts, keys, retrieval_to_graph=to_graph,
                                                   retrieval_to_kv=to_kv, num_sink=sinks, max_decode_tokens=decode)
    got_offsets, got_positions = build_member_csr(labels.to(device), counts.to(device), num_sink=sinks)
    got_centroids, got_sizes = compute_centroids(labels.to(device), counts.to(device), keys.to(device),
                                                 retrieval_to_graph=to_graph.to(device),
                                                 retrieval_to_kv=to_kv.to(device), num_sink=sinks,
                                                 max_decode_tokens=decode)
    assert torch.equal(got_offsets.cpu(), want_offsets)
    assert torch.equal(got_positions.cpu(), want_positions)
    assert torch.equal(got_sizes.cpu(), want_sizes)
    assert got_centroids.shape == want_centroids.shape
    assert torch.equal(got_centroids.cpu().view(torch.uint8), want_centroids.view(torch.uint8))


def test_assembly_fixture_from_the_reference(golden_dir):
    """The reference-generated fixture (labels -> offsets, member positions, sizes, e4m3 centroids)."""

    device = torch.device("cuda", 0)
    data = np.load(golden_dir / "assembly.npz")
    sinks, decode = int(data["meta"][3]), int(data["meta"][4])
    keys = torch.from_numpy(data["keys"])
    keys_are_bf16 = torch.equal(keys, keys.to(torch.bfloat16).float())  # the kernel takes bf16 keys
    for case in range(3):
        labels = torch.from_numpy(data[f"labels_{case}"])
        to_graph = torch.from_numpy(data[f"to_graph_{case}"])
        to_kv = torch.from_numpy(data[f"to_kv_{case}"])
        counts = (labels.amax(dim=1) + 1).to(torch.int32)
        offsets, positions = build_member_csr(labels.to(device), counts.to(device), num_sink=sinks)
        centroids, sizes = compute_centroids(labels.to(device), counts.to(device), keys.to(torch.bfloat16).to(device),
                                             retrieval_to_graph=to_graph.to(device), retrieval_to_kv=to_kv.to(device),
                                             num_sink=sinks, max_decode_tokens=decode)
        assert torch.equal(offsets.cpu(), torch.from_numpy(data[f"offsets_{case}"])), case
        assert torch.equal(positions.cpu(), torch.from_numpy(data[f"positions_{case}"])), case
        assert torch.equal(sizes.cpu(), torch.from_numpy(data[f"sizes_{case}"])), case
        if keys_are_bf16:
            assert torch.equal(centroids.cpu().view(torch.uint8), torch.from_numpy(data[f"centroids_{case}"])), case


def test_modularity_state_from_an_edge_list():
    device = torch.device("cuda", 0)
    graphs, length, communities = 3, 4000, 50
    labels = _labels(graphs, length, communities, seed=9)
    generator = torch.Generator().manual_seed(10)
    edges = 60000
    graph = torch.randint(0, graphs, (edges,), generator=generator)
    source = graph * length + torch.randint(0, length, (edges,), generator=generator)
    destination = graph * length + torch.randint(0, length, (edges,), generator=generator)
    weight = torch.rand((edges,), generator=generator)
    want_weight, want_total = init_modularity_state(labels, source, destination, weight, community_capacity=64)
    got_weight, got_total = init_modularity_state(labels.to(device), source.to(device), destination.to(device),
                                                  weight.to(device), community_capacity=64)
    torch.testing.assert_close(got_weight.cpu(), want_weight, rtol=2e-5, atol=1e-6)
    torch.testing.assert_close(got_total.cpu(), want_total, rtol=2e-5, atol=1e-6)
    empty = torch.empty((0,), dtype=torch.int64, device=device)
    zero_weight, zero_total = init_modularity_state(labels.to(device), empty, empty, empty.float(),
                                                    community_capacity=64)
    assert float(zero_weight.abs().sum()) == 0.0 and float(zero_total.abs().sum()) == 0.0


def test_assembled_layer_on_the_device_equals_the_host_one():
    device = torch.device("cuda", 0)
    labels = _labels(2, 6000, 90, seed=3, zipf=1.1)
    keys = (torch.randn((2, 6000, 128), generator=torch.Generator().manual_seed(4)) / 128**0.5).to(torch.bfloat16)
    host = assemble_layer(labels, keys, aggregation="query_group", query_heads=8, num_sink=10, max_decode_tokens=5)
    dev = assemble_layer(labels.to(device), keys.to(device), aggregation="query_group", query_heads=8, num_sink=10,
                         max_decode_tokens=5)
    for name in host.__slots__:
        a, b = getattr(host, name), getattr(dev, name).cpu()
        if a.dtype == torch.float8_e4m3fn:
            assert torch.equal(a.view(torch.uint8), b.view(torch.uint8)), name
        elif a.dtype == torch.float32:
            torch.testing.assert_close(b, a, rtol=1e-6, atol=0, msg=name)
        else:
            assert torch.equal(a, b), name


# ---- edge list -> adjacency -----------------------------------------------------------------------
def _adjacency_equal(got, want, where):
    source, destination, weight = (t.cpu().numpy() for t in got)
    assert np.array_equal(source, want[0]), where
    assert np.array_equal(destination, want[1]), where
    assert np.array_equal(weight.view(np.int32), want[2].view(np.int32)), where  # fp32 sums bit for bit


def test_adjacency_fixture_from_the_reference(golden_dir):
    from community_kv_b200.assembly import build_adjacency

    device = torch.device("cuda", 0)
    data = np.load(golden_dir / "adjacency.npz")
    for case in data["cases"].tolist():
        length, lam = int(data[f"scalars_{case}"][0]), float(data[f"scalars_{case}"][1])
        got = build_adjacency(torch.from_numpy(data[f"indices_{case}"]).to(device),
                              torch.from_numpy(data[f"scores_{case}"]).to(device),
                              torch.from_numpy(data[f"positions_{case}"]).to(device), seq_len=length, lam=lam)
        _adjacency_equal(got, (data[f"source_{case}"], data[f"destination_{case}"], data[f"weight_{case}"]),
                         f"case {case}")


@pytest.mark.parametrize("graphs,rows,length,lam", [(8, 4 * 4000, 4096, 0.5), (2, 30000, 32768, 0.5),
                                                    (1, 50000, 131072, 1.0)])
def test_adjacency_against_the_cpu_restatement(graphs, rows, length, lam):
    """Sizes of a real prefill (causal neighbours, hub keys, several heads sharing a graph): every
    distinct edge, in order, with its weight summed in the reference's order."""

    from community_kv_b200.assembly import build_adjacency
    from oracle.adjacency_oracle import build_adjacency as oracle_adjacency

    device = torch.device("cuda", 0)
    rng = np.random.default_rng(rows)
    positions = rng.integers(20, length, size=(graphs, rows)).astype(np.int64)
    # neighbours are earlier positions, a few of them shared hubs; some slots are empty
    indices = (positions[..., None] * rng.uniform(0, 1, size=(graphs, rows, 8))).astype(np.int32)
    hubs = rng.integers(0, 64, size=(graphs, rows, 8)).astype(np.int32)
    indices = np.where(rng.uniform(size=indices.shape) < 0.2, hubs, indices)
    indices = np.where(rng.uniform(size=indices.shape) < 0.05, -1, indices).astype(np.int32)
    scores = rng.uniform(0, 1, size=indices.shape).astype(np.float32)
    want = oracle_adjacency(indices, scores, positions, seq_len=length, lam=lam)
    got = build_adjacency(torch.from_numpy(indices).to(device), torch.from_numpy(scores).to(device),
                          torch.from_numpy(positions).to(device), seq_len=length, lam=lam)
    _adjacency_equal(got, want, f"{graphs}x{rows}")

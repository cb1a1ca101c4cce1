"""Seeded synthetic decode workloads with the shapes of the benchmark configurations.

No dataset is involved: keys are planted Gaussian clusters (or plain Gaussian
rows with Zipf-sized random communities), labels are the cluster ids, and the
decode state is assembled from them exactly like a partitioned prefill would be
(``community_kv_b200.assembly``).  Used by the tests, the smoke check and the
benchmark to build inputs; it is not on the decode path.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from community_kv_b200.assembly import (
    AssembledLayer,
    aggregation_mappings,
    assemble_layer,
    build_adjacency,
    init_modularity_state,
    reshape_by_aggregation,
)
from community_kv_b200.config import GraphAggregation

HEAD_DIM = 128


@dataclass(slots=True)
class SyntheticLayer:
    """One layer of one sequence: cache, labels, assembled decode state."""

    key: torch.Tensor  # [Hkv, S_cap, 128] bf16
    value: torch.Tensor
    labels: torch.Tensor  # [graphs, S] int32
    assembled: AssembledLayer
    prefill_seq_len: int
    max_decode_tokens: int
    group_size: int
    query_heads: int
    kv_heads: int
    aggregation: GraphAggregation

    def prepare_kwargs(self) -> dict:
        """Keyword arguments for ``DecodeRuntime.prepare_layer`` / ``convert_prefill_tensors``."""

        a = self.assembled
        return dict(
            member_offsets=a.member_offsets,
            member_positions=a.member_positions,
            num_communities=a.num_communities,
            centroids=a.centroids,
            community_sizes=a.community_sizes,
            community_weight=a.community_weight,
            total_weight=a.total_weight,
            token_communities=a.token_communities,
            retrieval_to_graph=a.retrieval_to_graph,
            retrieval_to_kv=a.retrieval_to_kv,
            prefill_seq_len=self.prefill_seq_len,
            max_decode_tokens=self.max_decode_tokens,
            group_size=self.group_size,
            aggregation=self.aggregation,
            query_heads=self.query_heads,
            kv_heads=self.kv_heads,
        )

    def to(self, device: torch.device | str) -> "SyntheticLayer":
        a = self.assembled
        moved = AssembledLayer(**{name: getattr(a, name).to(device) for name in a.__slots__})
        return SyntheticLayer(
            key=self.key.to(device),
            value=self.value.to(device),
            labels=self.labels.to(device),
            assembled=moved,
            prefill_seq_len=self.prefill_seq_len,
            max_decode_tokens=self.max_decode_tokens,
            group_size=self.group_size,
            query_heads=self.query_heads,
            kv_heads=self.kv_heads,
            aggregation=self.aggregation,
        )


def zipf_sizes(total: int, communities: int, exponent: float, generator: torch.Generator) -> torch.Tensor:
    """Positive integer sizes summing to ``total``, proportional to rank**-exponent."""

    rank = torch.arange(1, communities + 1, dtype=torch.float64)
    share = rank.pow(-exponent)
    share = share / share.sum()
    sizes = torch.floor(share * (total - communities)).long() + 1
    shortfall = total - int(sizes.sum())
    if shortfall > 0:
        extra = torch.multinomial(share, shortfall, replacement=True, generator=generator)
        sizes += torch.bincount(extra, minlength=communities)
    return sizes[torch.randperm(communities, generator=generator)]


def make_layer(
    *,
    seed: int,
    kv_heads: int = 8,
    group_size: int = 4,
    seq_len: int = 8192,
    communities: int = 64,
    sigma: float = 0.3,
    num_sink: int = 10,
    max_decode_tokens: int = 16,
    aggregation: GraphAggregation | str = GraphAggregation.QUERY_GROUP,
    zipf_exponent: float | None = None,
    integer_valued: bool = False,
) -> SyntheticLayer:
    """Planted-cluster layer on the CPU.

    ``zipf_exponent=None``: keys are ``centre + sigma * noise`` with multinomial
    cluster sizes, labels are the cluster ids.  With an exponent: keys are plain
    Gaussian rows and labels are random with Zipf-distributed community sizes.
    ``integer_valued`` draws small integers for every operand so that all fp32
    sums are exact whatever their order.
    """

    aggregation = GraphAggregation(aggregation)
    generator = torch.Generator().manual_seed(seed)
    query_heads = kv_heads * group_size
    rows = seq_len + max_decode_tokens + 1
    to_graph, _ = aggregation_mappings(aggregation, query_heads=query_heads, kv_heads=kv_heads)
    graphs = int(to_graph.max()) + 1
    heads_per_graph = {GraphAggregation.PER_QUERY_HEAD: group_size}.get(aggregation, 1)

    kv_labels = torch.empty((kv_heads, seq_len), dtype=torch.int64)
    if zipf_exponent is None:
        centres = torch.randn((kv_heads, communities, HEAD_DIM), generator=generator)
        for head in range(kv_heads):
            kv_labels[head] = torch.multinomial(
                torch.ones(communities), seq_len, replacement=True, generator=generator
            )
            kv_labels[head, :communities] = torch.randperm(communities, generator=generator)
        noise = torch.randn((kv_heads, rows, HEAD_DIM), generator=generator) * sigma
        padded = torch.cat(
            (kv_labels, torch.randint(0, communities, (kv_heads, rows - seq_len), generator=generator)),
            dim=1,
        )
        key = torch.gather(centres, 1, padded.unsqueeze(-1).expand(-1, -1, HEAD_DIM)) + noise
    else:
        for head in range(kv_heads):
            sizes = zipf_sizes(seq_len, communities, zipf_exponent, generator)
            ids = torch.repeat_interleave(torch.arange(communities), sizes)
            kv_labels[head] = ids[torch.randperm(seq_len, generator=generator)]
        key = torch.randn((kv_heads, rows, HEAD_DIM), generator=generator)
    value = torch.randn((kv_heads, rows, HEAD_DIM), generator=generator)
    if integer_valued:
        key = torch.randint(-3, 4, key.shape, generator=generator).float()
        value = torch.randint(-3, 4, value.shape, generator=generator).float()
    else:
        key = key / HEAD_DIM**0.5
        value = value / HEAD_DIM**0.5
    key = key.to(torch.bfloat16)
    value = value.to(torch.bfloat16)

    if aggregation is GraphAggregation.LAYER_WISE:
        labels = kv_labels[:1]
    elif aggregation is GraphAggregation.QUERY_GROUP:
        labels = kv_labels
    else:
        labels = kv_labels.repeat_interleave(heads_per_graph, dim=0)
    labels = labels.to(torch.int32).contiguous()
    assert labels.shape[0] == graphs
    assembled = assemble_layer(
        labels,
        key[:, :seq_len],
        aggregation=aggregation,
        query_heads=query_heads,
        num_sink=num_sink,
        max_decode_tokens=max_decode_tokens,
    )
    return SyntheticLayer(
        key=key,
        value=value,
        labels=labels,
        assembled=assembled,
        prefill_seq_len=seq_len,
        max_decode_tokens=max_decode_tokens,
        group_size=query_heads // assembled.retrieval_to_graph.numel(),
        query_heads=query_heads,
        kv_heads=kv_heads,
        aggregation=aggregation,
    )


@dataclass(slots=True)
class SyntheticPartitionedLayer:
    """What ``DecodeRuntime.prepare_partitioned_layer`` reads (the reference's ``PartitionedLayer``
    fields, community_kv/graph/partition.py:30-68)."""

    layer_idx: int
    member_offsets: torch.Tensor
    member_positions: torch.Tensor
    community_counts: torch.Tensor
    centroids: torch.Tensor
    community_sizes: torch.Tensor
    community_weight: torch.Tensor
    total_weight: torch.Tensor
    token_communities: torch.Tensor
    retrieval_to_graph: torch.Tensor
    retrieval_to_kv: torch.Tensor
    prefill_seq_len: int
    query_heads: int
    kv_heads: int
    aggregation: GraphAggregation


class SyntheticPartitioner:
    """Stand-in for the host-side Leiden partitioner: random labels with Zipf-sized communities.

    Callable with the keyword arguments ``CommunityKVRuntime.submit_prefill_layer`` passes
    to its ``partitioner``.  Everything around the partition itself is the real pipeline: on
    CUDA tensors the prefill edges are regrouped per graph and coalesced into the adjacency a
    partitioner would be handed (``assembly.build_adjacency``), the modularity weights of the
    labels are taken from that adjacency (``assembly.init_modularity_state``), and the decode
    state is assembled by the assembly kernels.  Only the labels are synthetic: drawn per
    (layer, graph) from a seeded generator, ``communities`` per graph with sizes proportional
    to ``rank ** -zipf_exponent`` (or equal sizes of contiguous position blocks with
    ``zipf_exponent=None``).  For benchmarks and tests that need a whole model running through
    the plug-in without a graph partitioner.
    """

    def __init__(self, *, communities: int, zipf_exponent: float | None = 1.1, seed: int = 0) -> None:
        if communities <= 0:
            raise ValueError("communities must be positive")
        self.communities = communities
        self.zipf_exponent = zipf_exponent
        self.seed = seed
        self.edges_seen: dict[int, tuple[int, ...]] = {}
        self.adjacency_edges: dict[int, int] = {}

    def __call__(self, *, layer_idx: int, topk_indices: torch.Tensor, topk_scores: torch.Tensor,
                 keys: torch.Tensor, num_sink: int, max_decode_tokens: int,
                 aggregation: GraphAggregation | str, lam: float = 0.5,
                 **_: object) -> SyntheticPartitionedLayer:
        aggregation = GraphAggregation(aggregation)
        kv_heads, length, _dim = keys.shape
        query_heads = int(topk_indices.shape[0])
        self.edges_seen[layer_idx] = tuple(topk_indices.shape)
        graphs = aggregation.graph_count(query_heads=query_heads, kv_heads=kv_heads)
        count = min(self.communities, max(1, length - num_sink))
        labels = torch.empty((graphs, length), dtype=torch.int64)
        for graph in range(graphs):
            generator = torch.Generator().manual_seed((self.seed * 1000003 + layer_idx) * 4099 + graph)
            if self.zipf_exponent is None:
                ids = (torch.arange(length) * count) // length
            else:
                sizes = zipf_sizes(length, count, self.zipf_exponent, generator)
                ids = torch.repeat_interleave(torch.arange(count), sizes)[torch.randperm(length, generator=generator)]
            labels[graph] = ids
        labels = labels.to(torch.int32).to(keys.device)
        weights: dict[str, torch.Tensor] = {}
        if keys.is_cuda:
            shaped = reshape_by_aggregation(topk_indices, topk_scores, aggregation=aggregation,
                                            num_kv_heads=kv_heads, num_sink=num_sink)
            source, destination, weight = build_adjacency(*shaped, seq_len=length, lam=lam)
            self.adjacency_edges[layer_idx] = int(source.numel())
            capacity = int(labels.max()) + 1 + max_decode_tokens
            community_weight, total_weight = init_modularity_state(
                labels, source.long(), destination.long(), weight, community_capacity=capacity)
            weights = dict(community_weight=community_weight, total_weight=total_weight)
        assembled = assemble_layer(
            labels, keys, aggregation=aggregation, query_heads=query_heads,
            num_sink=num_sink, max_decode_tokens=max_decode_tokens, **weights,
        )
        return SyntheticPartitionedLayer(
            layer_idx=layer_idx,
            member_offsets=assembled.member_offsets,
            member_positions=assembled.member_positions,
            community_counts=assembled.num_communities,
            centroids=assembled.centroids,
            community_sizes=assembled.community_sizes,
            community_weight=assembled.community_weight,
            total_weight=assembled.total_weight,
            token_communities=assembled.token_communities,
            retrieval_to_graph=assembled.retrieval_to_graph,
            retrieval_to_kv=assembled.retrieval_to_kv,
            prefill_seq_len=length,
            query_heads=query_heads,
            kv_heads=kv_heads,
            aggregation=aggregation,
        )


def make_query(*, seed: int, query_heads: int, integer_valued: bool = False) -> torch.Tensor:
    generator = torch.Generator().manual_seed(seed)
    if integer_valued:
        return torch.randint(-2, 3, (query_heads, HEAD_DIM), generator=generator).to(torch.bfloat16)
    return torch.randn((query_heads, HEAD_DIM), generator=generator).to(torch.bfloat16)


__all__ = ["SyntheticLayer", "SyntheticPartitionedLayer", "SyntheticPartitioner", "make_layer", "make_query",
           "zipf_sizes"]

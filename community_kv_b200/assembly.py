"""Assembly of the decode state from community labels.

Produces the layout the decode kernels consume - per-community member lists in
recency-descending order, e4m3 mean-key centroids with decode headroom, the
modularity bookkeeping and the retrieval-head -> (graph, KV head) maps - with the
semantics of the reference's ``build_member_csr``, ``compute_centroids``,
``init_modularity_state`` and ``aggregation_mappings``
(``community_kv/graph/partition.py:71-94, 382-535``).  CUDA tensors go through the
assembly kernels of the CUDA library (``ckv_assemble_*``; bf16 keys); CPU tensors
take a plain torch path that exists for building fixtures and synthetic workloads
on the host.  The Leiden partition that produces the labels stays on the host and
is not part of this package.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from community_kv_b200.config import GraphAggregation

FP8_MAX = 448.0


def aggregation_mappings(
    aggregation: GraphAggregation | str,
    *,
    query_heads: int,
    kv_heads: int,
    device: torch.device | str = "cpu",
) -> tuple[torch.Tensor, torch.Tensor]:
    """``(retrieval_to_graph, retrieval_to_kv)`` int32 vectors for an aggregation mode."""

    aggregation = GraphAggregation(aggregation)
    heads = aggregation.retrieval_head_count(query_heads=query_heads, kv_heads=kv_heads)
    index = torch.arange(heads, dtype=torch.int32, device=device)
    if aggregation is GraphAggregation.PER_QUERY_HEAD:
        return index, index // (query_heads // kv_heads)
    if aggregation is GraphAggregation.QUERY_GROUP:
        return index, index.clone()
    return torch.zeros_like(index), index


def build_member_csr(
    community_ids: torch.Tensor,
    community_counts: torch.Tensor,
    *,
    num_sink: int,
) -> tuple[torch.Tensor, torch.Tensor]:
    """CSR of non-sink positions by community; members sorted newest first."""

    graphs, length = community_ids.shape
    widest = int(community_counts.max())
    if community_ids.is_cuda:
        return _member_csr_cuda(community_ids, widest, num_sink)
    labels = community_ids[:, num_sink:].long()
    where = torch.arange(num_sink, length, device=community_ids.device).expand(graphs, -1)
    order = (labels * length + (length - 1 - where)).argsort(dim=1)
    member_positions = where.gather(1, order).to(torch.int32)
    histogram = torch.zeros((graphs, widest), dtype=torch.int64, device=community_ids.device)
    histogram.scatter_add_(1, labels, torch.ones_like(labels))
    offsets = torch.zeros((graphs, widest + 1), dtype=torch.int32, device=community_ids.device)
    offsets[:, 1:] = histogram.cumsum(1).to(torch.int32)
    return offsets, member_positions


def compute_centroids(
    community_ids: torch.Tensor,
    community_counts: torch.Tensor,
    keys: torch.Tensor,
    *,
    retrieval_to_graph: torch.Tensor | None = None,
    retrieval_to_kv: torch.Tensor | None = None,
    num_sink: int,
    max_decode_tokens: int,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-retrieval-head e4m3 mean keys ``[R, max count + headroom, D]`` and sizes."""

    graphs, length = community_ids.shape
    if keys.ndim != 3 or keys.shape[1] != length:
        raise ValueError("keys must have shape [KV heads, sequence, head dim]")
    if retrieval_to_graph is None or retrieval_to_kv is None:
        if keys.shape[0] != graphs:
            raise ValueError("aggregation mappings are required when graph and KV counts differ")
        retrieval_to_graph = torch.arange(graphs, dtype=torch.int32, device=community_ids.device)
        retrieval_to_kv = retrieval_to_graph
    heads = retrieval_to_graph.numel()
    live = int(community_counts.max())
    capacity = live + max_decode_tokens
    dim = keys.shape[-1]
    if community_ids.is_cuda and keys.dtype == torch.bfloat16 and dim == 128:
        return _centroids_cuda(community_ids, keys, retrieval_to_graph, retrieval_to_kv, live, capacity, num_sink)
    labels = community_ids[retrieval_to_graph.long(), num_sink:].long()
    rows = keys[retrieval_to_kv.long(), num_sink:].float()
    sums = torch.zeros((heads, capacity, dim), dtype=torch.float32, device=keys.device)
    sums.scatter_add_(1, labels.unsqueeze(-1).expand(-1, -1, dim), rows)
    sizes = torch.zeros((heads, capacity), dtype=torch.int32, device=keys.device)
    sizes.scatter_add_(1, labels, torch.ones_like(labels, dtype=torch.int32))
    sums[:, :live] /= sizes[:, :live].float().clamp_min(1).unsqueeze(-1)
    return sums.clamp_(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn), sizes


def _native():
    from community_kv_b200 import native

    return native


def _check(status: int) -> None:
    if status:
        native = _native()
        raise native.NativeError(native.library().ckv_status_string(status).decode())


def _member_csr_cuda(community_ids: torch.Tensor, widest: int, num_sink: int) -> tuple[torch.Tensor, torch.Tensor]:
    native = _native()
    graphs, length = community_ids.shape
    labels = community_ids.to(torch.int32).contiguous()
    device = labels.device
    counts = torch.empty((graphs, widest), dtype=torch.int32, device=device)
    offsets = torch.empty((graphs, widest + 1), dtype=torch.int32, device=device)
    positions = torch.empty((graphs, length - num_sink), dtype=torch.int32, device=device)
    with torch.cuda.device(device):
        _check(native.library().ckv_assemble_member_csr(
            labels.data_ptr(), graphs, length, num_sink, widest, counts.data_ptr(), offsets.data_ptr(),
            positions.data_ptr(), length - num_sink, native.current_stream(device)))
    return offsets, positions


def _centroids_cuda(community_ids, keys, retrieval_to_graph, retrieval_to_kv, live, capacity, num_sink):
    native = _native()
    device = keys.device
    counts = torch.full((community_ids.shape[0],), live, dtype=torch.int32, device=device)
    offsets, positions = build_member_csr(community_ids, counts, num_sink=num_sink)
    heads = retrieval_to_graph.numel()
    if keys.stride(-1) != 1:
        keys = keys.contiguous()
    centroids = torch.empty((heads, capacity, 128), dtype=torch.float8_e4m3fn, device=device)
    sizes = torch.empty((heads, capacity), dtype=torch.int32, device=device)
    to_graph = retrieval_to_graph.to(torch.int32).contiguous()
    to_kv = retrieval_to_kv.to(torch.int32).contiguous()
    with torch.cuda.device(device):
        _check(native.library().ckv_assemble_centroids(
            offsets.data_ptr(), positions.data_ptr(), live, positions.shape[1], keys.data_ptr(),
            keys.stride(0), keys.stride(1), to_graph.data_ptr(), to_kv.data_ptr(), heads, live, capacity,
            centroids.data_ptr(), sizes.data_ptr(), native.current_stream(device)))
    return centroids, sizes


def init_modularity_state(
    community_ids: torch.Tensor,
    edge_src: torch.Tensor,
    edge_dst: torch.Tensor,
    edge_weight: torch.Tensor,
    *,
    community_capacity: int,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Community weights ``[graphs, capacity]`` and total weight ``[graphs]`` of an edge list whose
    vertices are flat ``graph * length + position`` indices (the reference's
    ``init_modularity_state``, ``community_kv/graph/partition.py:495-535``)."""

    graphs, length = community_ids.shape
    device = community_ids.device
    weight = torch.zeros((graphs, community_capacity), dtype=torch.float32, device=device)
    total = torch.zeros((graphs,), dtype=torch.float32, device=device)
    if not edge_src.numel():
        return weight, total
    if community_ids.is_cuda:
        native = _native()
        labels = community_ids.to(torch.int32).contiguous()
        source, destination = edge_src.long().contiguous(), edge_dst.long().contiguous()
        values = edge_weight.float().contiguous()
        with torch.cuda.device(device):
            _check(native.library().ckv_assemble_modularity(
                labels.data_ptr(), graphs, length, source.data_ptr(), destination.data_ptr(), values.data_ptr(),
                source.numel(), community_capacity, weight.data_ptr(), total.data_ptr(),
                native.current_stream(device)))
        return weight, total
    source, destination = edge_src.long(), edge_dst.long()
    graph = source // length
    flat = weight.view(-1)
    values = edge_weight.float()
    flat.scatter_add_(0, graph * community_capacity + community_ids[graph, source % length].long(), values)
    flat.scatter_add_(0, graph * community_capacity + community_ids[graph, destination % length].long(), values)
    total.scatter_add_(0, graph, 2.0 * values)
    return weight, total


def reshape_by_aggregation(
    topk_indices: torch.Tensor,
    topk_scores: torch.Tensor,
    *,
    aggregation: GraphAggregation | str,
    num_kv_heads: int,
    num_sink: int,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Per-query-head prefill edges ``[Hq, rows, kappa]`` -> per-graph rows and their positions.

    Row ``i`` of the prefill kernel's output belongs to position ``kappa - 1 + num_sink + i``;
    a graph that several query heads share gets those heads' rows one after the other (the
    reference's ``_reshape_by_aggregation``, ``community_kv/graph/partition.py:96-147``).
    """

    aggregation = GraphAggregation(aggregation)
    heads, rows, kappa = topk_indices.shape
    group = heads // num_kv_heads
    first = kappa - 1 + num_sink
    positions = torch.arange(first, first + rows, dtype=torch.int64, device=topk_indices.device)
    if aggregation is GraphAggregation.PER_QUERY_HEAD:
        return topk_indices, topk_scores, positions.unsqueeze(0).expand(heads, -1)
    if aggregation is GraphAggregation.QUERY_GROUP:
        return (
            topk_indices.reshape(num_kv_heads, group * rows, kappa),
            topk_scores.reshape(num_kv_heads, group * rows, kappa),
            positions.repeat(group).unsqueeze(0).expand(num_kv_heads, -1),
        )
    return (
        topk_indices.reshape(1, heads * rows, kappa),
        topk_scores.reshape(1, heads * rows, kappa),
        positions.repeat(heads).unsqueeze(0),
    )


def build_adjacency(
    topk_indices: torch.Tensor,
    topk_scores: torch.Tensor,
    query_positions: torch.Tensor,
    *,
    seq_len: int,
    lam: float,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Coalesced undirected edge list ``(src int32, dst int32, weight fp32)`` of the batched graph.

    CUDA tensors only (``ckv_build_adjacency``): this is the consumer of the prefill kernel's
    edges, there is no host variant.  Same result as the reference's ``build_adjacency``
    (``community_kv/graph/partition.py:168-249``), with the duplicate weights added in the
    reference's enumeration order.
    """

    if not topk_indices.is_cuda:
        raise ValueError("build_adjacency runs on CUDA tensors")
    if topk_indices.ndim != 3 or topk_scores.shape != topk_indices.shape:
        raise ValueError("top-k tensors must have shape [graphs, rows, kappa]")
    native = _native()
    graphs, rows, kappa = topk_indices.shape
    device = topk_indices.device
    indices = topk_indices.to(torch.int32).contiguous()
    scores = topk_scores.float().contiguous()
    positions = query_positions.to(torch.int64).expand(graphs, rows).contiguous()
    lib = native.library()
    raw = int(lib.ckv_adjacency_raw_edges(graphs, rows, kappa, float(lam)))
    scratch = torch.empty((int(lib.ckv_adjacency_scratch_bytes(graphs, rows, kappa, float(lam))),),
                          dtype=torch.uint8, device=device)
    source = torch.empty((raw,), dtype=torch.int32, device=device)
    destination = torch.empty((raw,), dtype=torch.int32, device=device)
    weight = torch.empty((raw,), dtype=torch.float32, device=device)
    count = torch.zeros((1,), dtype=torch.int64, device=device)
    with torch.cuda.device(device):
        _check(lib.ckv_build_adjacency(
            indices.data_ptr(), scores.data_ptr(), positions.data_ptr(), graphs, rows, kappa, int(seq_len),
            float(lam), source.data_ptr(), destination.data_ptr(), weight.data_ptr(), raw, count.data_ptr(),
            scratch.data_ptr(), scratch.numel(), native.current_stream(device)))
    edges = int(count.item())
    return source[:edges], destination[:edges], weight[:edges]


@dataclass(slots=True)
class AssembledLayer:
    """Everything ``DecodeRuntime.prepare_layer`` takes, built from labels and keys."""

    member_offsets: torch.Tensor
    member_positions: torch.Tensor
    num_communities: torch.Tensor
    centroids: torch.Tensor
    community_sizes: torch.Tensor
    community_weight: torch.Tensor
    total_weight: torch.Tensor
    token_communities: torch.Tensor
    retrieval_to_graph: torch.Tensor
    retrieval_to_kv: torch.Tensor


def assemble_layer(
    community_ids: torch.Tensor,
    keys: torch.Tensor,
    *,
    aggregation: GraphAggregation | str,
    query_heads: int,
    num_sink: int,
    max_decode_tokens: int,
    community_weight: torch.Tensor | None = None,
    total_weight: torch.Tensor | None = None,
) -> AssembledLayer:
    """Decode state of one layer from dense labels ``[graphs, S]`` and keys ``[Hkv, S, D]``.

    Sink positions must carry labels of their own (size-zero communities after
    the sink exclusion), like the reference's isolated-vertex fill.  Modularity
    weights default to the community sizes (a unit-weight star per member),
    which keeps the online rule well defined for synthetic labels.
    """

    graphs, length = community_ids.shape
    kv_heads = keys.shape[0]
    counts = (community_ids.amax(dim=1) + 1).to(torch.int32)
    to_graph, to_kv = aggregation_mappings(
        aggregation, query_heads=query_heads, kv_heads=kv_heads, device=keys.device
    )
    centroids, sizes = compute_centroids(
        community_ids,
        counts,
        keys,
        retrieval_to_graph=to_graph,
        retrieval_to_kv=to_kv,
        num_sink=num_sink,
        max_decode_tokens=max_decode_tokens,
    )
    offsets, positions = build_member_csr(community_ids, counts, num_sink=num_sink)
    capacity = centroids.shape[1]
    if community_weight is None:
        community_weight = torch.zeros((graphs, capacity), dtype=torch.float32, device=keys.device)
        leaders = torch.unique(to_graph.long())
        community_weight[:] = sizes[leaders].float() if leaders.numel() == graphs else 0.0
    if total_weight is None:
        total_weight = community_weight.sum(dim=1)
    labels = torch.full(
        (graphs, length + max_decode_tokens), -1, dtype=torch.int32, device=keys.device
    )
    labels[:, :length] = community_ids
    return AssembledLayer(
        member_offsets=offsets,
        member_positions=positions,
        num_communities=counts,
        centroids=centroids,
        community_sizes=sizes,
        community_weight=community_weight,
        total_weight=total_weight,
        token_communities=labels,
        retrieval_to_graph=to_graph,
        retrieval_to_kv=to_kv,
    )


__all__ = [
    "AssembledLayer",
    "aggregation_mappings",
    "assemble_layer",
    "build_adjacency",
    "build_member_csr",
    "compute_centroids",
    "init_modularity_state",
    "reshape_by_aggregation",
]

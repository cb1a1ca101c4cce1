"""Cache / community-label layout and fixed-address workspaces of the decode path.

The tensors keep the reference's names, dtypes and shapes
(``community_kv/graph/state.py:16-349``, the workspace classes of
``community_kv/attention/kernels/centroid_selection.py:191-327``,
``segmented_attention.py:953-1013`` and ``graph/kernels/online_update.py``).
Every ``allocate`` additionally accepts ``batch``: with ``batch=None`` the
shapes are exactly the reference's per-layer shapes; with an integer every
tensor gains a leading, contiguous batch axis (one slot per sequence), which is
the layout the CUDA library consumes in one launch.
"""

from __future__ import annotations

from collections.abc import Sequence
from dataclasses import dataclass, fields

import torch

HEAD_DIM = 128
ATTENTION_TILE = 64
KAPPA = 8
PARTIAL_STRIDE = 132
DEFAULT_SPLITS = 8


def _lead(batch: int | None) -> tuple[int, ...]:
    if batch is None:
        return ()
    if batch <= 0:
        raise ValueError("batch must be positive")
    return (batch,)


def _int32(name: str, tensor: torch.Tensor) -> None:
    if tensor.dtype != torch.int32:
        raise TypeError(f"{name} must use torch.int32")


RESIDENT_ATTENTION_CTAS = 3 * 148  # three attention CTAs fit one SM; a B200 has 148 SMs


def choose_splits(token_budget: int, units: int, requested: int | None = None) -> int:
    """Attention CTAs per retrieval head.

    By default the (sequence, head) units of one launch share a single wave of
    resident CTAs; a head's tokens are cut into 16-token steps, so at most
    ``token_budget // 16`` (and never more than 32) CTAs can work on one head.
    With few units the default stops at eight, the largest thread-block cluster,
    so that ``ckv_decode_layer`` stays a single launch.
    """

    if requested:
        wanted = requested
    else:
        wanted = max(1, RESIDENT_ATTENTION_CTAS // max(units, 1))
        # Up to eight splits the whole layer is one cluster launch; more only pay off when
        # a split would otherwise have to walk through more than 512 tokens.
        if wanted > 8 and token_budget // 8 <= 512:
            wanted = 8
    return max(1, min(wanted, 32, token_budget // 16))


@dataclass(slots=True)
class PrefillCSR:
    """Immutable community -> prefill-position index (members newest first)."""

    member_offsets: torch.Tensor
    member_positions: torch.Tensor
    community_counts: torch.Tensor

    @property
    def graph_count(self) -> int:
        return self.member_offsets.shape[-2]

    @property
    def community_capacity(self) -> int:
        return self.member_offsets.shape[-1] - 1

    def validate(self) -> None:
        for item in fields(self):
            _int32(item.name, getattr(self, item.name))
        if self.member_offsets.ndim != 2 or self.member_positions.ndim != 2:
            raise ValueError("member offsets and positions must be rank two")
        graphs = self.member_offsets.shape[0]
        if self.community_counts.shape != (graphs,):
            raise ValueError("community_counts must have one entry per graph")
        if self.member_positions.shape[0] != graphs:
            raise ValueError("member_positions must have one row per graph")
        offsets = self.member_offsets.cpu().long()
        counts = self.community_counts.cpu().long()
        width = self.member_positions.shape[1]
        for graph in range(graphs):
            count = int(counts[graph])
            if not 0 <= count < offsets.shape[1]:
                raise ValueError("community count exceeds offset capacity")
            row = offsets[graph, : count + 1]
            if int(row[0]) != 0 or bool((row[1:] < row[:-1]).any()):
                raise ValueError("active CSR offsets must start at zero and be monotonic")
            if int(row[-1]) > width:
                raise ValueError("CSR offsets exceed member-position capacity")

    def members(self, graph: int, community: int) -> torch.Tensor:
        if not 0 <= graph < self.graph_count:
            raise IndexError("graph is outside the CSR")
        if not 0 <= community < int(self.community_counts[graph]):
            raise IndexError("community is outside the active CSR")
        low = int(self.member_offsets[graph, community])
        high = int(self.member_offsets[graph, community + 1])
        return self.member_positions[graph, low:high]


_DELTA_CHUNK_FIELDS = ("chunk_start", "chunk_capacity", "chunk_size", "chunk_next", "chunk_previous")
_DELTA_TABLE_FIELDS = ("community_head", "community_tail", "community_sizes")
_DELTA_CURSOR_FIELDS = ("next_free_chunk", "next_free_position")
_DELTA_MINUS_ONE = {"positions", "chunk_start", "chunk_next", "chunk_previous", "community_head", "community_tail"}


@dataclass(slots=True)
class DecodeDeltaChunks:
    """Per-community chains of geometrically growing chunks for decode-time members."""

    positions: torch.Tensor
    chunk_start: torch.Tensor
    chunk_capacity: torch.Tensor
    chunk_size: torch.Tensor
    chunk_next: torch.Tensor
    chunk_previous: torch.Tensor
    community_head: torch.Tensor
    community_tail: torch.Tensor
    community_sizes: torch.Tensor
    next_free_chunk: torch.Tensor
    next_free_position: torch.Tensor

    @classmethod
    def allocate(
        cls,
        *,
        graph_count: int,
        community_capacity: int,
        max_decode_tokens: int,
        device: torch.device | str = "cpu",
        batch: int | None = None,
    ) -> "DecodeDeltaChunks":
        if min(graph_count, community_capacity, max_decode_tokens) <= 0:
            raise ValueError("all capacities must be positive")
        lead = _lead(batch)
        shapes = {"positions": (graph_count, 2 * max_decode_tokens)}
        shapes.update({name: (graph_count, max_decode_tokens) for name in _DELTA_CHUNK_FIELDS})
        shapes.update({name: (graph_count, community_capacity) for name in _DELTA_TABLE_FIELDS})
        shapes.update({name: (graph_count,) for name in _DELTA_CURSOR_FIELDS})
        tensors = {
            name: torch.full(
                lead + shape,
                -1 if name in _DELTA_MINUS_ONE else 0,
                dtype=torch.int32,
                device=device,
            )
            for name, shape in shapes.items()
        }
        return cls(**tensors)

    @property
    def graph_count(self) -> int:
        return self.positions.shape[-2]

    @property
    def position_capacity(self) -> int:
        return self.positions.shape[-1]

    @property
    def chunk_capacity_per_graph(self) -> int:
        return self.chunk_start.shape[-1]

    @property
    def community_capacity(self) -> int:
        return self.community_head.shape[-1]

    def validate(self) -> None:
        for item in fields(self):
            _int32(item.name, getattr(self, item.name))
        if self.positions.ndim != 2 or self.chunk_start.ndim != 2:
            raise ValueError("delta position and chunk pools must be rank two")
        graphs = self.positions.shape[0]
        if self.chunk_start.shape[0] != graphs or min(self.positions.shape[1], self.chunk_start.shape[1]) <= 0:
            raise ValueError("delta pool capacities must be positive")
        for name in _DELTA_CHUNK_FIELDS:
            if getattr(self, name).shape != self.chunk_start.shape:
                raise ValueError("chunk metadata shapes must match")
        if self.community_head.ndim != 2 or self.community_head.shape[0] != graphs:
            raise ValueError("community chunk tables must match graph count")
        for name in _DELTA_TABLE_FIELDS:
            if getattr(self, name).shape != self.community_head.shape:
                raise ValueError("community chunk tables and sizes must match")
        for name in _DELTA_CURSOR_FIELDS:
            if getattr(self, name).shape != (graphs,):
                raise ValueError(f"{name} must have one entry per graph")

    def append(self, graph: int, community: int, position: int) -> None:
        """Host-side append with the same chunk-growth rule as the device update."""

        if not 0 <= graph < self.graph_count:
            raise IndexError("graph is outside the delta store")
        if not 0 <= community < self.community_capacity:
            raise IndexError("community is outside the delta store")
        tail = int(self.community_tail[graph, community])
        used = int(self.chunk_size[graph, tail]) if tail >= 0 else 0
        room = int(self.chunk_capacity[graph, tail]) if tail >= 0 else 0
        if tail < 0 or used == room:
            fresh = int(self.next_free_chunk[graph])
            start = int(self.next_free_position[graph])
            capacity = 2 * room if tail >= 0 else 1
            if fresh >= self.chunk_capacity_per_graph:
                raise RuntimeError("decode-delta chunk capacity exhausted")
            if start + capacity > self.position_capacity:
                raise RuntimeError("decode-delta position capacity exhausted")
            self.next_free_chunk[graph] = fresh + 1
            self.next_free_position[graph] = start + capacity
            self.chunk_start[graph, fresh] = start
            self.chunk_capacity[graph, fresh] = capacity
            self.chunk_previous[graph, fresh] = tail
            if tail >= 0:
                self.chunk_next[graph, tail] = fresh
            else:
                self.community_head[graph, community] = fresh
            self.community_tail[graph, community] = fresh
            tail, used = fresh, 0
        self.positions[graph, int(self.chunk_start[graph, tail]) + used] = position
        self.chunk_size[graph, tail] = used + 1
        self.community_sizes[graph, community] += 1

    def members(self, graph: int, community: int) -> torch.Tensor:
        """Decode-time members of one community, oldest first."""

        size = int(self.community_sizes[graph, community])
        pieces = []
        chunk = int(self.community_head[graph, community])
        gathered = 0
        while chunk >= 0 and gathered < size:
            count = int(self.chunk_size[graph, chunk])
            start = int(self.chunk_start[graph, chunk])
            pieces.append(self.positions[graph, start : start + count])
            gathered += count
            chunk = int(self.chunk_next[graph, chunk])
        if gathered != size:
            raise RuntimeError("decode-delta chunk chain ended early")
        if not pieces:
            return torch.empty((0,), dtype=torch.int32, device=self.positions.device)
        return torch.cat(pieces)


@dataclass(slots=True)
class MutableGraphState:
    """Centroids, sizes, modularity weights and labels mutated once per decode token."""

    centroids: torch.Tensor
    community_sizes: torch.Tensor
    community_counts: torch.Tensor
    community_weight: torch.Tensor
    total_weight: torch.Tensor
    token_communities: torch.Tensor
    deltas: DecodeDeltaChunks
    retrieval_to_graph: torch.Tensor
    retrieval_to_kv: torch.Tensor

    @property
    def graph_count(self) -> int:
        return self.total_weight.shape[-1]

    @property
    def retrieval_head_count(self) -> int:
        return self.centroids.shape[-3]

    @property
    def community_capacity(self) -> int:
        return self.centroids.shape[-2]

    @property
    def head_dim(self) -> int:
        return self.centroids.shape[-1]

    def tensors(self) -> list[torch.Tensor]:
        own = [getattr(self, item.name) for item in fields(self) if item.name != "deltas"]
        return own + [getattr(self.deltas, item.name) for item in fields(self.deltas)]

    def validate(self) -> None:
        if self.centroids.ndim != 3:
            raise ValueError("centroids must have shape [graphs, communities, dim]")
        if self.centroids.dtype not in (torch.float8_e4m3fn, torch.float32):
            raise TypeError("centroids must use FP8 E4M3 (the reference's layout) or FP32")
        heads, capacity, _ = self.centroids.shape
        graphs = self.graph_count
        if self.community_sizes.shape != (heads, capacity):
            raise ValueError("community_sizes must match centroid rows")
        _int32("community_sizes", self.community_sizes)
        if self.community_counts.shape != (heads,):
            raise ValueError("community_counts must have one entry per retrieval head")
        _int32("community_counts", self.community_counts)
        if self.community_weight.shape != (graphs, capacity):
            raise ValueError("community_weight must have one row per graph")
        if self.community_weight.dtype != torch.float32:
            raise TypeError("community_weight must use float32")
        if self.total_weight.shape != (graphs,):
            raise ValueError("total_weight must have one entry per graph")
        if self.total_weight.dtype != torch.float32:
            raise TypeError("total_weight must use float32")
        if self.token_communities.ndim != 2 or self.token_communities.shape[0] != graphs:
            raise ValueError("token_communities must have one row per graph")
        _int32("token_communities", self.token_communities)
        self.deltas.validate()
        if self.deltas.graph_count != graphs:
            raise ValueError("delta pages must match graph count")
        if self.deltas.community_capacity != capacity:
            raise ValueError("delta pages must match community capacity")
        for name in ("retrieval_to_graph", "retrieval_to_kv"):
            mapping = getattr(self, name)
            _int32(name, mapping)
            if mapping.shape != (heads,):
                raise ValueError(f"{name} must have one entry per retrieval head")
        if (
            int(self.retrieval_to_graph.min()) < 0
            or int(self.retrieval_to_graph.max()) >= graphs
            or int(self.retrieval_to_kv.min()) < 0
        ):
            raise ValueError("retrieval mapping index is out of bounds")
        device = self.centroids.device
        if any(tensor.device != device for tensor in self.tensors()):
            raise ValueError("all mutable graph tensors must share one device")


@dataclass(frozen=True, slots=True)
class PackedSegments:
    """Selected-community descriptors consumed by the attention operator."""

    communities: torch.Tensor
    cumulative_ends: torch.Tensor
    descriptor_counts: torch.Tensor
    tile_descriptors: torch.Tensor
    token_budget: int
    num_sink: int


@dataclass(slots=True)
class CentroidSelectionWorkspace:
    """Preallocated scoring and descriptor-selection outputs."""

    scores: torch.Tensor
    score_cover: torch.Tensor | None
    native_threshold: torch.Tensor
    communities: torch.Tensor
    cumulative_ends: torch.Tensor
    descriptor_counts: torch.Tensor
    tile_descriptors: torch.Tensor
    positions: torch.Tensor
    token_budget: int
    num_sink: int
    max_communities: int = 0

    @classmethod
    def allocate(
        cls,
        *,
        kv_heads: int,
        community_capacity: int,
        token_budget: int,
        num_sink: int,
        score_community_counts: Sequence[int] | None = None,
        score_headroom: int = 0,
        device: torch.device | str,
        batch: int | None = None,
        max_communities: int = 0,
    ) -> "CentroidSelectionWorkspace":
        if kv_heads <= 0 or community_capacity <= 0:
            raise ValueError("head and community capacities must be positive")
        if token_budget <= 0 or token_budget % ATTENTION_TILE:
            raise ValueError("token budget must be a positive multiple of 64")
        if num_sink < 0 or num_sink + 1 >= token_budget:
            raise ValueError("num_sink leaves no selected-token capacity")
        if score_headroom < 0:
            raise ValueError("score_headroom must be nonnegative")
        if max_communities < 0:
            raise ValueError("max_communities must be nonnegative")
        lead = _lead(batch)
        cover = None
        if score_community_counts is not None:
            counts = torch.as_tensor(score_community_counts, dtype=torch.int64).reshape(-1, kv_heads)
            if counts.shape[0] != (batch or 1):
                raise ValueError("score counts must contain one value per KV head")
            if bool((counts <= 0).any()) or bool((counts > community_capacity).any()):
                raise ValueError("score counts must fit the community capacity")
            cover = (
                (counts + score_headroom)
                .clamp(max=community_capacity)
                .to(torch.int32)
                .reshape(lead + (kv_heads,))
                .to(device)
            )
        selected = token_budget - num_sink - 1
        heads = lead + (kv_heads,)
        return cls(
            scores=torch.zeros(heads + (community_capacity,), dtype=torch.float16, device=device),
            score_cover=cover,
            native_threshold=torch.full(heads + (4,), -1, dtype=torch.int32, device=device),
            communities=torch.full(heads + (selected,), -1, dtype=torch.int32, device=device),
            cumulative_ends=torch.zeros(heads + (selected,), dtype=torch.int32, device=device),
            descriptor_counts=torch.zeros(heads, dtype=torch.int32, device=device),
            tile_descriptors=torch.zeros(
                heads + (token_budget // ATTENTION_TILE,), dtype=torch.int32, device=device
            ),
            positions=torch.full(heads + (token_budget,), -1, dtype=torch.int32, device=device),
            token_budget=token_budget,
            num_sink=num_sink,
            max_communities=max_communities,
        )

    @property
    def selected_budget(self) -> int:
        return self.token_budget - self.num_sink - 1

    @property
    def community_capacity(self) -> int:
        return self.scores.shape[-1]

    @property
    def kv_heads(self) -> int:
        return self.scores.shape[-2]

    @property
    def batch(self) -> int | None:
        return self.scores.shape[0] if self.scores.ndim == 3 else None

    def packed_segments(self) -> PackedSegments:
        return PackedSegments(
            communities=self.communities,
            cumulative_ends=self.cumulative_ends,
            descriptor_counts=self.descriptor_counts,
            tile_descriptors=self.tile_descriptors,
            token_budget=self.token_budget,
            num_sink=self.num_sink,
        )


@dataclass(slots=True)
class SegmentedAttentionWorkspace:
    """Split partials and outputs of the gather + attention operator."""

    group_size: int
    splits: int
    partials: torch.Tensor
    partial_topk_packed: torch.Tensor
    output: torch.Tensor
    lse: torch.Tensor
    topk_scores: torch.Tensor
    topk_positions: torch.Tensor
    status: torch.Tensor

    @classmethod
    def allocate(
        cls,
        *,
        kv_heads: int,
        group_size: int = 4,
        token_budget: int,
        dtype: torch.dtype,
        device: torch.device | str,
        batch: int | None = None,
        splits: int | None = None,
    ) -> "SegmentedAttentionWorkspace":
        if kv_heads <= 0:
            raise ValueError("kv_heads must be positive")
        if not 1 <= group_size <= 16:
            raise ValueError("group_size must be in [1, 16]")
        if token_budget <= 0 or token_budget % ATTENTION_TILE:
            raise ValueError("token_budget must be a positive multiple of 64")
        if dtype != torch.bfloat16:
            raise TypeError("the attention operator requires BF16 Q/K/V")
        splits = choose_splits(token_budget, (batch or 1) * kv_heads, splits)
        lead = _lead(batch)
        heads = lead + (kv_heads,)
        query_heads = lead + (kv_heads * group_size,)
        return cls(
            group_size=group_size,
            splits=splits,
            partials=torch.zeros(
                heads + (splits, group_size, PARTIAL_STRIDE), dtype=torch.float32, device=device
            ),
            partial_topk_packed=torch.zeros(heads + (splits, KAPPA), dtype=torch.int64, device=device),
            output=torch.zeros(query_heads + (HEAD_DIM,), dtype=dtype, device=device),
            lse=torch.zeros(query_heads, dtype=torch.float32, device=device),
            topk_scores=torch.zeros(heads + (KAPPA,), dtype=torch.float32, device=device),
            topk_positions=torch.zeros(heads + (KAPPA,), dtype=torch.int32, device=device),
            status=torch.zeros((1,), dtype=torch.int32, device=device),
        )


@dataclass(slots=True)
class OnlineUpdateWorkspace:
    """Per-graph results of the online assignment: community id and overflow bits."""

    assigned_communities: torch.Tensor
    overflow: torch.Tensor

    @classmethod
    def allocate(
        cls,
        *,
        graph_count: int,
        device: torch.device | str,
        batch: int | None = None,
    ) -> "OnlineUpdateWorkspace":
        if graph_count <= 0:
            raise ValueError("graph_count must be positive")
        shape = _lead(batch) + (graph_count,)
        return cls(
            assigned_communities=torch.zeros(shape, dtype=torch.int32, device=device),
            overflow=torch.zeros(shape, dtype=torch.int32, device=device),
        )


@dataclass(slots=True)
class DecodeLayerWorkspace:
    """The three workspaces of one layer transition."""

    selection: CentroidSelectionWorkspace
    attention: SegmentedAttentionWorkspace
    update: OnlineUpdateWorkspace

    @classmethod
    def allocate(
        cls,
        *,
        retrieval_head_count: int,
        graph_count: int,
        group_size: int = 4,
        community_capacity: int,
        token_budget: int,
        num_sink: int,
        dtype: torch.dtype,
        device: torch.device | str,
        score_community_counts: Sequence[int] | None = None,
        score_headroom: int = 0,
        batch: int | None = None,
        splits: int | None = None,
        max_communities: int = 0,
    ) -> "DecodeLayerWorkspace":
        return cls(
            selection=CentroidSelectionWorkspace.allocate(
                kv_heads=retrieval_head_count,
                community_capacity=community_capacity,
                token_budget=token_budget,
                num_sink=num_sink,
                score_community_counts=score_community_counts,
                score_headroom=score_headroom,
                device=device,
                batch=batch,
                max_communities=max_communities,
            ),
            attention=SegmentedAttentionWorkspace.allocate(
                kv_heads=retrieval_head_count,
                group_size=group_size,
                token_budget=token_budget,
                dtype=dtype,
                device=device,
                batch=batch,
                splits=splits,
            ),
            update=OnlineUpdateWorkspace.allocate(
                graph_count=graph_count, device=device, batch=batch
            ),
        )


__all__ = [
    "ATTENTION_TILE",
    "CentroidSelectionWorkspace",
    "DecodeDeltaChunks",
    "DecodeLayerWorkspace",
    "HEAD_DIM",
    "KAPPA",
    "MutableGraphState",
    "OnlineUpdateWorkspace",
    "PackedSegments",
    "PrefillCSR",
    "SegmentedAttentionWorkspace",
    "choose_splits",
]

"""Batched decode: many sequences of one layer in a single launch.

The reference decodes one sequence at a time (``community_kv/runtime.py:358``
rejects any other batch size).  Every (sequence, retrieval head) pair is
independent, so this module stacks the per-sequence state tensors along a
leading, contiguous batch axis - the layout ``ckv_decode_layer`` consumes - and
runs all of them with one library call per layer.  ``sequence_view`` hands back
reference-shaped views of one slot.
"""

from __future__ import annotations

from dataclasses import dataclass, fields
from typing import Sequence

import torch

from community_kv_b200 import native, ops
from community_kv_b200.config import CommunityKVConfig
from community_kv_b200.runtime import ConvertedPrefillState, _effective_token_budget
from community_kv_b200.state import (
    HEAD_DIM,
    DecodeDeltaChunks,
    DecodeLayerWorkspace,
    MutableGraphState,
    PrefillCSR,
)


def _stack(tensors: Sequence[torch.Tensor], width: int | None = None, fill: float = 0) -> torch.Tensor:
    """Stack along a new axis 0, right-padding axis 1 of each tensor to ``width``."""

    if width is None:
        return torch.stack(list(tensors)).contiguous()
    first = tensors[0]
    shape = (len(tensors), first.shape[0], width) + tuple(first.shape[2:])
    out = torch.full(shape, fill, dtype=first.dtype, device=first.device)
    for index, tensor in enumerate(tensors):
        out[index, :, : tensor.shape[1]] = tensor
    return out


@dataclass(slots=True)
class BatchedLayerState:
    csr: PrefillCSR
    mutable: MutableGraphState
    current_position: torch.Tensor
    workspace: DecodeLayerWorkspace
    sink_positions: torch.Tensor
    batch: int
    group_size: int
    query_heads: int
    kv_heads: int
    token_budget: int
    args: native.LayerArgs | None = None
    cache_key: tuple | None = None
    update_done: object = None  # deferred update: event of the layer's last online assignment

    def sequence_view(self, index: int) -> tuple[PrefillCSR, MutableGraphState, torch.Tensor]:
        """Reference-shaped views (no copy) of one sequence slot."""

        def pick(obj, skip=()):
            return {
                item.name: getattr(obj, item.name)[index]
                for item in fields(obj)
                if item.name not in skip and isinstance(getattr(obj, item.name), torch.Tensor)
            }

        deltas = DecodeDeltaChunks(**pick(self.mutable.deltas))
        shared = ("retrieval_to_graph", "retrieval_to_kv", "deltas")
        mutable = MutableGraphState(
            **pick(self.mutable, skip=shared),
            deltas=deltas,
            retrieval_to_graph=self.mutable.retrieval_to_graph,
            retrieval_to_kv=self.mutable.retrieval_to_kv,
        )
        return PrefillCSR(**pick(self.csr)), mutable, self.current_position[index]


def stack_sequences(
    sequences: Sequence[ConvertedPrefillState],
    *,
    config: CommunityKVConfig,
    splits: int | None = None,
    max_communities: int = 0,
) -> BatchedLayerState:
    """Stack validated per-sequence states of one layer into batch-major tensors."""

    if not sequences:
        raise ValueError("at least one sequence is required")
    first = sequences[0]
    for other in sequences[1:]:
        same = (
            other.group_size == first.group_size
            and other.query_heads == first.query_heads
            and other.kv_heads == first.kv_heads
            and other.prefill_seq_len == first.prefill_seq_len
            and other.decode_capacity == first.decode_capacity
            and torch.equal(other.mutable.retrieval_to_graph, first.mutable.retrieval_to_graph)
            and torch.equal(other.mutable.retrieval_to_kv, first.mutable.retrieval_to_kv)
        )
        if not same:
            raise ValueError("batched sequences must share geometry, length and aggregation")
    batch = len(sequences)
    capacity = max(s.mutable.community_capacity for s in sequences)
    members = max(s.csr.member_positions.shape[1] for s in sequences)
    tokens = max(s.mutable.token_communities.shape[1] for s in sequences)
    device = first.mutable.centroids.device
    graphs = first.mutable.graph_count
    heads = first.mutable.retrieval_head_count

    offsets = torch.empty((batch, graphs, capacity + 1), dtype=torch.int32, device=device)
    for index, seq in enumerate(sequences):
        have = seq.csr.member_offsets.shape[1]
        offsets[index, :, :have] = seq.csr.member_offsets
        offsets[index, :, have:] = seq.csr.member_offsets[:, -1:]
    centroid_bytes = _stack([s.mutable.centroids.view(torch.uint8) for s in sequences], capacity)
    csr = PrefillCSR(
        member_offsets=offsets,
        member_positions=_stack([s.csr.member_positions for s in sequences], members),
        community_counts=_stack([s.csr.community_counts for s in sequences]),
    )
    mutable = MutableGraphState(
        centroids=centroid_bytes.view(torch.float8_e4m3fn),
        community_sizes=_stack([s.mutable.community_sizes for s in sequences], capacity),
        community_counts=_stack([s.mutable.community_counts for s in sequences]),
        community_weight=_stack([s.mutable.community_weight for s in sequences], capacity),
        total_weight=_stack([s.mutable.total_weight for s in sequences]),
        token_communities=_stack([s.mutable.token_communities for s in sequences], tokens, fill=-1),
        deltas=DecodeDeltaChunks.allocate(
            graph_count=graphs,
            community_capacity=capacity,
            max_decode_tokens=first.decode_capacity,
            device=device,
            batch=batch,
        ),
        retrieval_to_graph=first.mutable.retrieval_to_graph.contiguous(),
        retrieval_to_kv=first.mutable.retrieval_to_kv.contiguous(),
    )
    budget = _effective_token_budget(
        configured_budget=config.token_budget,
        prefill_seq_len=first.prefill_seq_len,
        num_sink=config.num_sink,
    )
    counts = [list(s.initial_community_counts) for s in sequences]
    workspace = DecodeLayerWorkspace.allocate(
        retrieval_head_count=heads,
        graph_count=graphs,
        group_size=first.group_size,
        community_capacity=capacity,
        token_budget=budget,
        num_sink=config.num_sink,
        dtype=torch.bfloat16,
        device=device,
        score_community_counts=counts,
        score_headroom=first.decode_capacity,
        batch=batch,
        splits=splits,
        max_communities=max_communities,
    )
    return BatchedLayerState(
        csr=csr,
        mutable=mutable,
        current_position=_stack([s.current_position for s in sequences]),
        workspace=workspace,
        sink_positions=torch.arange(config.num_sink, dtype=torch.int32, device=device),
        batch=batch,
        group_size=first.group_size,
        query_heads=first.query_heads,
        kv_heads=first.kv_heads,
        token_budget=budget,
    )


class BatchedDecodeRuntime:
    """Per-layer batched states; ``decode`` is one CUDA-library call per layer and step."""

    def __init__(self, config: CommunityKVConfig, *, splits: int | None = None,
                 defer_update: bool = False) -> None:
        self.config = config
        self.splits = splits
        self.defer_update = defer_update  # see ops.DeferredUpdate
        self._deferred: ops.DeferredUpdate | None = None
        self.layers: dict[int, BatchedLayerState] = {}

    def synchronize_updates(self) -> None:
        if self._deferred is not None:
            self._deferred.synchronize()

    def install(self, layer_idx: int, state: BatchedLayerState) -> BatchedLayerState:
        if layer_idx in self.layers:
            raise ValueError(f"layer {layer_idx} is already prepared")
        self.layers[layer_idx] = state
        return state

    def prepare_layer(
        self,
        layer_idx: int,
        sequences: Sequence[ConvertedPrefillState],
        *,
        max_communities: int = 0,
    ) -> BatchedLayerState:
        return self.install(
            layer_idx,
            stack_sequences(
                sequences, config=self.config, splits=self.splits, max_communities=max_communities
            ),
        )

    def pack(
        self,
        layer_idx: int,
        *,
        query: torch.Tensor,
        key: torch.Tensor,
        value: torch.Tensor,
        softmax_scale: float,
    ) -> native.LayerArgs:
        """Validated argument block for one layer (cached while K/V storage is unchanged)."""

        layer = self.layers.get(layer_idx)
        if layer is None:
            raise RuntimeError(f"decode layer {layer_idx} is not prepared")
        if query.shape != (layer.batch, layer.query_heads, HEAD_DIM):
            raise ValueError("batched decode requires query shape [B, Hq, 128]")
        if key.ndim != 4 or key.shape[0] != layer.batch or key.shape[1] != layer.kv_heads:
            raise ValueError("batched decode requires key/value shape [B, Hkv, S, 128]")
        cache_key = (key.data_ptr(), value.data_ptr(), *key.stride(), float(softmax_scale))
        if layer.args is None or layer.cache_key != cache_key:
            layer.args = ops.build_layer_args(
                query=query,
                key=key,
                value=value,
                csr=layer.csr,
                state=layer.mutable,
                sink_positions=layer.sink_positions,
                current_position=layer.current_position,
                softmax_scale=softmax_scale,
                lam=self.config.lam,
                workspace=layer.workspace,
            )
            layer.cache_key = cache_key
        layer.args.query = query.data_ptr()
        return layer.args

    def decode(
        self,
        *,
        layer_idx: int,
        query: torch.Tensor,
        key: torch.Tensor,
        value: torch.Tensor,
        softmax_scale: float,
    ) -> torch.Tensor:
        """``query [B, Hq, 128]``, ``key/value [B, Hkv, S, 128]`` -> ``[B, Hq, 128]`` bf16."""

        if not query.is_contiguous():
            query = query.contiguous()
        args = self.pack(layer_idx, query=query, key=key, value=value, softmax_scale=softmax_scale)
        if self.defer_update:
            if self._deferred is None:
                self._deferred = ops.DeferredUpdate(query.device)
            layer = self.layers[layer_idx]
            layer.update_done = self._deferred.launch(args, pending=layer.update_done)
        else:
            native.call("ckv_decode_layer", args, native.current_stream(query.device))
        return self.layers[layer_idx].workspace.attention.output

    def assert_no_overflow(self) -> None:
        self.synchronize_updates()
        failures = {}
        for layer_idx, layer in self.layers.items():
            if int(torch.count_nonzero(layer.workspace.update.overflow)):
                failures[layer_idx] = layer.workspace.update.overflow.cpu().tolist()
            if int(layer.workspace.attention.status[0]):
                failures[layer_idx] = f"device status {int(layer.workspace.attention.status[0])}"
        if failures:
            raise RuntimeError(f"decode state overflow: {failures}")


__all__ = ["BatchedDecodeRuntime", "BatchedLayerState", "stack_sequences"]

"""Sequence-sharded decode of one very long layer (one sequence, rows split across GPUs).

Graph state, centroids and labels are replicated, so every rank scores and
selects identically; each rank holds a contiguous slice of the K/V rows and
attends only to the selected rows it owns.  The ranks then exchange their
partial ``(max, sum, out)`` triples and their best neighbour candidates, merge
them with the log-sum-exp rule, and every rank applies the same online
assignment to its replica of the state (``ckv_online_update``), so the replicas
stay bit-identical without any further traffic.

The reference has no counterpart (it is single-GPU); semantics are those of the
unsharded layer transition.
"""

from __future__ import annotations

from typing import Sequence

import torch
import torch.distributed as dist

from community_kv_b200 import distributed as ckv_dist
from community_kv_b200 import native, ops
from community_kv_b200.config import CommunityKVConfig
from community_kv_b200.runtime import ConvertedPrefillState, _effective_token_budget
from community_kv_b200.state import HEAD_DIM, KAPPA, PARTIAL_STRIDE, DecodeLayerWorkspace

_SIGN = -(2**63)


def pack_candidates(scores: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
    """(score, position) -> the kernels' 64-bit keys (ordered score << 32 | ~position), 0 if empty."""

    bits = scores.contiguous().view(torch.int32).long() & 0xFFFFFFFF
    ordered = torch.where(bits >= 0x80000000, (~bits) & 0xFFFFFFFF, bits ^ 0x80000000)
    low = (0xFFFFFFFF - positions.long()) & 0xFFFFFFFF
    high = torch.where(ordered >= 0x80000000, ordered - (1 << 32), ordered)  # as signed upper half
    packed = (high << 32) | low
    return torch.where(positions >= 0, packed, torch.zeros_like(packed))


def unpack_candidates(packed: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    ordered = (packed >> 32) & 0xFFFFFFFF
    bits = torch.where(ordered >= 0x80000000, ordered ^ 0x80000000, (~ordered) & 0xFFFFFFFF)
    signed = torch.where(bits >= 0x80000000, bits - (1 << 32), bits).to(torch.int32)
    positions = (0xFFFFFFFF - (packed & 0xFFFFFFFF)).to(torch.int64)
    positions = torch.where(packed == 0, torch.full_like(positions, -1), positions)
    return signed.view(torch.float32), positions.to(torch.int32)


class SequenceShardedLayer:
    """This rank's share of one layer: replicated state, rows ``[row_begin, row_begin + rows)`` of K/V."""

    def __init__(
        self,
        *,
        converted: ConvertedPrefillState,
        key_shard: torch.Tensor,
        value_shard: torch.Tensor,
        row_begin: int,
        total_rows: int,
        config: CommunityKVConfig,
        splits: int | None = None,
    ) -> None:
        if key_shard.ndim != 3 or key_shard.shape != value_shard.shape or key_shard.shape[-1] != HEAD_DIM:
            raise ValueError("key/value shards must have shape [Hkv, local rows, 128]")
        if row_begin < 0 or row_begin + key_shard.shape[1] > total_rows:
            raise ValueError("the shard must lie inside the cache")
        mutable = converted.mutable
        device = mutable.centroids.device
        self.converted = converted
        self.config = config
        self.key = key_shard
        self.value = value_shard
        self.row_begin = row_begin
        self.total_rows = total_rows
        budget = _effective_token_budget(
            configured_budget=config.token_budget,
            prefill_seq_len=converted.prefill_seq_len,
            num_sink=config.num_sink,
        )
        self.workspace = DecodeLayerWorkspace.allocate(
            retrieval_head_count=mutable.retrieval_head_count,
            graph_count=mutable.graph_count,
            group_size=converted.group_size,
            community_capacity=mutable.community_capacity,
            token_budget=budget,
            num_sink=config.num_sink,
            dtype=torch.bfloat16,
            device=device,
            score_community_counts=converted.initial_community_counts,
            score_headroom=converted.decode_capacity,
            splits=splits,
        )
        self.sinks = torch.arange(config.num_sink, dtype=torch.int32, device=device)
        heads = mutable.retrieval_head_count
        self.merged = torch.zeros(
            (heads, converted.group_size, PARTIAL_STRIDE), dtype=torch.float32, device=device
        )

    # -- step 1: replicated scoring + selection, local attention partials ---------------------
    def partial(self, query: torch.Tensor, softmax_scale: float):
        """Returns ``(maxima [Hq], sums [Hq], accumulators [Hq, 128], packed candidates [R, 8])``."""

        conv, ws = self.converted, self.workspace
        state = conv.mutable
        segments = ops.score_and_select(
            query=query,
            centroids=state.centroids,
            community_sizes=state.community_sizes,
            community_counts=state.community_counts,
            workspace=ws.selection,
            csr=conv.csr,
            state=state,
            sink_positions=self.sinks,
            current_position=conv.current_position,
        )
        args = native.LayerArgs()
        ops._graph_args(
            args, csr=conv.csr, state=state, sink_positions=self.sinks,
            current_position=conv.current_position,
        )
        ops._attention_args(
            args, query=query, key=self.key, value=self.value, softmax_scale=softmax_scale,
            lam=self.config.lam, workspace=ws.attention, update=None, token_budget=segments.token_budget,
        )
        native.fill(
            args,
            device=query.device.index or 0,
            batch=1,
            num_sink=segments.num_sink,
            descriptor_capacity=segments.communities.shape[-1],
            communities=native.pointer(segments.communities),
            cumulative_ends=native.pointer(segments.cumulative_ends),
            descriptor_counts=native.pointer(segments.descriptor_counts),
            tile_descriptors=native.pointer(segments.tile_descriptors),
            positions=native.pointer(ws.selection.positions),
            kv_row_begin=self.row_begin,
            kv_row_count=self.key.shape[1],
            merged=native.pointer(self.merged),
        )
        native.call("ckv_segmented_attention", args, native.current_stream(query.device))
        flat = self.merged.view(-1, PARTIAL_STRIDE)
        packed = pack_candidates(ws.attention.topk_scores, ws.attention.topk_positions)
        return flat[:, HEAD_DIM], flat[:, HEAD_DIM + 1], flat[:, :HEAD_DIM], packed

    # -- step 2: every rank applies the same combined result to its replica --------------------
    def finish(
        self,
        output: torch.Tensor,
        lse: torch.Tensor,
        packed_topk: torch.Tensor,
        current_key: torch.Tensor,
        softmax_scale: float,
    ) -> torch.Tensor:
        conv, ws = self.converted, self.workspace
        state = conv.mutable
        attention = ws.attention
        attention.output.copy_(output.to(torch.bfloat16))
        attention.lse.copy_(lse)
        scores, positions = unpack_candidates(packed_topk)
        attention.topk_scores.copy_(scores)
        attention.topk_positions.copy_(positions)
        key_rows = current_key[state.retrieval_to_kv.long()].contiguous()  # [R, 128]
        args = native.LayerArgs()
        ops._graph_args(
            args, csr=conv.csr, state=state, sink_positions=self.sinks,
            current_position=conv.current_position,
        )
        native.fill(
            args,
            device=output.device.index or 0,
            batch=1,
            group_size=conv.group_size,
            token_budget=ws.selection.token_budget,
            num_sink=ws.selection.num_sink,
            sequence_capacity=self.total_rows,
            lam=float(self.config.lam),
            softmax_scale=float(softmax_scale),
            splits=1,
            lse=native.pointer(attention.lse),
            topk_scores=native.pointer(attention.topk_scores),
            topk_positions=native.pointer(attention.topk_positions),
            output=native.pointer(attention.output),
            partials=native.pointer(attention.partials),
            partial_topk=native.pointer(attention.partial_topk_packed),
            assigned=native.pointer(ws.update.assigned_communities),
            overflow=native.pointer(ws.update.overflow),
            current_key=native.pointer(key_rows),
        )
        native.call("ckv_online_update", args, native.current_stream(output.device))
        self._keep = key_rows  # the kernel reads it asynchronously
        return attention.output

    def decode(
        self,
        query: torch.Tensor,
        current_key: torch.Tensor,
        softmax_scale: float,
        group: dist.ProcessGroup | None = None,
    ) -> torch.Tensor:
        """One decode step across the ranks of ``group``; returns bf16 ``[Hq, 128]`` on every rank."""

        maxima, sums, accumulators, packed = self.partial(query, softmax_scale)
        output, lse = ckv_dist.combine_partials(maxima, sums, accumulators, group=group)
        world = dist.get_world_size(group)
        gathered = torch.empty((world,) + packed.shape, dtype=packed.dtype, device=packed.device)
        dist.all_gather_into_tensor(gathered.view(world * packed.shape[0], KAPPA), packed.contiguous(), group=group)
        return self.finish(output, lse, ckv_dist.merge_topk(gathered), current_key, softmax_scale)


def decode_emulated(
    shards: Sequence[SequenceShardedLayer],
    query: torch.Tensor,
    current_key: torch.Tensor,
    softmax_scale: float,
) -> torch.Tensor:
    """All shards in one process, one after the other (no collectives): for tests on one GPU."""

    pieces = [shard.partial(query, softmax_scale) for shard in shards]
    output, lse = ckv_dist.merge_partials(
        torch.stack([p[0] for p in pieces]), torch.stack([p[1] for p in pieces]),
        torch.stack([p[2] for p in pieces]),
    )
    top = ckv_dist.merge_topk(torch.stack([p[3] for p in pieces]))
    result = None
    for shard in shards:
        result = shard.finish(output, lse, top, current_key, softmax_scale)
    return result


__all__ = ["SequenceShardedLayer", "decode_emulated", "pack_candidates", "unpack_candidates"]

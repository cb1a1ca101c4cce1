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
    """This rank's share of one layer: replicated state, rows ``[row_begin, row_begin + rows)`` of K/V.

    A step is ``local`` (scoring, selection, attention over the rows held here, merged into
    one un-normalised ``(acc, max, sum)`` row per head plus this shard's eight best neighbour
    candidates, written straight into ``record``), ONE all-gather of the ranks' records, and
    ``finish`` (``ckv_merge_partials`` with one "split" per rank, reading the gathered records
    in place: log-sum-exp merge, global top-8, online update of this rank's replica).
    """

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
        # what one rank contributes to the exchange: [R, G, 132] floats, then [R, 8] packed candidates
        self.merged_floats = heads * converted.group_size * PARTIAL_STRIDE
        self.record_bytes = self.merged_floats * 4 + heads * KAPPA * 8
        self.record = torch.zeros((self.record_bytes,), dtype=torch.uint8, device=device)
        self.merged = self.record[: self.merged_floats * 4].view(torch.float32).view(
            heads, converted.group_size, PARTIAL_STRIDE)
        self.merged_topk = self.record[self.merged_floats * 4 :].view(torch.int64).view(heads, KAPPA)
        self._gathered: torch.Tensor | None = None
        kv_map = mutable.retrieval_to_kv.cpu()
        self._identity_kv = bool(torch.equal(kv_map, torch.arange(heads, dtype=kv_map.dtype)))
        self._kv_index = mutable.retrieval_to_kv.long()
        self._keep: torch.Tensor | None = None

    def _layer_args(self, query: torch.Tensor, softmax_scale: float, *, update: bool) -> native.LayerArgs:
        conv, ws = self.converted, self.workspace
        args = ops.build_layer_args(
            query=query, key=self.key, value=self.value, csr=conv.csr, state=conv.mutable,
            sink_positions=self.sinks, current_position=conv.current_position,
            softmax_scale=softmax_scale, lam=self.config.lam, workspace=ws,
        )
        native.fill(args, sequence_capacity=self.total_rows)
        if not update:
            args.flags |= native.FLAG_SKIP_UPDATE
        return args

    def _key_rows(self, current_key: torch.Tensor) -> torch.Tensor:
        """The new token's key per retrieval head ``[R, 128]`` (bf16, contiguous)."""

        rows = current_key if self._identity_kv else current_key[self._kv_index]
        rows = rows.contiguous()
        self._keep = rows  # the kernel reads it asynchronously
        return rows

    # -- step 1: replicated scoring + selection, attention over the local rows ----------------
    def local(self, query: torch.Tensor, softmax_scale: float) -> torch.Tensor:
        """Fills and returns ``record`` (uint8 ``[record_bytes]``): this shard's merged rows and candidates."""

        args = self._layer_args(query, softmax_scale, update=False)
        native.fill(
            args,
            kv_row_begin=self.row_begin,
            kv_row_count=self.key.shape[1],
            merged=native.pointer(self.merged),
            merged_topk=native.pointer(self.merged_topk),
        )
        native.call("ckv_decode_layer", args, native.current_stream(query.device))
        return self.record

    # -- step 2: every rank applies the same combined result to its replica --------------------
    def finish(
        self,
        query: torch.Tensor,
        gathered: torch.Tensor,
        current_key: torch.Tensor,
        softmax_scale: float,
    ) -> torch.Tensor:
        """``gathered`` uint8 ``[ranks, record_bytes]``: every rank's record, merged in place."""

        ranks = gathered.shape[0]
        if gathered.dtype != torch.uint8 or gathered.shape[1] != self.record_bytes or not gathered.is_contiguous():
            raise ValueError("gathered must be contiguous uint8 [ranks, record_bytes]")
        args = self._layer_args(query, softmax_scale, update=True)
        group = self.converted.group_size
        native.fill(
            args,
            splits=ranks,
            partials=gathered.data_ptr(),
            partial_unit_stride=group * PARTIAL_STRIDE,
            partial_split_stride=self.record_bytes // 4,
            partial_topk=gathered.data_ptr() + self.merged_floats * 4,
            topk_unit_stride=KAPPA,
            topk_split_stride=self.record_bytes // 8,
            current_key=native.pointer(self._key_rows(current_key)),
        )
        native.call("ckv_merge_partials", args, native.current_stream(query.device))
        return self.workspace.attention.output

    def decode(
        self,
        query: torch.Tensor,
        current_key: torch.Tensor,
        softmax_scale: float,
        group: dist.ProcessGroup | None = None,
    ) -> torch.Tensor:
        """One decode step across the ranks of ``group``; returns bf16 ``[Hq, 128]`` on every rank."""

        world = dist.get_world_size(group) if dist.is_initialized() else 1
        if world == 1 and self.row_begin == 0 and self.key.shape[1] == self.total_rows:
            return self.decode_whole(query, current_key, softmax_scale)
        record = self.local(query, softmax_scale)
        if self._gathered is None or self._gathered.shape[0] != world:
            self._gathered = torch.empty((world, self.record_bytes), dtype=torch.uint8, device=record.device)
        dist.all_gather_into_tensor(self._gathered.view(-1), record, group=group)
        return self.finish(query, self._gathered, current_key, softmax_scale)

    def decode_whole(self, query: torch.Tensor, current_key: torch.Tensor, softmax_scale: float) -> torch.Tensor:
        """The whole cache is local: one ``ckv_decode_layer`` call, nothing to exchange."""

        args = self._layer_args(query, softmax_scale, update=True)
        native.fill(args, current_key=native.pointer(self._key_rows(current_key)))
        native.call("ckv_decode_layer", args, native.current_stream(query.device))
        return self.workspace.attention.output


def decode_emulated(
    shards: Sequence[SequenceShardedLayer],
    query: torch.Tensor,
    current_key: torch.Tensor,
    softmax_scale: float,
) -> torch.Tensor:
    """All shards in one process, one after the other (no collectives): for tests on one GPU."""

    gathered = torch.stack([shard.local(query, softmax_scale) for shard in shards])
    result = None
    for shard in shards:
        result = shard.finish(query, gathered, current_key, softmax_scale)
    return result


__all__ = ["SequenceShardedLayer", "decode_emulated", "pack_candidates", "unpack_candidates"]

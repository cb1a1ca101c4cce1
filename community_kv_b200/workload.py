"""Device-side builder of multi-layer, batched synthetic decode workloads.

Builds the long-context benchmark shapes directly on the GPU: per (layer,
sequence, KV head) a random community assignment with Zipf-distributed sizes
over the whole context, Gaussian K/V rows, mean-key e4m3 centroids and the
recency-descending member lists, stacked into the batch-major state the CUDA
library consumes.  Every draw is keyed by (seed, layer, sequence, global KV
head), so a KV-head shard of the workload holds exactly the rows the unsharded
workload holds for those heads.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from community_kv_b200.assembly import assemble_layer
from community_kv_b200.batched import BatchedDecodeRuntime, BatchedLayerState, stack_sequences
from community_kv_b200.config import CommunityKVConfig, GraphAggregation
from community_kv_b200.runtime import convert_prefill_tensors

HEAD_DIM = 128


@dataclass(slots=True)
class DecodeWorkload:
    config: CommunityKVConfig
    runtime: BatchedDecodeRuntime
    key: torch.Tensor    # [launches, slots, Hkv_local, rows, 128] bf16
    value: torch.Tensor
    layers: int
    batch: int
    kv_heads: int        # heads held by this process
    group_size: int
    seq_len: int
    max_decode_tokens: int
    layers_per_launch: int
    community_counts: list[int]  # initial active communities per unit, flattened

    @property
    def launches(self) -> int:
        return self.layers // self.layers_per_launch

    @property
    def slots(self) -> int:
        return self.batch * self.layers_per_launch

    def state(self, launch: int) -> BatchedLayerState:
        return self.runtime.layers[launch]


def _unit_generator(seed: int, layer: int, sequence: int, head: int, device: torch.device) -> torch.Generator:
    generator = torch.Generator(device=device)
    generator.manual_seed((seed * 1_000_003 + layer * 10_007 + sequence * 101 + head) & 0x7FFFFFFF)
    return generator


def _zipf_labels(
    tokens: int, communities: int, exponent: float, generator: torch.Generator, device: torch.device
) -> torch.Tensor:
    rank = torch.arange(1, communities + 1, dtype=torch.float64, device=device)
    share = rank.pow(-exponent)
    share = share / share.sum()
    sizes = torch.floor(share * (tokens - communities)).long() + 1
    sizes[0] += tokens - int(sizes.sum())
    ids = torch.randperm(communities, generator=generator, device=device)
    labels = torch.repeat_interleave(ids, sizes)
    return labels[torch.randperm(tokens, generator=generator, device=device)]


def build_decode_workload(
    *,
    layers: int,
    batch: int,
    kv_heads: int,
    group_size: int = 4,
    seq_len: int,
    communities: tuple[int, int],
    token_budget: int,
    num_sink: int = 10,
    max_decode_tokens: int,
    device: torch.device,
    seed: int = 0,
    zipf_exponent: float = 1.1,
    head_offset: int = 0,
    sequence_offset: int = 0,
    layers_per_launch: int = 1,
    splits: int | None = None,
    lam: float = 0.5,
) -> DecodeWorkload:
    """Random-label, Zipf-sized communities per (layer, sequence, KV head) on ``device``."""

    if layers % layers_per_launch:
        raise ValueError("layers_per_launch must divide layers")
    config = CommunityKVConfig(
        token_budget=token_budget, num_sink=num_sink, lam=lam, aggregation=GraphAggregation.QUERY_GROUP
    )
    rows = seq_len + max_decode_tokens + 1
    launches = layers // layers_per_launch
    slots = batch * layers_per_launch
    key = torch.empty((launches, slots, kv_heads, rows, HEAD_DIM), dtype=torch.bfloat16, device=device)
    value = torch.empty_like(key)
    runtime = BatchedDecodeRuntime(config, splits=splits)
    host = torch.Generator().manual_seed(seed)
    low, high = communities
    counts: list[int] = []
    for launch in range(launches):
        sequences = []
        for slot in range(slots):
            layer = launch * layers_per_launch + slot // batch
            sequence = sequence_offset + slot % batch
            labels = torch.zeros((kv_heads, seq_len), dtype=torch.int32, device=device)
            for head in range(kv_heads):
                generator = _unit_generator(seed, layer, sequence, head_offset + head, device)
                # community count per unit: keyed like the data so that shards agree
                pick = torch.Generator().manual_seed(int(generator.initial_seed()))
                count = int(torch.randint(low, high + 1, (1,), generator=pick))
                counts.append(count)
                labels[head, num_sink:] = _zipf_labels(
                    seq_len - num_sink, count, zipf_exponent, generator, device
                ).to(torch.int32)
                key[launch, slot, head].normal_(generator=generator)
                value[launch, slot, head].normal_(generator=generator)
            key[launch, slot].mul_(HEAD_DIM**-0.5)
            value[launch, slot].mul_(HEAD_DIM**-0.5)
            assembled = assemble_layer(
                labels,
                key[launch, slot, :, :seq_len],
                aggregation=GraphAggregation.QUERY_GROUP,
                query_heads=kv_heads * group_size,
                num_sink=num_sink,
                max_decode_tokens=max_decode_tokens,
            )
            sequences.append(
                convert_prefill_tensors(
                    member_offsets=assembled.member_offsets,
                    member_positions=assembled.member_positions,
                    num_communities=assembled.num_communities,
                    centroids=assembled.centroids,
                    community_sizes=assembled.community_sizes,
                    community_weight=assembled.community_weight,
                    total_weight=assembled.total_weight,
                    token_communities=assembled.token_communities,
                    retrieval_to_graph=assembled.retrieval_to_graph,
                    retrieval_to_kv=assembled.retrieval_to_kv,
                    prefill_seq_len=seq_len,
                    max_decode_tokens=max_decode_tokens,
                    group_size=group_size,
                    aggregation=GraphAggregation.QUERY_GROUP,
                    query_heads=kv_heads * group_size,
                    kv_heads=kv_heads,
                )
            )
            del assembled, labels
        runtime.install(launch, stack_sequences(sequences, config=config, splits=splits))
        del sequences
    del host
    return DecodeWorkload(
        config=config,
        runtime=runtime,
        key=key,
        value=value,
        layers=layers,
        batch=batch,
        kv_heads=kv_heads,
        group_size=group_size,
        seq_len=seq_len,
        max_decode_tokens=max_decode_tokens,
        layers_per_launch=layers_per_launch,
        community_counts=counts,
    )


def build_planted_layer(
    *,
    seq_len: int,
    clusters: int,
    kv_heads: int,
    group_size: int,
    num_sink: int,
    max_decode_tokens: int,
    device: torch.device,
    seed: int = 0,
    noise: float = 0.3,
):
    """One single-sequence layer with planted key clusters, built on ``device``.

    Keys are cluster centres ~N(0, 1) plus ``noise``-scaled Gaussian noise, times
    ``1/sqrt(128)``; the community of a token is its cluster (per KV head), sinks are
    isolated.  Returns ``(converted state, key [Hkv, rows, 128], value)`` with
    ``rows = seq_len + max_decode_tokens + 1``.  Every rank of a sequence-sharded
    run builds the same layer from the same seed and keeps its slice of the rows.
    """

    rows = seq_len + max_decode_tokens + 1
    key = torch.empty((kv_heads, rows, HEAD_DIM), dtype=torch.bfloat16, device=device)
    value = torch.empty_like(key)
    labels = torch.zeros((kv_heads, seq_len), dtype=torch.int32, device=device)
    for head in range(kv_heads):
        generator = _unit_generator(seed, 0, 0, head, device)
        centres = torch.randn((clusters, HEAD_DIM), generator=generator, device=device)
        cluster = torch.randint(0, clusters, (rows,), generator=generator, device=device)
        cluster[:clusters] = torch.randperm(clusters, generator=generator, device=device)  # none empty
        for begin in range(0, rows, 1 << 18):  # bounded temporaries
            end = min(rows, begin + (1 << 18))
            chunk = centres[cluster[begin:end]]
            chunk += noise * torch.randn(chunk.shape, generator=generator, device=device)
            key[head, begin:end] = (chunk * HEAD_DIM**-0.5).to(torch.bfloat16)
            value[head, begin:end] = (
                torch.randn(chunk.shape, generator=generator, device=device) * HEAD_DIM**-0.5
            ).to(torch.bfloat16)
        # sinks carry labels of their own behind the planted ones
        labels[head, num_sink:] = cluster[num_sink:seq_len].to(torch.int32)
        labels[head, :num_sink] = clusters + torch.arange(num_sink, dtype=torch.int32, device=device)
    assembled = assemble_layer(
        labels,
        key[:, :seq_len],
        aggregation=GraphAggregation.QUERY_GROUP,
        query_heads=kv_heads * group_size,
        num_sink=num_sink,
        max_decode_tokens=max_decode_tokens,
    )
    converted = convert_prefill_tensors(
        member_offsets=assembled.member_offsets,
        member_positions=assembled.member_positions,
        num_communities=assembled.num_communities,
        centroids=assembled.centroids,
        community_sizes=assembled.community_sizes,
        community_weight=assembled.community_weight,
        total_weight=assembled.total_weight,
        token_communities=assembled.token_communities,
        retrieval_to_graph=assembled.retrieval_to_graph,
        retrieval_to_kv=assembled.retrieval_to_kv,
        prefill_seq_len=seq_len,
        max_decode_tokens=max_decode_tokens,
        group_size=group_size,
        aggregation=GraphAggregation.QUERY_GROUP,
        query_heads=kv_heads * group_size,
        kv_heads=kv_heads,
    )
    return converted, key, value


__all__ = ["DecodeWorkload", "build_decode_workload", "build_planted_layer"]

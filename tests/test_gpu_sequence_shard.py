"""Sequence-sharded decoding: four row shards emulated on one GPU against the unsharded oracle."""

from __future__ import annotations

import pytest
import torch

from community_kv_b200 import distributed as ckv_dist
from community_kv_b200.config import CommunityKVConfig
from community_kv_b200.runtime import convert_prefill_tensors
from community_kv_b200.sequence_shard import SequenceShardedLayer, decode_emulated
from community_kv_b200.synthetic import make_layer, make_query
from tests.helpers import OUTPUT_MAX_ABS, OUTPUT_MEAN_ABS, OracleLayer, assert_state_equal

pytestmark = pytest.mark.gpu
SCALE = 128 ** -0.5


@pytest.mark.parametrize("aggregation", ["query_group", "layer_wise"])
def test_four_shards_match_the_unsharded_layer(aggregation):
    device = torch.device("cuda", 0)
    shards_n, steps = 4, 5
    config = CommunityKVConfig(token_budget=1024, num_sink=10, lam=0.5, aggregation=aggregation)
    layer = make_layer(seed=60, kv_heads=2, seq_len=16384, communities=512, max_decode_tokens=steps + 1,
                       aggregation=aggregation)
    total_rows = layer.key.shape[1]
    shards = []
    for rank in range(shards_n):
        begin, end = ckv_dist.sequence_shard(total_rows, shards_n, rank)
        replica = convert_prefill_tensors(**layer.to(device).prepare_kwargs())
        shards.append(
            SequenceShardedLayer(
                converted=replica,
                key_shard=layer.key[:, begin:end].contiguous().to(device),
                value_shard=layer.value[:, begin:end].contiguous().to(device),
                row_begin=begin,
                total_rows=total_rows,
                config=config,
                splits=4,
            )
        )
    first = shards[0].converted
    capacity = first.mutable.community_capacity
    twin = OracleLayer(
        first.csr, first.mutable, first.current_position, token_budget=1024, num_sink=10,
        cover=[min(capacity, c + first.decode_capacity) for c in first.initial_community_counts],
    )
    for step in range(steps):
        query = make_query(seed=1000 + step, query_heads=8)
        current = int(twin.current[0])
        out = decode_emulated(shards, query.to(device), layer.key[:, current].to(device), SCALE)
        want = twin.step(query=query, key=layer.key, value=layer.value, softmax_scale=SCALE, lam=0.5,
                         device_scores=shards[0].workspace.selection.scores)
        diff = (out.float().cpu() - want.output.float()).abs()
        assert float(diff.max()) <= OUTPUT_MAX_ABS and float(diff.mean()) <= OUTPUT_MEAN_ABS, step
        for rank, shard in enumerate(shards):
            where = f"step {step} shard {rank}"
            attention = shard.workspace.attention
            assert torch.equal(attention.topk_positions.cpu(), want.topk_positions), where
            assert torch.equal(attention.topk_scores.cpu().view(torch.int32), want.topk_scores.view(torch.int32)), where
            torch.testing.assert_close(attention.lse.cpu(), want.lse, rtol=0, atol=2e-3)
            assert torch.equal(shard.workspace.selection.positions.cpu(), want.positions), where
            assert torch.equal(shard.workspace.update.assigned_communities.cpu(), want.assigned), where
            assert_state_equal(shard.converted.mutable, twin.state, where)
            assert torch.equal(shard.converted.current_position.cpu(), twin.current), where


def test_large_context_shards_agree_with_one_gpu():
    """The sequence-sharded stress configuration (scaled to 262144 tokens so that two replicas fit comfortably):
    16384 planted clusters per head, budget 8192.  Two row shards against the whole cache in one
    piece: same selection, same neighbours and labels bit for bit, outputs within 2e-2."""

    import copy

    from community_kv_b200.workload import build_planted_layer

    device = torch.device("cuda", 0)
    steps = 3
    config = CommunityKVConfig(token_budget=8192, num_sink=10, lam=0.5, aggregation="query_group")
    converted, key, value = build_planted_layer(
        seq_len=262144, clusters=16384, kv_heads=8, group_size=4, num_sink=10,
        max_decode_tokens=steps + 2, device=device, seed=3,
    )
    total_rows = key.shape[1]
    whole = SequenceShardedLayer(converted=copy.deepcopy(converted), key_shard=key, value_shard=value,
                                 row_begin=0, total_rows=total_rows, config=config)
    shards = []
    for rank in range(2):
        begin, end = ckv_dist.sequence_shard(total_rows, 2, rank)
        shards.append(SequenceShardedLayer(
            converted=copy.deepcopy(converted), key_shard=key[:, begin:end].contiguous(),
            value_shard=value[:, begin:end].contiguous(), row_begin=begin, total_rows=total_rows, config=config))
    generator = torch.Generator(device=device).manual_seed(11)
    for step in range(steps):
        query = torch.randn((32, 128), generator=generator, device=device).to(torch.bfloat16)
        new_key = (torch.randn((8, 128), generator=generator, device=device) * SCALE).to(torch.bfloat16)
        one = decode_emulated([whole], query, new_key, SCALE).float().clone()
        two = decode_emulated(shards, query, new_key, SCALE).float()
        diff = (one - two).abs()
        assert float(diff.max()) <= OUTPUT_MAX_ABS and float(diff.mean()) <= OUTPUT_MEAN_ABS, step
        for shard in shards:
            assert torch.equal(shard.workspace.selection.positions, whole.workspace.selection.positions), step
            assert torch.equal(shard.workspace.attention.topk_positions, whole.workspace.attention.topk_positions), step
            assert torch.equal(shard.workspace.update.assigned_communities, whole.workspace.update.assigned_communities), step
            assert torch.equal(shard.converted.mutable.centroids.view(torch.uint8),
                               whole.converted.mutable.centroids.view(torch.uint8)), step
        assert int(whole.workspace.update.overflow.max()) == 0

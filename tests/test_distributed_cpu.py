"""Multi-rank host logic on CPU: two gloo ranks, no GPU."""

from __future__ import annotations

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from community_kv_b200 import distributed as ckv_dist
from oracle import decode_oracle as oracle


def _free_port() -> int:
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def _worker(rank: int, world: int, port: int, results) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        generator = torch.Generator().manual_seed(7)
        # ---- KV-head sharding: the gathered tensor is in head order ----
        full = torch.randn((3, 32, 128), generator=generator)
        heads = ckv_dist.head_shard(8, world, rank)
        mine = full[:, heads.start * 4 : heads.stop * 4]
        gathered = ckv_dist.gather_head_outputs(mine)
        assert torch.equal(gathered, full)

        # ---- sequence sharding: partial softmax triples combine to the dense result ----
        tokens, group = 512, 4
        q = torch.randn((group, 128), generator=generator)
        k = torch.randn((tokens, 128), generator=generator) / 11.3
        v = torch.randn((tokens, 128), generator=generator) / 11.3
        positions = torch.randperm(4096, generator=generator)[:tokens]
        begin, end = ckv_dist.sequence_shard(4096, world, rank)
        local = ckv_dist.localize_positions(positions, begin, end)
        owned = local >= 0
        assert int(owned.sum()) > 0 and bool(((local < end - begin)).all())
        scores = (q @ k.T) * 0.088
        scores = torch.where(owned.unsqueeze(0), scores, torch.full_like(scores, float("-inf")))
        top = scores.amax(dim=1)
        weights = torch.exp(scores - top.unsqueeze(1))
        output, lse = ckv_dist.combine_partials(top, weights.sum(dim=1), weights @ v)
        dense = (q @ k.T) * 0.088
        want = torch.softmax(dense, dim=1) @ v
        torch.testing.assert_close(output, want, atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(lse, torch.logsumexp(dense, dim=1), atol=1e-5, rtol=1e-5)

        # ---- neighbour candidates: global top-8 of per-rank packed keys ----
        rep = dense[0].numpy().astype(np.float32)
        pos = positions.numpy().astype(np.int32)
        mask = owned.numpy()
        local_scores, local_positions = oracle.global_topk(rep, np.where(mask, pos, -1), np.zeros(tokens, bool))
        keys = (oracle.ordered_f32_bits(local_scores).astype(np.uint64) << np.uint64(32)) | (
            np.uint64(0xFFFFFFFF) - local_positions.astype(np.int64).astype(np.uint64)
        )
        mine_packed = torch.from_numpy(keys.view(np.int64).copy()).reshape(1, 8)
        everyone = [torch.empty_like(mine_packed) for _ in range(world)]
        dist.all_gather(everyone, mine_packed)
        merged = ckv_dist.merge_topk(torch.stack(everyone))[0].numpy().view(np.uint64)
        want_scores, want_positions = oracle.global_topk(rep, pos, np.zeros(tokens, bool))
        got_positions = (np.uint64(0xFFFFFFFF) - (merged & np.uint64(0xFFFFFFFF))).astype(np.int64)
        assert got_positions.tolist() == want_positions.tolist()
        results.put((rank, "ok"))
    except BaseException as error:  # report instead of hanging the peer
        results.put((rank, repr(error)))
        raise
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_head_gather_and_partial_combine():
    world = 2
    context = mp.get_context("spawn")
    results = context.Queue()
    port = _free_port()
    workers = [context.Process(target=_worker, args=(rank, world, port, results)) for rank in range(world)]
    for worker in workers:
        worker.start()
    for worker in workers:
        worker.join(timeout=120)
    outcomes = dict(results.get(timeout=5) for _ in range(world))
    assert outcomes == {0: "ok", 1: "ok"}, outcomes
    assert all(worker.exitcode == 0 for worker in workers)


def test_shard_helpers():
    assert list(ckv_dist.head_shard(8, 4, 3)) == [6, 7]
    with pytest.raises(ValueError):
        ckv_dist.head_shard(8, 3, 0)
    assert ckv_dist.sequence_shard(10, 4, 3) == (9, 10)
    assert ckv_dist.sequence_shard(1 << 20, 8, 2) == (262144, 393216)
    local = ckv_dist.localize_positions(torch.tensor([0, 5, 9, -1, 12]), 5, 10)
    assert local.tolist() == [-1, 0, 4, -1, -1]
    empty = ckv_dist.merge_partials(
        torch.tensor([[float("-inf")], [1.0]]), torch.tensor([[0.0], [2.0]]),
        torch.tensor([[[0.0, 0.0]], [[4.0, 6.0]]]),
    )
    assert empty[0].tolist() == [[2.0, 3.0]]

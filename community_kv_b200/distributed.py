"""Multi-GPU decomposition of the decode path: one process per GPU, NCCL for the exchange.

The reference has no multi-GPU decode (its only cross-device traffic is
``Tensor.to`` inside the partition workers, ``community_kv/graph/runtime.py:121-158``).
Two decompositions follow from the independence of (sequence, layer, head) units:

* **KV-head sharding** for whole-model decode: rank ``p`` of ``N`` owns KV heads
  ``p*H/N .. (p+1)*H/N - 1`` with their cache slices, graph state and query
  group; selection and the online update need no exchange at all, the head
  outputs are all-gathered once per layer.
* **Sequence sharding** for very long single-layer contexts: every rank scores
  and selects identically (centroids and labels are replicated) but holds only
  a contiguous slice of the K/V rows; it attends to the selected rows it owns
  and the ranks combine their partial ``(max, sum, out)`` triples with the
  log-sum-exp rule.

Everything above is plain ``torch.distributed`` on tensors, so the logic also
runs on CPU with the ``gloo`` backend (that is how it is tested without GPUs).

``PeerOutputExchange`` replaces the per-layer all-gather of head outputs by stores
from inside the decode kernel: every rank's gathered tensor lives in symmetric
memory, the merging CTA of each unit writes its output rows into every peer's
tensor over NVLink and bumps a per-layer counter there, and the consumer waits
for the counter (``ckv_wait_peers``) instead of running a collective.
"""

from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from community_kv_b200 import native


def head_shard(kv_heads: int, world: int, rank: int) -> range:
    """KV heads owned by ``rank``: a contiguous block of ``kv_heads / world``."""

    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank must be in [0, world)")
    if kv_heads % world:
        raise ValueError("the number of ranks must divide the number of KV heads")
    per_rank = kv_heads // world
    return range(rank * per_rank, (rank + 1) * per_rank)


def gather_head_outputs(
    local: torch.Tensor,
    *,
    group: dist.ProcessGroup | None = None,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """All-gather ``local [B, Hq/N, D]`` into ``[B, Hq, D]`` in rank (= head) order."""

    world = dist.get_world_size(group)
    batch, heads, dim = local.shape
    staged = (
        out
        if out is not None
        else torch.empty((world, batch, heads, dim), dtype=local.dtype, device=local.device)
    )
    if staged.shape != (world, batch, heads, dim):
        raise ValueError("out must have shape [world, B, Hq/N, D]")
    dist.all_gather_into_tensor(staged.view(world * batch, heads, dim), local.contiguous(), group=group)
    return staged.permute(1, 0, 2, 3).reshape(batch, world * heads, dim)


def sequence_shard(length: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous ``[begin, end)`` slice of the sequence held by ``rank``."""

    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank must be in [0, world)")
    per_rank = -(-length // world)
    return min(length, rank * per_rank), min(length, (rank + 1) * per_rank)


def localize_positions(positions: torch.Tensor, begin: int, end: int) -> torch.Tensor:
    """Map global cache rows to rows of this rank's slice; rows it does not hold become -1."""

    owned = (positions >= begin) & (positions < end)
    return torch.where(owned, positions - begin, torch.full_like(positions, -1))


def combine_partials(
    maxima: torch.Tensor,
    sums: torch.Tensor,
    accumulators: torch.Tensor,
    *,
    group: dist.ProcessGroup | None = None,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Exchange per-rank softmax partials and merge them.

    ``maxima [H]``, ``sums [H]``, ``accumulators [H, D]`` (fp32, the accumulator
    is not normalised).  One all-gather of the packed ``[H, D + 2]`` block per
    rank; every rank then computes the same ``(output fp32 [H, D], lse [H])``.
    A rank that holds none of the selected rows contributes ``max = -inf``.
    """

    world = dist.get_world_size(group)
    packed = torch.cat((accumulators, maxima.unsqueeze(-1), sums.unsqueeze(-1)), dim=-1).contiguous()
    gathered = torch.empty((world,) + packed.shape, dtype=packed.dtype, device=packed.device)
    dist.all_gather_into_tensor(gathered.view((world * packed.shape[0],) + packed.shape[1:]), packed, group=group)
    return merge_partials(gathered[..., -2], gathered[..., -1], gathered[..., :-2])


def merge_partials(
    maxima: torch.Tensor, sums: torch.Tensor, accumulators: torch.Tensor
) -> tuple[torch.Tensor, torch.Tensor]:
    """Log-sum-exp merge over the leading axis of stacked partials."""

    top = maxima.amax(dim=0)
    safe = torch.where(torch.isfinite(top), top, torch.zeros_like(top))
    weight = torch.exp(maxima - safe)
    weight = torch.where(torch.isfinite(maxima), weight, torch.zeros_like(weight))
    denominator = (sums * weight).sum(dim=0)
    output = (accumulators * weight.unsqueeze(-1)).sum(dim=0) / denominator.unsqueeze(-1)
    return output, top + torch.log(denominator)


def merge_topk(packed: torch.Tensor, k: int = 8) -> torch.Tensor:
    """Global top-``k`` of per-rank packed (ordered score << 32 | ~position) candidates.

    ``packed int64 [ranks, H, k]`` holding unsigned 64-bit keys; returns
    ``int64 [H, k]`` in descending unsigned order.  Ties cannot occur between
    ranks because a position lives on exactly one rank.
    """

    ranks, heads, width = packed.shape
    flat = packed.permute(1, 0, 2).reshape(heads, ranks * width)
    # order as unsigned: flip the sign bit, sort signed, flip back
    # (a Python scalar operand, not a tensor built on the host: the step stays capturable)
    flipped = torch.bitwise_xor(flat, -(2**63))
    top = torch.sort(flipped, dim=1, descending=True).values[:, :k]
    return torch.bitwise_xor(top, -(2**63))


__all__ = [
    "combine_partials",
    "gather_head_outputs",
    "head_shard",
    "localize_positions",
    "merge_partials",
    "merge_topk",
    "sequence_shard",
]


class PeerOutputExchange:
    """Head outputs of all ranks, written by the decode kernels themselves.

    ``gathered[launch, rank]`` (shape ``[slots, heads_local * G, 128]`` each) is this
    rank's copy of everybody's outputs of one launch.  ``attach`` points a launch's
    ``ckv_layer_args`` at the peers' slots and counters; ``wait`` enqueues the
    bounded wait for the peers' rows of that launch.  No NVLink multicast object is
    created (plain peer mappings only).

    There is no acknowledgement back to the writer: a peer may store the rows of step
    t + 1 into ``gathered[launch]`` as soon as it has received this rank's rows of step
    t for that launch.  With two or more launches per step, stream order on every rank
    keeps a launch's rows intact until the rank's own next launch has been enqueued
    behind its consumer; a step made of a single launch has no such slack, so the
    constructor refuses ``launches < 2`` (use the collective, ``gather_head_outputs``,
    there).  A consumer that reads ``gathered`` outside the stream (a host copy, another
    stream) must finish before it enqueues the next step.  After a wait has timed out
    (``check`` raises) the counters are out of step with the peers for good: the
    exchange must be rebuilt, not reused.
    """

    def __init__(self, *, launches: int, slots: int, heads: int, head_dim: int, units: int,
                 device: torch.device, group: dist.ProcessGroup | None = None) -> None:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world - 1 > native.MAX_PEERS:
            raise ValueError("at most %d peers" % native.MAX_PEERS)
        if launches < 2:
            raise ValueError("the peer exchange needs at least two launches per step (no back-pressure)")
        self.units = units
        self.gathered = symm_mem.empty(
            (launches, self.world, slots, heads, head_dim), dtype=torch.bfloat16, device=device
        )
        self.flags = symm_mem.empty((max(launches, 4),), dtype=torch.int32, device=device)
        self.gathered.zero_()
        self.flags.zero_()
        self.status = torch.zeros((1,), dtype=torch.int32, device=device)
        self.done = torch.zeros((max(launches, 4),), dtype=torch.int32, device=device)  # local unit counters
        torch.cuda.synchronize(device)
        outputs = symm_mem.rendezvous(self.gathered, group)
        counters = symm_mem.rendezvous(self.flags, group)
        self._output_ptrs = [int(p) for p in outputs.buffer_ptrs]
        self._flag_ptrs = [int(p) for p in counters.buffer_ptrs]
        self._slot_bytes = slots * heads * head_dim * 2
        dist.barrier(group)

    def local_output(self, launch: int) -> torch.Tensor:
        """Where this rank's own kernels write: its slot of its own gathered tensor."""

        return self.gathered[launch, self.rank]

    def attach(self, args: "native.LayerArgs", launch: int, *, wait_in_kernel: bool = True) -> None:
        """Point ``args`` at the peers.  With ``wait_in_kernel`` the launch itself ends
        only when the peers' rows of this launch have arrived (no ``wait`` needed)."""

        peers = [p for p in range(self.world) if p != self.rank]
        args.peer_done = self.done.data_ptr() + 4 * launch
        if wait_in_kernel:
            args.peer_wait_flag = self.flags.data_ptr() + 4 * launch
            args.peer_wait_expected = self.world - 1
            args.status = self.status.data_ptr()
        args.peer_count = len(peers)
        for index, peer in enumerate(peers):
            args.peer_output[index] = self._output_ptrs[peer] + (launch * self.world + self.rank) * self._slot_bytes
            args.peer_flag[index] = self._flag_ptrs[peer] + 4 * launch

    def wait(self, launch: int, stream: int) -> None:
        """Enqueue the wait for the peers' rows of ``launch`` (bounded; see ``check``)."""

        status = native.library().ckv_wait_peers(
            ctypes.c_void_p(self.flags.data_ptr() + 4 * launch),
            ctypes.c_uint32(self.world - 1),
            ctypes.c_void_p(self.status.data_ptr()),
            ctypes.c_void_p(stream),
        )
        if status:
            raise native.NativeError(native.library().ckv_status_string(status).decode())

    def check(self) -> None:
        """Raise if any wait gave up (a peer never delivered its rows)."""

        if int(self.status.item()) != 0:
            raise RuntimeError("a bounded wait for peer head outputs timed out")

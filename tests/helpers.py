"""Shared helpers for the parity tests: CPU clones of the state and field-by-field comparison."""

from __future__ import annotations

from dataclasses import fields

import numpy as np
import torch

from community_kv_b200 import ops
from community_kv_b200.state import DecodeDeltaChunks, MutableGraphState, PrefillCSR
from oracle import decode_oracle as oracle

OUTPUT_MAX_ABS = 2e-2   # bf16 attention output, the tolerance the task states
OUTPUT_MEAN_ABS = 1e-3
WEIGHT_RTOL = 2e-5      # fp32 modularity weights (device exp vs libm exp)


def cpu_clone(csr: PrefillCSR, mutable: MutableGraphState, current: torch.Tensor):
    deltas = DecodeDeltaChunks(
        **{f.name: getattr(mutable.deltas, f.name).detach().cpu().clone() for f in fields(mutable.deltas)}
    )
    state = MutableGraphState(
        **{
            f.name: getattr(mutable, f.name).detach().cpu().clone()
            for f in fields(mutable)
            if f.name != "deltas"
        },
        deltas=deltas,
    )
    csr_c = PrefillCSR(**{f.name: getattr(csr, f.name).detach().cpu().clone() for f in fields(csr)})
    return csr_c, state, current.detach().cpu().clone()


def assert_state_equal(device_state: MutableGraphState, cpu_state: MutableGraphState, where: str = "") -> None:
    for f in fields(cpu_state):
        if f.name == "deltas":
            continue
        got = getattr(device_state, f.name).detach().cpu()
        want = getattr(cpu_state, f.name)
        if got.dtype == torch.float8_e4m3fn:
            assert torch.equal(got.view(torch.uint8), want.view(torch.uint8)), f"{where} {f.name}"
        elif got.dtype == torch.float32 and f.name == "centroids":  # the fp32 table: same operations, same bits
            assert torch.equal(got.view(torch.int32), want.view(torch.int32)), f"{where} {f.name}"
        elif got.dtype == torch.float32:
            torch.testing.assert_close(got, want, rtol=WEIGHT_RTOL, atol=1e-7, msg=f"{where} {f.name}")
        else:
            assert torch.equal(got, want), f"{where} {f.name}"
    for f in fields(cpu_state.deltas):
        got = getattr(device_state.deltas, f.name).detach().cpu()
        assert torch.equal(got, getattr(cpu_state.deltas, f.name)), f"{where} deltas.{f.name}"


def assert_step_equal(*, selection, attention, update, result: oracle.LayerResult, where: str = "",
                      check_update: bool = True) -> None:
    """Compare one device layer transition (workspace tensors of one sequence) with the oracle."""

    got_scores = selection.scores.detach().cpu().view(torch.int16)
    assert torch.equal(got_scores, result.scores.view(torch.int16)), f"{where} fp16 scores"
    counts = selection.descriptor_counts.detach().cpu()
    assert torch.equal(counts, result.descriptor_counts), f"{where} descriptor counts"
    for head in range(counts.shape[0]):
        n = int(counts[head])
        assert torch.equal(selection.communities[head, :n].cpu(), result.communities[head, :n]), f"{where} communities"
        assert torch.equal(selection.cumulative_ends[head, :n].cpu(), result.cumulative_ends[head, :n]), f"{where} ends"
    assert torch.equal(selection.tile_descriptors.cpu(), result.tile_descriptors), f"{where} tile starts"
    assert torch.equal(selection.positions.cpu(), result.positions), f"{where} gather positions"
    out = attention.output.detach().cpu().float()
    want = result.output.float()
    diff = (out - want).abs()
    assert float(diff.max()) <= OUTPUT_MAX_ABS, f"{where} output max-abs {float(diff.max())}"
    assert float(diff.mean()) <= OUTPUT_MEAN_ABS, f"{where} output mean-abs {float(diff.mean())}"
    torch.testing.assert_close(attention.lse.cpu(), result.lse, rtol=0, atol=2e-3, msg=f"{where} lse")
    assert torch.equal(attention.topk_positions.cpu(), result.topk_positions), f"{where} top-8 positions"
    assert torch.equal(
        attention.topk_scores.cpu().view(torch.int32), result.topk_scores.view(torch.int32)
    ), f"{where} top-8 scores"
    if check_update:
        assert torch.equal(update.assigned_communities.cpu(), result.assigned), f"{where} assigned"
        assert torch.equal(update.overflow.cpu(), result.overflow), f"{where} overflow"


def fp16_ulp_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance between fp16 tensors in units in the last place (0 where both are -inf)."""

    def ordered(x):
        bits = x.view(torch.int16).to(torch.int32) & 0xFFFF
        return torch.where(bits >= 0x8000, 0xFFFF - bits, bits + 0x8000)

    return (ordered(a) - ordered(b)).abs()


class OracleLayer:
    """Persistent CPU twin of one sequence's layer state, stepped by the oracle."""

    def __init__(self, csr, mutable, current, *, token_budget, num_sink, cover, max_communities=0):
        self.csr, self.state, self.current = cpu_clone(csr, mutable, current)
        heads, capacity, _ = self.state.centroids.shape
        self.token_budget = token_budget
        self.num_sink = num_sink
        self.cover = cover
        self.max_communities = max_communities
        selected = token_budget - num_sink - 1
        self.scores = torch.zeros((heads, capacity), dtype=torch.float16)
        self.communities = torch.full((heads, selected), -1, dtype=torch.int32)
        self.ends = torch.zeros((heads, selected), dtype=torch.int32)
        self.counts = torch.zeros((heads,), dtype=torch.int32)
        self.tiles = torch.zeros((heads, token_budget // 64), dtype=torch.int32)
        self.sinks = torch.arange(num_sink, dtype=torch.int32)

    def exact_scores(self, query) -> torch.Tensor:
        """Fixed-order fp16 scores of the current state (what the default device path reproduces)."""

        scores = torch.zeros_like(self.scores)
        oracle.score_centroids(
            query=query, centroids=self.state.centroids, community_sizes=self.state.community_sizes,
            community_counts=self.state.community_counts, scores=scores, cover=self.cover,
        )
        return scores

    def step(self, *, query, key, value, softmax_scale, lam, update=True, given_scores=None,
             device_scores=None, assignment="modularity") -> oracle.LayerResult:
        """``device_scores``: the fp16 scores the device produced for this step.  When the library
        scores on the tensor cores (its default) they are checked against the fixed-order scores to
        one unit in the last place and the rest of the step is computed from them, so that everything
        downstream is compared bit for bit; with ``CKV_TENSOR_SCORES=0`` they are ignored and the
        comparison of the scores themselves is exact."""

        if device_scores is not None and given_scores is None and ops.tensor_scores_enabled():
            given_scores = device_scores.detach().cpu().clone()
            exact = self.exact_scores(query)
            covered = torch.ones_like(exact, dtype=torch.bool)
            if self.cover is not None:
                covered = torch.arange(exact.shape[1])[None, :] < torch.as_tensor(self.cover)[:, None]
            distance = fp16_ulp_distance(given_scores, exact)[covered]
            assert int(distance.max()) <= 1, f"tensor-core score {int(distance.max())} ulp from the fixed-order score"
            assert float((distance > 0).float().mean()) < 5e-3
        return oracle.decode_layer(
            given_scores=given_scores,
            query=query,
            key=key,
            value=value,
            csr=self.csr,
            state=self.state,
            sink_positions=self.sinks,
            current_position=self.current,
            softmax_scale=softmax_scale,
            lam=lam,
            token_budget=self.token_budget,
            num_sink=self.num_sink,
            scores=self.scores,
            communities=self.communities,
            cumulative_ends=self.ends,
            descriptor_counts=self.counts,
            tile_descriptors=self.tiles,
            cover=self.cover,
            max_communities=self.max_communities,
            update=update,
            assignment=assignment,
        )

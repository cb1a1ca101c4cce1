"""The prefill score-graph kernel (tcgen05) against the CPU oracle, through the C ABI."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from community_kv_b200.prefill import (
    check_status,
    prefill_attention,
    prefill_attention_edges,
    prefill_attention_topk,
)
from oracle import prefill_oracle as oracle

pytestmark = pytest.mark.gpu
SCALE = 128 ** -0.5


def _inputs(seed, length, heads, kv_heads, clusters=16, batch=1):
    generator = torch.Generator().manual_seed(seed)
    centres = torch.randn((kv_heads, clusters, 128), generator=generator)
    labels = torch.randint(0, clusters, (batch, length, kv_heads), generator=generator)
    key = centres[torch.arange(kv_heads).view(1, 1, -1), labels] + 0.3 * torch.randn(
        (batch, length, kv_heads, 128), generator=generator
    )
    value = torch.randn((batch, length, kv_heads, 128), generator=generator)
    query = torch.randn((batch, length, heads, 128), generator=generator)
    # planted structure: queries lean towards their own cluster centre
    query = query + 0.5 * key.repeat_interleave(heads // kv_heads, dim=2)
    return (query.to(torch.bfloat16), (key / 128**0.5).to(torch.bfloat16) * 4, (value / 128**0.5).to(torch.bfloat16))


def _check_attention(out, lse, q, k, v, want_out, want_lse):
    diff = (out.float().cpu().numpy() - want_out)
    assert np.abs(diff).max() <= 2e-2, np.abs(diff).max()
    assert np.abs(diff).mean() <= 1e-3
    np.testing.assert_allclose(lse.cpu().numpy(), want_lse, atol=2e-3, rtol=0)


@pytest.mark.parametrize(
    "length,heads,kv_heads",
    [(256, 4, 1), (300, 8, 2), (640, 2, 2), (200, 8, 1), (512, 2, 1), (64, 4, 2), (1, 2, 1), (130, 4, 1), (129, 2, 2)],
)
def test_attention_output_and_lse(length, heads, kv_heads):
    q, k, v = _inputs(1, length, heads, kv_heads)
    out, lse = prefill_attention(q.cuda(), k.cuda(), v.cuda(), softmax_scale=SCALE)
    torch.cuda.synchronize()
    want_out, want_lse, _ = oracle.causal_attention(q[0].float().numpy(), k[0].float().numpy(), v[0].float().numpy(), SCALE)
    _check_attention(out[0], lse[0], q, k, v, want_out, want_lse)


def test_reference_topk_rule():
    length, heads, kv_heads, sinks = 640, 4, 1, 10
    q, k, v = _inputs(2, length, heads, kv_heads)
    out, lse, _, _, val, idx = prefill_attention_topk(q.cuda(), k.cuda(), v.cuda(), softmax_scale=SCALE, num_sink=sinks)
    torch.cuda.synchronize()
    assert val.shape == (1, heads, length - sinks - 7, 8) and idx.dtype == torch.int32
    want_out, want_lse, raw = oracle.causal_attention(q[0].float().numpy(), k[0].float().numpy(), v[0].float().numpy(), SCALE)
    _check_attention(out[0], lse[0], q, k, v, want_out, want_lse)
    got_idx = idx[0].cpu().numpy()
    got_val = val[0].cpu().numpy()
    exact_rows = 0
    total_rows = 0
    for head in range(heads):
        want_val, want_idx, want_key = oracle.reference_topk(raw[head], want_lse[head], SCALE, sinks)
        keys = oracle.quantised_keys(raw[head])
        for row in range(want_idx.shape[0]):
            position = row + sinks + 7
            total_rows += 1
            mine = got_idx[head, row]
            assert mine.min() >= sinks and mine.max() <= position
            assert len(set(mine.tolist())) == 8
            if np.array_equal(mine, want_idx[row]):
                exact_rows += 1
                np.testing.assert_allclose(got_val[head, row], want_val[row], rtol=2e-2, atol=1e-9)
                continue
            # the tensor-core score may land on the other side of a quantisation step:
            # every disagreement must sit within one step of the cut
            floor_key = want_key[row].min()
            for j in set(mine.tolist()) ^ set(want_idx[row].tolist()):
                assert abs(int(keys[position, j]) - int(floor_key)) <= 1, (head, row, j)
    assert exact_rows / total_rows > 0.97, exact_rows / total_rows


@pytest.mark.parametrize(
    "length,heads,kv_heads,edges",
    [(384, 4, 1, 16), (300, 8, 2, 8), (260, 2, 2, 16), (320, 4, 2, 16), (272, 8, 1, 16), (700, 8, 2, 16)],
)
def test_exact_edges_are_bit_exact(length, heads, kv_heads, edges):
    sinks = 4
    q, k, v = _inputs(3, length, heads, kv_heads)
    out, lse, edge_idx, edge_score, flags = prefill_attention_edges(
        q.cuda(), k.cuda(), v.cuda(), softmax_scale=SCALE, num_sink=sinks, edges_per_row=edges
    )
    torch.cuda.synchronize()
    want_idx, want_score = oracle.exact_edges(q[0].float().numpy(), k[0].float().numpy(), SCALE, sinks, edges)
    assert np.array_equal(edge_idx[0].cpu().numpy(), want_idx)
    assert np.array_equal(edge_score[0].cpu().numpy().view(np.uint32), want_score.view(np.uint32))
    want_out, want_lse, _ = oracle.causal_attention(q[0].float().numpy(), k[0].float().numpy(), v[0].float().numpy(), SCALE)
    _check_attention(out[0], lse[0], q, k, v, want_out, want_lse)
    assert int(flags.sum()) <= flags.numel() // 20


@pytest.mark.parametrize("length,heads,kv_heads,sinks", [(100, 4, 2, 4), (129, 8, 2, 0), (12, 2, 1, 3), (9, 4, 1, 4)])
def test_reference_topk_rule_short_and_ragged(length, heads, kv_heads, sinks):
    """Rows shorter than one tile, a tile of a single row, a prompt barely longer than the sinks."""

    q, k, v = _inputs(6, length, heads, kv_heads)
    out, lse, _, _, val, idx = prefill_attention_topk(q.cuda(), k.cuda(), v.cuda(), softmax_scale=SCALE, num_sink=sinks)
    torch.cuda.synchronize()
    rows = max(0, length - sinks - 7)
    assert val.shape == (1, heads, rows, 8) and idx.shape == (1, heads, rows, 8)
    want_out, want_lse, raw = oracle.causal_attention(q[0].float().numpy(), k[0].float().numpy(), v[0].float().numpy(), SCALE)
    _check_attention(out[0], lse[0], q, k, v, want_out, want_lse)
    for head in range(heads):
        if rows == 0:
            break
        want_val, want_idx, want_key = oracle.reference_topk(raw[head], want_lse[head], SCALE, sinks)
        keys = oracle.quantised_keys(raw[head])
        got_idx = idx[0, head].cpu().numpy()
        for row in range(rows):
            position = row + sinks + 7
            mine = got_idx[row]
            assert mine.min() >= sinks and mine.max() <= position and len(set(mine.tolist())) == 8
            floor_key = want_key[row].min()
            for j in set(mine.tolist()) ^ set(want_idx[row].tolist()):
                assert abs(int(keys[position, j]) - int(floor_key)) <= 1, (head, row, j)


def test_exact_edges_of_a_prompt_shorter_than_the_list():
    q, k, v = _inputs(7, 12, 4, 2)
    out, lse, edge_idx, edge_score, flags = prefill_attention_edges(
        q.cuda(), k.cuda(), v.cuda(), softmax_scale=SCALE, num_sink=4, edges_per_row=16)
    torch.cuda.synchronize()
    assert edge_idx.shape == (1, 2, 0, 16) and edge_score.shape == (1, 2, 0, 16) and flags.numel() == 0
    want_out, want_lse, _ = oracle.causal_attention(q[0].float().numpy(), k[0].float().numpy(), v[0].float().numpy(), SCALE)
    _check_attention(out[0], lse[0], q, k, v, want_out, want_lse)


def test_exact_edges_rescan_path():
    """A huge slack flags every row: the brute-force re-scan must give the same exact answer."""

    length, heads, kv_heads, edges, sinks = 200, 4, 1, 16, 3
    q, k, v = _inputs(4, length, heads, kv_heads)
    _, _, edge_idx, edge_score, flags = prefill_attention_edges(
        q.cuda(), k.cuda(), v.cuda(), softmax_scale=SCALE, num_sink=sinks, edges_per_row=edges, exact_slack=1e9
    )
    torch.cuda.synchronize()
    want_idx, want_score = oracle.exact_edges(q[0].float().numpy(), k[0].float().numpy(), SCALE, sinks, edges)
    assert np.array_equal(edge_idx[0].cpu().numpy(), want_idx)
    assert np.array_equal(edge_score[0].cpu().numpy().view(np.uint32), want_score.view(np.uint32))


def test_batch_and_validation():
    q, k, v = _inputs(5, 192, 4, 2, batch=2)
    out, lse = prefill_attention(q.cuda(), k.cuda(), v.cuda(), softmax_scale=SCALE)
    torch.cuda.synchronize()
    for b in range(2):
        want_out, want_lse, _ = oracle.causal_attention(q[b].float().numpy(), k[b].float().numpy(), v[b].float().numpy(), SCALE)
        _check_attention(out[b], lse[b], q, k, v, want_out, want_lse)
    # caller-owned status word: the calls queue without a host round trip, one check at the end
    status = torch.zeros((1,), dtype=torch.int32, device="cuda")
    again, _ = prefill_attention(q.cuda(), k.cuda(), v.cuda(), softmax_scale=SCALE, status=status)
    prefill_attention_topk(q.cuda(), k.cuda(), v.cuda(), softmax_scale=SCALE, num_sink=4, status=status)
    check_status(status)
    assert torch.equal(again, out)
    with pytest.raises(ValueError):
        prefill_attention(q.cuda(), k.cuda(), v.cuda(), softmax_scale=SCALE, status=status.to(torch.int64))
    with pytest.raises(RuntimeError):
        check_status(torch.full((1,), 4, dtype=torch.int32, device="cuda"))
    with pytest.raises(TypeError):
        prefill_attention(q.cuda().float(), k.cuda(), v.cuda(), softmax_scale=SCALE)
    with pytest.raises(ValueError):
        prefill_attention(q.cuda()[:, :, :3], k.cuda(), v.cuda(), softmax_scale=SCALE)


def test_full_size_properties():
    """The prefill configuration at full size (S = 16384, 32 / 8 heads, 256 planted clusters): sampled rows
    against fp32 torch arithmetic - attention within tolerance; every edge's score is the group
    maximum of that key, edges are sorted, and nothing outside the list beats the last edge."""

    device = torch.device("cuda", 0)
    length, heads, kv_heads, sinks, edges = 16384, 32, 8, 10, 16
    generator = torch.Generator(device=device).manual_seed(9)
    centres = torch.randn((kv_heads, 256, 128), generator=generator, device=device)
    labels = torch.randint(0, 256, (length, kv_heads), generator=generator, device=device)
    key = centres[torch.arange(kv_heads, device=device), labels] + 0.3 * torch.randn(
        (length, kv_heads, 128), generator=generator, device=device)
    key = (key * SCALE).to(torch.bfloat16)[None]
    value = (torch.randn((1, length, kv_heads, 128), generator=generator, device=device) * SCALE).to(torch.bfloat16)
    query = torch.randn((1, length, heads, 128), generator=generator, device=device).to(torch.bfloat16)
    out, lse, edge_idx, edge_score, flags = prefill_attention_edges(
        query, key, value, softmax_scale=SCALE, num_sink=sinks, edges_per_row=edges)
    torch.cuda.synchronize()
    skip = sinks + edges - 1
    group = heads // kv_heads
    rows = torch.randint(skip, length, (48,), generator=generator, device=device).tolist() + [skip, length - 1]
    k32, v32 = key[0].float(), value[0].float()
    for row in rows:
        q_row = query[0, row].float()  # [heads, 128]
        scores = torch.einsum("hd,jhd->hj", q_row.view(kv_heads, group, 128).reshape(heads, 128),
                              k32[: row + 1].repeat_interleave(group, dim=1)) * SCALE
        probabilities = torch.softmax(scores, dim=-1)
        want = torch.einsum("hj,jhd->hd", probabilities, v32[: row + 1].repeat_interleave(group, dim=1))
        assert float((out[0, row].float() - want).abs().max()) <= 2e-2, row
        best = scores.view(kv_heads, group, row + 1).amax(dim=1)  # [kv, keys]
        best[:, :sinks] = float("-inf")
        got_idx = edge_idx[0, :, row - skip].long()
        got_score = edge_score[0, :, row - skip]
        assert bool((got_idx >= sinks).all()) and bool((got_idx <= row).all()), row
        assert bool((got_score[:, :-1] >= got_score[:, 1:]).all()), row
        torch.testing.assert_close(got_score, best.gather(1, got_idx), rtol=0, atol=2e-5)
        rest = best.scatter(1, got_idx, float("-inf"))
        assert bool((rest.amax(dim=1) <= got_score[:, -1] + 2e-5).all()), row
    assert int(flags.sum()) <= flags.numel() // 100


def test_full_size_reference_topk_rule():
    """The reference's top-8 rule at full size (S = 16384, 32 / 8 heads): for sampled rows the rule is
    restated in fp32 torch arithmetic - key15 = clamp(rn((q.k + 48) * 256)), four column classes keep
    their six best packed candidates, the row reports the eight largest.  The kernel's scores come from
    the tensor cores, so a disagreement is accepted only where the keys involved sit within one
    quantisation step of the cut; the reported probabilities must match exp(score * scale - lse)."""

    device = torch.device("cuda", 0)
    length, heads, kv_heads, sinks = 16384, 32, 8, 10
    generator = torch.Generator(device=device).manual_seed(11)
    centres = torch.randn((kv_heads, 256, 128), generator=generator, device=device)
    labels = torch.randint(0, 256, (length, kv_heads), generator=generator, device=device)
    key = centres[torch.arange(kv_heads, device=device), labels] + 0.3 * torch.randn(
        (length, kv_heads, 128), generator=generator, device=device)
    key = (key * SCALE).to(torch.bfloat16)[None]
    value = (torch.randn((1, length, kv_heads, 128), generator=generator, device=device) * SCALE).to(torch.bfloat16)
    query = torch.randn((1, length, heads, 128), generator=generator, device=device).to(torch.bfloat16)
    out, lse, _, _, val, idx = prefill_attention_topk(query, key, value, softmax_scale=SCALE, num_sink=sinks)
    torch.cuda.synchronize()
    skip = sinks + 7
    group = heads // kv_heads
    rows = torch.randint(skip, length, (40,), generator=generator, device=device).tolist() + [skip, 127, 128, length - 1]
    k32 = key[0].float()
    exact_rows = 0
    for row in rows:
        q_row = query[0, row].float()  # [heads, 128]
        raw = torch.einsum("hd,jhd->hj", q_row, k32[: row + 1].repeat_interleave(group, dim=1))  # [heads, keys]
        keys = torch.clamp(torch.round((raw + 48.0) * 256.0), 0, 32767).long()
        columns = torch.arange(row + 1, device=device)
        packed = (keys << 17) | columns
        packed[:, :sinks] = -1
        kept = []
        for cls in range(4):
            members = packed[:, ((columns % 8) // 2) == cls]
            kept.append(members.topk(min(6, members.shape[1]), dim=1).values)
        want = torch.cat(kept, dim=1).topk(8, dim=1).values  # [heads, 8], descending
        want_idx = want & 0x1FFFF
        got_idx = idx[0, :, row - skip].long()
        got_val = val[0, :, row - skip]
        assert bool((got_idx >= sinks).all()) and bool((got_idx <= row).all()), row
        for head in range(heads):
            mine, theirs = set(got_idx[head].tolist()), set(want_idx[head].tolist())
            assert len(mine) == 8, (row, head)
            if got_idx[head].tolist() == want_idx[head].tolist():
                exact_rows += 1
            floor_key = int(want[head, -1] >> 17)
            for j in mine ^ theirs:
                assert abs(int(keys[head, j]) - floor_key) <= 1, (row, head, j)
        # probabilities from the dequantised key of the column the kernel chose
        chosen = keys.gather(1, got_idx).float() / 256.0 - 48.0
        want_val = torch.exp(chosen * SCALE - lse[0, :, row].unsqueeze(1))
        torch.testing.assert_close(got_val, want_val, rtol=3e-2, atol=1e-9)
    assert exact_rows / (len(rows) * heads) > 0.9, exact_rows / (len(rows) * heads)

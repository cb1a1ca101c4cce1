"""CPU oracle for one CommunityKV sparse-decode layer transition.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).  Parity pinned: the
functions below reproduce every known answer of the reference's unit tests
and the fixtures generated from the reference (``tests/test_oracle_golden.py``).

The functions are duck-typed on the reference's state objects (``PrefillCSR``,
``DecodeDeltaChunks``, ``MutableGraphState`` from ``community_kv/graph/state.py``)
holding CPU torch tensors; they mutate that state in place exactly as the
reference kernels do, so the same oracle runs against the reference's own
dataclasses and against this repository's mirrors of them.

Reference sources restated here (paths inside the reference project):

* centroid scoring        ``community_kv/attention/kernels/centroid_selection.py:56-108``
* ordered fp16 key        ``community_kv/attention/kernels/_csrc/descriptor_selection.cu:30-33``
* threshold search        ``descriptor_selection.cu:164-250``
* descriptor compaction   ``descriptor_selection.cu:342-455``
* tile start descriptors  ``descriptor_selection.cu:457-487``
* position resolution     ``community_kv/attention/kernels/segmented_attention.py:98-282``
* tile partials, top-8    ``segmented_attention.py:283-365``
* split merge             ``segmented_attention.py:446-484``
* online assignment       ``segmented_attention.py:486-864``
* shared-graph sync       ``segmented_attention.py:866-950``

Floating-point convention.  A 128-long dot product of bf16 (or fp8) operands is
accumulated in fp32 in one fixed order, ``fixed_dot``: eight 16-element slices
are each summed left to right starting from the first product, and the eight
slice sums are combined as ((p0+p4)+(p2+p6))+((p1+p5)+(p3+p7)).  Every product
of two such operands is exact in fp32, so a fused multiply-add and a separate
multiply and add give the same bits; the CUDA kernels use the same order, which
is what makes the integer outputs (selected communities, positions, labels)
reproducible bit for bit.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

HEAD_DIM = 128
TILE = 64
KAPPA = 8
MAX_DELTA_WALK = 32
FP8_MAX = 448.0


# --------------------------------------------------------------------------- #
# numeric helpers
# --------------------------------------------------------------------------- #
def f32(tensor: torch.Tensor) -> np.ndarray:
    """Exact widening of a bf16 / fp8 / fp16 / fp32 torch tensor to numpy fp32."""

    return tensor.detach().to(device="cpu", dtype=torch.float32).contiguous().numpy()


def fixed_dot(left: np.ndarray, right: np.ndarray) -> np.ndarray:
    """fp32 dot over the last axis (length 128) in the kernels' fixed order."""

    left = np.asarray(left, dtype=np.float32)
    right = np.asarray(right, dtype=np.float32)
    if left.shape[-1] != HEAD_DIM or right.shape[-1] != HEAD_DIM:
        raise ValueError("fixed_dot needs a trailing axis of 128")
    partial = []
    for piece in range(8):
        base = piece * 16
        acc = (left[..., base] * right[..., base]).astype(np.float32)
        for offset in range(1, 16):
            product = (left[..., base + offset] * right[..., base + offset]).astype(
                np.float32
            )
            acc = (acc + product).astype(np.float32)
        partial.append(acc)
    even = ((partial[0] + partial[4]).astype(np.float32)
            + (partial[2] + partial[6]).astype(np.float32)).astype(np.float32)
    odd = ((partial[1] + partial[5]).astype(np.float32)
           + (partial[3] + partial[7]).astype(np.float32)).astype(np.float32)
    return (even + odd).astype(np.float32)


def ordered_fp16_keys(bits: np.ndarray) -> np.ndarray:
    """Order-preserving uint16 key of fp16 bit patterns (descriptor_selection.cu:30-33)."""

    bits = np.asarray(bits, dtype=np.uint16)
    flip = np.where((bits & 0x8000) != 0, 0xFFFF, 0x8000).astype(np.uint16)
    return np.bitwise_xor(bits, flip)


def ordered_f32_bits(values: np.ndarray) -> np.ndarray:
    bits = np.asarray(values, dtype=np.float32).view(np.uint32)
    return np.where((bits & 0x80000000) != 0, ~bits, bits ^ np.uint32(0x80000000)).astype(
        np.uint32
    )


def to_fp8_saturating(values: np.ndarray) -> torch.Tensor:
    """fp32 -> e4m3 with round-to-nearest-even and saturation at +-448."""

    clipped = np.clip(np.asarray(values, dtype=np.float32), -FP8_MAX, FP8_MAX)
    return torch.from_numpy(clipped).to(torch.float8_e4m3fn)


# --------------------------------------------------------------------------- #
# A1: centroid scoring
# --------------------------------------------------------------------------- #
def score_centroids(
    *,
    query: torch.Tensor,
    centroids: torch.Tensor,
    community_sizes: torch.Tensor,
    community_counts: torch.Tensor,
    scores: torch.Tensor,
    cover: list[int] | None = None,
    exact: bool = True,
) -> torch.Tensor:
    """scores[r, c] = fp16(max_g q[rG+g] . centroid[r, c]); -inf if inactive or empty.

    ``cover[r]`` limits the written range to the 64-blocks below
    ``min(capacity, cover[r])`` like the reference's ragged schedule
    (centroid_selection.py:232-250); other entries stay untouched.  With
    ``exact=False`` the dot products use a BLAS einsum (same math, library
    summation order) - that is the timed CPU baseline, not the parity checker.
    """

    heads, capacity, _ = centroids.shape
    group = query.shape[0] // heads
    q = f32(query).reshape(heads, group, HEAD_DIM)
    out = scores.view(torch.int16).numpy().view(np.uint16)
    sizes = community_sizes.numpy()
    counts = community_counts.numpy()
    for head in range(heads):
        limit = capacity
        if cover is not None:
            limit = min(capacity, -(-min(capacity, int(cover[head])) // TILE) * TILE)
        if limit <= 0:
            continue
        cent = f32(centroids[head, :limit])
        if exact:
            dots = fixed_dot(q[head][:, None, :], cent[None, :, :])
        else:
            dots = np.einsum("gd,cd->gc", q[head], cent).astype(np.float32)
        best = dots.max(axis=0)
        index = np.arange(limit)
        live = (index < int(counts[head])) & (sizes[head, :limit] > 0)
        best = np.where(live, best, -np.inf).astype(np.float32)
        out[head, :limit] = best.astype(np.float16).view(np.uint16)
    return scores


# --------------------------------------------------------------------------- #
# A2: weighted radix-threshold descriptor selection
# --------------------------------------------------------------------------- #
@dataclass(frozen=True)
class Selection:
    communities: np.ndarray
    cumulative_ends: np.ndarray
    threshold_key: int


def _descending_threshold(histogram: np.ndarray, budget: int, start: int) -> tuple[int, int]:
    cumulative = start
    for bin_index in range(255, -1, -1):
        if cumulative + int(histogram[bin_index]) >= budget:
            return bin_index, cumulative
        cumulative += int(histogram[bin_index])
    return 0, start


def select_descriptors(
    score_bits: np.ndarray,
    sizes: np.ndarray,
    active: int,
    selected_budget: int,
    *,
    max_communities: int = 0,
) -> Selection:
    """Exact weighted selection of one retrieval head (descriptor_selection.cu:164-455).

    Communities whose ordered key exceeds the threshold come first, in
    ascending community index, followed by communities equal to the threshold
    while the running start is below the budget; the last one is truncated.

    ``max_communities > 0`` is this repository's extension ("top-k communities
    under a token budget"): the prefix in (key descending, index ascending)
    order additionally stops after that many communities.
    """

    capacity = score_bits.shape[0]
    active = max(0, min(capacity, int(active)))
    keys = ordered_fp16_keys(score_bits[:active]).astype(np.int64)
    size = sizes[:active].astype(np.int64)
    live = size > 0
    limit_count = max_communities if max_communities > 0 else None

    def threshold(byte_of, mask, start_mass, start_count):
        mass_hist = np.zeros(256, dtype=np.int64)
        count_hist = np.zeros(256, dtype=np.int64)
        np.add.at(mass_hist, byte_of[mask], size[mask])
        np.add.at(count_hist, byte_of[mask], 1)
        mass, count = start_mass, start_count
        for bin_index in range(255, -1, -1):
            hit = mass + int(mass_hist[bin_index]) >= selected_budget
            if limit_count is not None:
                hit = hit or count + int(count_hist[bin_index]) >= limit_count
            if hit:
                return bin_index, mass, count
            mass += int(mass_hist[bin_index])
            count += int(count_hist[bin_index])
        return 0, start_mass, start_count

    high_bin, mass_above, count_above = threshold(keys >> 8, live, 0, 0)
    in_bin = live & ((keys >> 8) == high_bin)
    low_bin, _, _ = threshold(keys & 0xFF, in_bin, mass_above, count_above)
    threshold_key = (high_bin << 8) | low_bin

    high = live & (keys > threshold_key)
    equal = live & (keys == threshold_key)
    high_index = np.nonzero(high)[0]
    high_ends = np.cumsum(size[high_index])
    total_high_mass = int(high_ends[-1]) if high_index.size else 0
    total_high_count = int(high_index.size)

    equal_index = np.nonzero(equal)[0]
    equal_sizes = size[equal_index]
    equal_start = total_high_mass + np.concatenate(([0], np.cumsum(equal_sizes)[:-1])) if equal_index.size else np.zeros(0, dtype=np.int64)
    stored = equal_start < selected_budget
    if limit_count is not None and equal_index.size:
        stored &= (total_high_count + np.arange(equal_index.size)) < limit_count
    equal_ends = np.minimum(selected_budget, equal_start + equal_sizes)

    communities = np.concatenate((high_index, equal_index[stored])).astype(np.int32)
    ends = np.concatenate((high_ends, equal_ends[stored])).astype(np.int32)
    return Selection(communities, ends, int(threshold_key))


def tile_start_descriptors(
    cumulative_ends: np.ndarray,
    count: int,
    tile_count: int,
    num_sink: int,
) -> np.ndarray:
    """First descriptor of every 64-token tile (descriptor_selection.cu:457-487)."""

    ends = cumulative_ends[:count]
    tiles = np.zeros(tile_count, dtype=np.int32)
    for tile in range(tile_count):
        offset = max(tile * TILE - num_sink, 0)
        low = int(np.searchsorted(ends, offset, side="right"))
        tiles[tile] = max(0, min(low, count - 1))
    return tiles


def select_into_workspace(
    *,
    scores: torch.Tensor,
    community_sizes: torch.Tensor,
    community_counts: torch.Tensor,
    communities: torch.Tensor,
    cumulative_ends: torch.Tensor,
    descriptor_counts: torch.Tensor,
    tile_descriptors: torch.Tensor,
    num_sink: int,
    max_communities: int = 0,
) -> list[Selection]:
    """Run the selection for every retrieval head and fill the packed-segment tensors."""

    heads = scores.shape[0]
    tile_count = tile_descriptors.shape[1]
    selected_budget = tile_count * TILE - num_sink - 1
    bits = scores.view(torch.int16).numpy().view(np.uint16)
    result = []
    for head in range(heads):
        selection = select_descriptors(
            bits[head],
            community_sizes[head].numpy(),
            int(community_counts[head]),
            selected_budget,
            max_communities=max_communities,
        )
        count = selection.communities.shape[0]
        communities[head, :count] = torch.from_numpy(selection.communities)
        cumulative_ends[head, :count] = torch.from_numpy(selection.cumulative_ends)
        descriptor_counts[head] = count
        tile_descriptors[head] = torch.from_numpy(
            tile_start_descriptors(selection.cumulative_ends, count, tile_count, num_sink)
        )
        result.append(selection)
    return result


# --------------------------------------------------------------------------- #
# A3 (integer half): logical token -> cache position
# --------------------------------------------------------------------------- #
def _delta_position(deltas, graph: int, community: int, member: int) -> int:
    """Newest-first member of the decode-delta chain (segmented_attention.py:186-258)."""

    chunk = int(deltas.community_tail[graph, community])
    remaining = member
    for _ in range(MAX_DELTA_WALK):
        if chunk < 0:
            break
        size = int(deltas.chunk_size[graph, chunk])
        if remaining < size:
            start = int(deltas.chunk_start[graph, chunk])
            return int(deltas.positions[graph, start + size - 1 - remaining])
        remaining -= size
        chunk = int(deltas.chunk_previous[graph, chunk])
    return 0


def resolve_positions(
    *,
    graph: int,
    csr,
    deltas,
    communities: np.ndarray,
    cumulative_ends: np.ndarray,
    count: int,
    sink_positions: np.ndarray,
    current_position: int,
    token_budget: int,
    num_sink: int,
) -> np.ndarray:
    """Cache position of each of the ``token_budget`` logical tokens of one head.

    Layout: sinks, then the selected members descriptor by descriptor (decode
    deltas newest first, then prefill members in stored order), then the
    current token.  Logical tokens beyond the selected mass (only possible when
    the budget is under-filled, which the reference never allows) are -1.
    """

    positions = np.full(token_budget, -1, dtype=np.int32)
    positions[:num_sink] = sink_positions[:num_sink]
    positions[token_budget - 1] = current_position
    offsets = csr.member_offsets[graph].numpy()
    members = csr.member_positions[graph].numpy()
    delta_sizes = deltas.community_sizes[graph].numpy()
    previous_end = 0
    for index in range(count):
        community = int(communities[index])
        end = int(cumulative_ends[index])
        delta_count = int(delta_sizes[community])
        base = int(offsets[community])
        for member in range(end - previous_end):
            logical = num_sink + previous_end + member
            if member < delta_count:
                positions[logical] = _delta_position(deltas, graph, community, member)
            else:
                positions[logical] = members[base + member - delta_count]
        previous_end = end
    return positions


# --------------------------------------------------------------------------- #
# A3 (floating half) + A4: tile partials and split merge
# --------------------------------------------------------------------------- #
def _bf16_round(values: np.ndarray) -> np.ndarray:
    return torch.from_numpy(np.ascontiguousarray(values, dtype=np.float32)).to(
        torch.bfloat16
    ).float().numpy()


def attention_unit(
    *,
    query_group: np.ndarray,
    key_rows: np.ndarray,
    value_rows: np.ndarray,
    valid: np.ndarray,
    softmax_scale: float,
    exact: bool = True,
) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Exact attention of one query group over its gathered rows.

    Returns ``(output fp32 [G,128] before the bf16 store, lse fp32 [G],
    scaled scores fp32 [G,T])``.  The arithmetic follows the reference's
    64-token tiles: ``p = exp(s - tile max)``, the row sum uses fp32 ``p``, the
    value product uses ``bf16(p)`` (segmented_attention.py:333-345), and tiles
    are merged with the log-sum-exp rule (segmented_attention.py:446-484).
    """

    scale = np.float32(softmax_scale)
    if exact:
        scores = fixed_dot(query_group[:, None, :], key_rows[None, :, :])
    else:
        scores = (query_group @ key_rows.T).astype(np.float32)
    scores = (scores * scale).astype(np.float32)
    scores = np.where(valid[None, :], scores, -np.inf).astype(np.float32)
    groups, tokens = scores.shape
    tiles = tokens // TILE
    tile_scores = scores.reshape(groups, tiles, TILE)
    tile_max = tile_scores.max(axis=2)
    safe_max = np.where(np.isfinite(tile_max), tile_max, 0.0).astype(np.float32)
    probability = np.exp(tile_scores - safe_max[:, :, None]).astype(np.float32)
    probability = np.where(np.isfinite(tile_scores), probability, 0.0).astype(np.float32)
    tile_sum = probability.sum(axis=2, dtype=np.float32)
    rounded = _bf16_round(probability)
    values = value_rows.reshape(tiles, TILE, HEAD_DIM)
    tile_acc = np.einsum("gtn,tnd->gtd", rounded, values).astype(np.float32)

    global_max = tile_max.max(axis=1)
    weight = np.exp(np.where(np.isfinite(tile_max), tile_max - global_max[:, None], -np.inf)).astype(
        np.float32
    )
    denominator = (tile_sum * weight).sum(axis=1, dtype=np.float32)
    output = (tile_acc * weight[:, :, None]).sum(axis=1, dtype=np.float32) / denominator[:, None]
    lse = (global_max + np.log(denominator)).astype(np.float32)
    return output.astype(np.float32), lse, scores


def global_topk(
    representative_scores: np.ndarray,
    positions: np.ndarray,
    is_sink: np.ndarray,
) -> tuple[np.ndarray, np.ndarray]:
    """Top-8 (score descending, position ascending) of the non-sink tokens.

    Equals the reference's per-tile top-8 followed by the global merge of the
    packed 64-bit keys (segmented_attention.py:304-331, 487-544).
    """

    valid = positions >= 0
    candidate = np.where(is_sink, -np.inf, representative_scores).astype(np.float32)
    packed = (ordered_f32_bits(candidate).astype(np.uint64) << np.uint64(32)) | (
        np.uint64(0xFFFFFFFF) - positions.astype(np.int64).astype(np.uint64) & np.uint64(0xFFFFFFFF)
    )
    packed = np.where(valid, packed, np.uint64(0))
    order = np.sort(packed)[::-1][:KAPPA]
    if order.shape[0] < KAPPA:
        order = np.concatenate((order, np.zeros(KAPPA - order.shape[0], dtype=np.uint64)))
    ordered = (order >> np.uint64(32)).astype(np.uint32)
    bits = np.where((ordered & 0x80000000) != 0, ordered ^ np.uint32(0x80000000), ~ordered)
    scores = bits.astype(np.uint32).view(np.float32)
    tie = (order & np.uint64(0xFFFFFFFF)).astype(np.uint32)
    top_positions = (np.uint32(0xFFFFFFFF) - tie).astype(np.uint32).view(np.int32)
    return scores.copy(), top_positions.copy()


# --------------------------------------------------------------------------- #
# A5: constant-time online assignment and state update
# --------------------------------------------------------------------------- #
def online_update(
    *,
    state,
    retrieval_head: int,
    graph: int,
    kv_head: int,
    topk_scores: np.ndarray,
    topk_positions: np.ndarray,
    representative_lse: np.float32,
    key_cache: torch.Tensor,
    current_position: torch.Tensor,
    lam: float,
    assigned_out: torch.Tensor,
    overflow_out: torch.Tensor,
    forced_community: int = -1,
) -> None:
    """Leader-program half of the reduce/update kernel (segmented_attention.py:546-864).

    ``forced_community`` (not in the reference): a live community the token joins instead of
    the one the dQ rule picks - the nearest-centroid assignment variant.
    """

    one = np.float32(1.0)
    lam32 = np.float32(lam)
    sequence_capacity = key_cache.shape[1]
    token_capacity = state.token_communities.shape[1]
    community_capacity = state.centroids.shape[1]
    deltas = state.deltas

    valid = (topk_positions >= 0) & (topk_positions < sequence_capacity)
    community = np.full(KAPPA, -1, dtype=np.int64)
    for rank in range(KAPPA):
        if valid[rank] and int(topk_positions[rank]) < token_capacity:
            community[rank] = int(state.token_communities[graph, int(topk_positions[rank])])
    with np.errstate(invalid="ignore", over="ignore"):
        score = np.where(
            valid, np.exp((topk_scores - representative_lse).astype(np.float32)), 0.0
        ).astype(np.float32)
    direct = (score * np.float32(lam32 * np.float32(0.5))).astype(np.float32)
    node_degree = np.float32(0.0)
    score_sum = np.float32(0.0)
    square_sum = np.float32(0.0)
    for rank in range(KAPPA):
        node_degree = np.float32(node_degree + direct[rank])
        score_sum = np.float32(score_sum + score[rank])
        square_sum = np.float32(square_sum + np.float32(score[rank] * score[rank]))
    pair_weight = np.float32(
        np.float32(np.float32(score_sum * score_sum) - square_sum)
        * np.float32(np.float32(0.5) * np.float32(one - lam32))
    )

    active = int(state.community_counts[retrieval_head])
    candidate = valid & (community >= 0) & (community < active)
    candidate_weight = np.zeros(KAPPA, dtype=np.float32)
    first_rank = np.full(KAPPA, KAPPA, dtype=np.int64)
    for rank in range(KAPPA):
        total = np.float32(0.0)
        for other in range(KAPPA):
            if candidate[other] and community[other] == community[rank]:
                total = np.float32(total + direct[other])
                first_rank[rank] = min(first_rank[rank], other)
        candidate_weight[rank] = total
    leader = candidate & (np.arange(KAPPA) == first_rank)

    old_total = np.float32(state.total_weight[graph])
    two_m = np.float32(max(np.float32(np.float32(2.0) * old_total), one))
    old_weight = np.zeros(KAPPA, dtype=np.float32)
    delta_q = np.full(KAPPA, -np.inf, dtype=np.float32)
    for rank in range(KAPPA):
        if candidate[rank]:
            old_weight[rank] = np.float32(state.community_weight[graph, int(community[rank])])
            if candidate_weight[rank] > 0.0:
                delta_q[rank] = np.float32(
                    candidate_weight[rank]
                    - np.float32(np.float32(node_degree * old_weight[rank]) / two_m)
                )
    best_delta = delta_q.max()
    tied = candidate & (delta_q == best_delta)
    best_community = int(community[tied].min()) if tied.any() else 0x7FFFFFFF
    join = bool(best_delta > 0.0)
    assigned = best_community if join else active
    if 0 <= forced_community < active:
        join = True
        assigned = forced_community
    community_overflow = assigned >= community_capacity
    safe_assigned = min(max(assigned, 0), community_capacity - 1)

    if not community_overflow:
        for rank in range(KAPPA):
            if leader[rank]:
                increment = candidate_weight[rank]
                if join and int(community[rank]) == safe_assigned:
                    increment = np.float32(increment + node_degree)
                state.community_weight[graph, int(community[rank])] = float(
                    np.float32(old_weight[rank] + increment)
                )
        if not join:
            state.community_weight[graph, safe_assigned] = float(node_degree)
        state.community_counts[retrieval_head] = active + (0 if join else 1)
        state.total_weight[graph] = float(
            np.float32(np.float32(old_total + node_degree) + pair_weight)
        )
    assigned_out[graph] = -1 if community_overflow else assigned

    current = int(current_position[graph])
    valid_position = 0 <= current < sequence_capacity
    chunk_overflow = False
    position_overflow = False
    if not community_overflow:
        old_size = int(state.community_sizes[retrieval_head, safe_assigned])
        new_size = old_size + 1
        state.community_sizes[retrieval_head, safe_assigned] = new_size
        if valid_position:
            if current < token_capacity:
                state.token_communities[graph, current] = assigned
            apply_centroid_update(
                state, retrieval_head, safe_assigned, old_size, key_cache[kv_head, current]
            )

        delta_size = int(deltas.community_sizes[graph, safe_assigned])
        old_tail = int(deltas.community_tail[graph, safe_assigned])
        old_chunk_size = int(deltas.chunk_size[graph, old_tail]) if old_tail >= 0 else 0
        old_chunk_capacity = int(deltas.chunk_capacity[graph, old_tail]) if old_tail >= 0 else 0
        allocate = old_tail < 0 or old_chunk_size >= old_chunk_capacity
        free_chunk = int(deltas.next_free_chunk[graph])
        free_position = int(deltas.next_free_position[graph])
        new_capacity = 1 if old_tail < 0 else old_chunk_capacity * 2
        chunks_per_graph = deltas.chunk_start.shape[1]
        position_capacity = deltas.positions.shape[1]
        chunk_overflow = allocate and free_chunk >= chunks_per_graph
        position_overflow = allocate and free_position + new_capacity > position_capacity
        allocation_overflow = chunk_overflow or position_overflow
        chunk = free_chunk if allocate else old_tail
        valid_chunk = (not allocation_overflow) and 0 <= chunk < chunks_per_graph
        if allocate and not allocation_overflow:
            deltas.next_free_chunk[graph] = free_chunk + 1
            deltas.next_free_position[graph] = free_position + new_capacity
            deltas.chunk_start[graph, free_chunk] = free_position
            deltas.chunk_capacity[graph, free_chunk] = new_capacity
            deltas.chunk_previous[graph, free_chunk] = old_tail
            if old_tail < 0:
                deltas.community_head[graph, safe_assigned] = free_chunk
            else:
                deltas.chunk_next[graph, old_tail] = free_chunk
            deltas.community_tail[graph, safe_assigned] = free_chunk
        if valid_chunk and valid_position:
            if allocate:
                target_start, target_slot = free_position, 0
            else:
                target_start, target_slot = int(deltas.chunk_start[graph, old_tail]), old_chunk_size
            deltas.positions[graph, target_start + target_slot] = current
            deltas.chunk_size[graph, chunk] = target_slot + 1
            deltas.community_sizes[graph, safe_assigned] = delta_size + 1

    overflow = (
        int(community_overflow)
        | (int(chunk_overflow) << 1)
        | (int(position_overflow) << 2)
        | (int(not valid_position) << 3)
    )
    overflow_out[graph] = overflow
    if overflow == 0:
        current_position[graph] = current + 1


def apply_centroid_update(state, retrieval_head: int, community: int, old_size: int, key_row: torch.Tensor) -> None:
    """Running mean in fp32 stored back as saturating e4m3 (segmented_attention.py:685-717);
    stored as it is when the table is fp32 (not the reference's layout)."""

    old = f32(state.centroids[retrieval_head, community])
    key = f32(key_row)
    if old_size > 0:
        scaled = (old * np.float32(old_size)).astype(np.float32)
        updated = ((scaled + key).astype(np.float32) / np.float32(old_size + 1)).astype(np.float32)
    else:
        updated = key
    if state.centroids.dtype == torch.float32:
        state.centroids[retrieval_head, community] = torch.from_numpy(np.asarray(updated, dtype=np.float32))
    else:
        state.centroids[retrieval_head, community] = to_fp8_saturating(updated)


def sync_shared_graph(
    *,
    state,
    retrieval_head: int,
    key_cache: torch.Tensor,
    current_position: torch.Tensor,
    assigned: torch.Tensor,
    overflow: torch.Tensor,
) -> None:
    """Follower heads of a shared graph (segmented_attention.py:866-950)."""

    graph = int(state.retrieval_to_graph[retrieval_head])
    if retrieval_head == graph:
        return
    community = int(assigned[graph])
    if int(overflow[graph]) != 0 or community < 0:
        return
    kv_head = int(state.retrieval_to_kv[retrieval_head])
    current = int(current_position[graph]) - 1
    old_size = int(state.community_sizes[retrieval_head, community])
    state.community_sizes[retrieval_head, community] = old_size + 1
    if 0 <= current < key_cache.shape[1]:
        apply_centroid_update(state, retrieval_head, community, old_size, key_cache[kv_head, current])
    state.community_counts[retrieval_head] = int(state.community_counts[graph])


# --------------------------------------------------------------------------- #
# composition: one layer transition (decode.py:67-111)
# --------------------------------------------------------------------------- #
@dataclass
class LayerResult:
    output: torch.Tensor
    lse: torch.Tensor
    topk_scores: torch.Tensor
    topk_positions: torch.Tensor
    assigned: torch.Tensor
    overflow: torch.Tensor
    scores: torch.Tensor
    communities: torch.Tensor
    cumulative_ends: torch.Tensor
    descriptor_counts: torch.Tensor
    tile_descriptors: torch.Tensor
    positions: torch.Tensor


def decode_layer(
    *,
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    csr,
    state,
    sink_positions: torch.Tensor,
    current_position: torch.Tensor,
    softmax_scale: float,
    lam: float,
    token_budget: int,
    num_sink: int,
    scores: torch.Tensor | None = None,
    communities: torch.Tensor | None = None,
    cumulative_ends: torch.Tensor | None = None,
    descriptor_counts: torch.Tensor | None = None,
    tile_descriptors: torch.Tensor | None = None,
    cover: list[int] | None = None,
    max_communities: int = 0,
    update: bool = True,
    exact: bool = True,
    given_scores: torch.Tensor | None = None,
    assignment: str = "modularity",
) -> LayerResult:
    """Score, select, attend, assign: the whole per-layer decode transition on CPU.

    With ``given_scores`` (fp16 ``[heads, capacity]``) the scoring step is skipped and the
    selection starts from those scores: that is how a device path whose scores come out
    of the tensor cores (hardware summation order, last fp16 bit not reproducible here)
    is checked - its scores against ``score_centroids`` to one unit in the last place,
    everything downstream bit for bit given its scores.

    ``assignment="nearest_centroid"`` (not in the reference): the decoded token joins the live
    community whose centroid has the largest inner product with its key - the scores are those
    of ``score_centroids`` for a query group whose rows all equal the key, the first maximum
    wins - instead of the community the dQ rule picks.
    """

    heads, capacity, _ = state.centroids.shape
    group = query.shape[0] // heads
    graph_count = state.total_weight.shape[0]
    tile_count = token_budget // TILE
    selected_budget = token_budget - num_sink - 1
    if scores is None:
        scores = torch.zeros((heads, capacity), dtype=torch.float16)
    if communities is None:
        communities = torch.full((heads, selected_budget), -1, dtype=torch.int32)
    if cumulative_ends is None:
        cumulative_ends = torch.zeros((heads, selected_budget), dtype=torch.int32)
    if descriptor_counts is None:
        descriptor_counts = torch.zeros((heads,), dtype=torch.int32)
    if tile_descriptors is None:
        tile_descriptors = torch.zeros((heads, tile_count), dtype=torch.int32)

    if given_scores is not None:
        scores.copy_(given_scores)
    else:
        score_centroids(
            query=query,
            centroids=state.centroids,
            community_sizes=state.community_sizes,
            community_counts=state.community_counts,
            scores=scores,
            cover=cover,
            exact=exact,
        )
    select_into_workspace(
        scores=scores,
        community_sizes=state.community_sizes,
        community_counts=state.community_counts,
        communities=communities,
        cumulative_ends=cumulative_ends,
        descriptor_counts=descriptor_counts,
        tile_descriptors=tile_descriptors,
        num_sink=num_sink,
        max_communities=max_communities,
    )

    q = f32(query).reshape(heads, group, HEAD_DIM)
    sinks = sink_positions.numpy()
    output = torch.zeros((heads * group, HEAD_DIM), dtype=torch.bfloat16)
    lse = torch.zeros((heads * group,), dtype=torch.float32)
    topk_scores = torch.zeros((heads, KAPPA), dtype=torch.float32)
    topk_positions = torch.zeros((heads, KAPPA), dtype=torch.int32)
    positions_out = torch.zeros((heads, token_budget), dtype=torch.int32)
    assigned = torch.zeros((graph_count,), dtype=torch.int32)
    overflow = torch.zeros((graph_count,), dtype=torch.int32)
    is_sink = np.arange(token_budget) < num_sink

    for head in range(heads):
        graph = int(state.retrieval_to_graph[head])
        kv_head = int(state.retrieval_to_kv[head])
        count = int(descriptor_counts[head])
        positions = resolve_positions(
            graph=graph,
            csr=csr,
            deltas=state.deltas,
            communities=communities[head].numpy(),
            cumulative_ends=cumulative_ends[head].numpy(),
            count=count,
            sink_positions=sinks,
            current_position=int(current_position[graph]),
            token_budget=token_budget,
            num_sink=num_sink,
        )
        positions_out[head] = torch.from_numpy(positions)
        valid = positions >= 0
        safe = torch.from_numpy(np.where(valid, positions, 0).astype(np.int64))
        key_rows = f32(key[kv_head].index_select(0, safe))
        value_rows = f32(value[kv_head].index_select(0, safe))
        out, head_lse, unit_scores = attention_unit(
            query_group=q[head],
            key_rows=key_rows,
            value_rows=value_rows,
            valid=valid,
            softmax_scale=softmax_scale,
            exact=exact,
        )
        output[head * group : (head + 1) * group] = torch.from_numpy(out).to(torch.bfloat16)
        lse[head * group : (head + 1) * group] = torch.from_numpy(head_lse)
        top_scores, top_positions = global_topk(unit_scores[0], positions, is_sink)
        topk_scores[head] = torch.from_numpy(top_scores)
        topk_positions[head] = torch.from_numpy(top_positions)

    nearest = None
    if update and assignment == "nearest_centroid":
        # the new token's key per retrieval head (already in the cache at the graph's cursor), as a
        # query group of identical rows, against the centroids as they are before this update
        rows = []
        for head in range(heads):
            graph = int(state.retrieval_to_graph[head])
            cursor = min(int(current_position[graph]), key.shape[1] - 1)
            rows.append(key[int(state.retrieval_to_kv[head]), cursor])
        key_query = torch.stack(rows).repeat_interleave(group, dim=0)
        key_scores = torch.zeros((heads, capacity), dtype=torch.float16)
        score_centroids(
            query=key_query, centroids=state.centroids, community_sizes=state.community_sizes,
            community_counts=state.community_counts, scores=key_scores, cover=None, exact=True,
        )
        best = key_scores.float().max(dim=1)
        nearest = torch.where(torch.isinf(best.values) & (best.values < 0), -1, best.indices)
    if update:
        for head in range(heads):
            graph = int(state.retrieval_to_graph[head])
            if head != graph:
                continue
            forced = -1
            if assignment == "nearest_centroid":
                forced = int(nearest[head])
            online_update(
                forced_community=forced,
                state=state,
                retrieval_head=head,
                graph=graph,
                kv_head=int(state.retrieval_to_kv[head]),
                topk_scores=topk_scores[head].numpy(),
                topk_positions=topk_positions[head].numpy(),
                representative_lse=np.float32(lse[head * group]),
                key_cache=key,
                current_position=current_position,
                lam=lam,
                assigned_out=assigned,
                overflow_out=overflow,
            )
        if heads != graph_count:
            for head in range(heads):
                sync_shared_graph(
                    state=state,
                    retrieval_head=head,
                    key_cache=key,
                    current_position=current_position,
                    assigned=assigned,
                    overflow=overflow,
                )

    return LayerResult(
        output=output,
        lse=lse,
        topk_scores=topk_scores,
        topk_positions=topk_positions,
        assigned=assigned,
        overflow=overflow,
        scores=scores,
        communities=communities,
        cumulative_ends=cumulative_ends,
        descriptor_counts=descriptor_counts,
        tile_descriptors=tile_descriptors,
        positions=positions_out,
    )

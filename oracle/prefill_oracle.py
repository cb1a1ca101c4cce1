"""CPU oracle for the prefill score-graph kernel.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

Parity status: the reference's unit tests pin only the call contract of its
patched FlashAttention kernel (``tests/community_kv/attention/test_flash_attention.py:8-41``),
no numbers, and that kernel runs on SM90 only, so the numerical parity of this
function is **unpinned** by reference outputs.  What is restated here, from the
patch itself (``third_party/flash_attention/community-kv.patch``):

* output rows / shapes and the omitted first ``num_sink + 7`` rows (``:69-82``);
* the candidate key ``key15 = clamp(rn((s + 48) * 256), 0, 32767)`` on the raw
  score, packed with the 17-bit key index (``hopper/topk_warpselect.h`` ``:547-560``);
* four column classes per row, each keeping its six largest packed candidates,
  merged to the eight largest (``:509, 562-571, 657-690``).  The class of a column
  is the accumulator lane that holds it, ``(j % 8) // 2`` for the m64nNk16
  accumulator fragment;
* the reported value ``exp2(dequant(key15) * scale * log2e - lse * log2e)`` (``:674-678``).

The exact-edge variant (top-m per KV head of the group-maximum scaled score,
fixed fp32 summation order, ties to the smaller index) has no reference
counterpart; it is defined here and in the kernel together.
"""

from __future__ import annotations

import numpy as np

from oracle.decode_oracle import fixed_dot, ordered_f32_bits

KAPPA = 8
LOCAL_K = 6
LOG2E = np.float32(1.4426950408889634)


def causal_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float):
    """``q [S, Hq, 128]``, ``k, v [S, Hkv, 128]`` fp32 -> ``(out [S, Hq, 128], lse [Hq, S], raw [Hq, S, S])``."""

    length, heads, _ = q.shape
    group = heads // k.shape[1]
    raw = np.empty((heads, length, length), dtype=np.float32)
    out = np.empty((length, heads, 128), dtype=np.float64)
    lse = np.empty((heads, length), dtype=np.float64)
    mask = np.tril(np.ones((length, length), dtype=bool))
    for head in range(heads):
        kv = head // group
        scores = q[:, head].astype(np.float64) @ k[:, kv].astype(np.float64).T
        raw[head] = scores.astype(np.float32)
        scaled = np.where(mask, scores * scale, -np.inf)
        top = scaled.max(axis=1, keepdims=True)
        weights = np.exp(scaled - top)
        total = weights.sum(axis=1, keepdims=True)
        out[:, head] = (weights / total) @ v[:, kv].astype(np.float64)
        lse[head] = (top + np.log(total))[:, 0]
    return out.astype(np.float32), lse.astype(np.float32), raw


def quantised_keys(raw: np.ndarray) -> np.ndarray:
    return np.clip(np.rint((raw.astype(np.float32) + np.float32(48.0)) * np.float32(256.0)), 0, 32767).astype(np.int64)


def reference_topk(raw: np.ndarray, lse: np.ndarray, scale: float, num_sink: int):
    """Top-8 edges of one query head by the reference's rule.

    ``raw [S, S]`` unscaled scores, ``lse [S]``.  Returns ``(val [S-skip, 8] fp32,
    idx [S-skip, 8] int32, key15 [S-skip, 8])``.
    """

    length = raw.shape[0]
    skip = num_sink + KAPPA - 1
    rows = max(0, length - skip)
    keys = quantised_keys(raw)
    val = np.zeros((rows, KAPPA), dtype=np.float32)
    idx = np.zeros((rows, KAPPA), dtype=np.int32)
    key_out = np.zeros((rows, KAPPA), dtype=np.int64)
    columns = np.arange(length)
    scale_log2 = np.float32(scale) * LOG2E
    for row in range(skip, length):
        eligible = columns[num_sink : row + 1]
        packed = (keys[row, eligible] << 17) | eligible
        pool = []
        for cls in range(4):
            members = packed[((eligible % 8) // 2) == cls]
            pool.append(np.sort(members)[::-1][:LOCAL_K])
        best = np.sort(np.concatenate(pool))[::-1][:KAPPA]
        key15 = best >> 17
        idx[row - skip] = (best & 0x1FFFF).astype(np.int32)
        key_out[row - skip] = key15
        dequant = key15.astype(np.float32) / np.float32(256.0) - np.float32(48.0)
        val[row - skip] = np.exp2(dequant * scale_log2 - np.float32(lse[row]) * LOG2E)
    return val, idx, key_out


def exact_edges(q: np.ndarray, k: np.ndarray, scale: float, num_sink: int, edges: int):
    """Exact top-``edges`` keys per KV head and row.

    Score of key ``j`` for row ``i``: ``max_h fp32(fixed_dot(q[i, h], k[j]) * scale)``
    over the heads of the group; rank by (score descending, index ascending) over
    ``num_sink <= j <= i``.  Returns ``(idx [Hkv, rows, edges] int32, score fp32)``.
    """

    length, heads, _ = q.shape
    kv_heads = k.shape[1]
    group = heads // kv_heads
    skip = num_sink + edges - 1
    rows = max(0, length - skip)
    idx = np.full((kv_heads, rows, edges), -1, dtype=np.int32)
    score = np.zeros((kv_heads, rows, edges), dtype=np.float32)
    scale32 = np.float32(scale)
    for kv in range(kv_heads):
        best = None
        for h in range(group):
            dots = fixed_dot(q[:, kv * group + h][:, None, :], k[:, kv][None, :, :])
            scaled = (dots * scale32).astype(np.float32)
            best = scaled if best is None else np.maximum(best, scaled)
        for row in range(skip, length):
            eligible = np.arange(num_sink, row + 1)
            packed = (ordered_f32_bits(best[row, eligible]).astype(np.uint64) << np.uint64(32)) | (
                np.uint64(0xFFFFFFFF) - eligible.astype(np.uint64)
            )
            top = np.sort(packed)[::-1][:edges]
            idx[kv, row - skip] = (np.uint64(0xFFFFFFFF) - (top & np.uint64(0xFFFFFFFF))).astype(np.int64)
            chosen = idx[kv, row - skip]
            score[kv, row - skip] = best[row, chosen]
    return idx, score

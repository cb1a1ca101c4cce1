"""Prefill attention that also emits the score graph's neighbour edges.

``prefill_attention_topk`` keeps the reference's call
(``community_kv/attention/flash_attention.py:23-51``): causal attention over
``[B, S, H, 128]`` bf16 tensors with grouped query heads, returning the
attention output, the log-sum-exp and, per query head and row, the eight
strongest keys by the reference's quantised-score rule
(``third_party/flash_attention/community-kv.patch``, ``hopper/topk_warpselect.h``).
``prefill_attention_edges`` is the exact variant: the top-``m`` keys per KV head
by the group maximum of the scaled scores, ties to the smaller index.  Both run
the tcgen05 kernel of ``csrc/prefill_topk.cu`` through ``ckv_prefill_topk``.
"""

from __future__ import annotations

import torch

from community_kv_b200 import native

HEAD_DIM = 128
TOPK = 8
EXACT_KEEP = 16


def _pack(query, key, value, *, softmax_scale, num_sink, mode, edges_per_row=0, exact_slack=0.0, status=None):
    if query.ndim != 4 or key.ndim != 4 or value.shape != key.shape:
        raise ValueError("query/key/value must have shape [B, S, H, 128]")
    if query.shape[-1] != HEAD_DIM or key.shape[-1] != HEAD_DIM:
        raise ValueError("head dimension must be 128")
    if query.shape[0] != key.shape[0] or query.shape[1] != key.shape[1]:
        raise ValueError("query and key must share batch and sequence length")
    if query.dtype != torch.bfloat16 or key.dtype != torch.bfloat16 or value.dtype != torch.bfloat16:
        raise TypeError("query, key and value must use BF16")
    if query.shape[2] % key.shape[2]:
        raise ValueError("query heads must divide evenly into KV-head groups")
    if num_sink < 0:
        raise ValueError("num_sink must be non-negative")
    if query.device.type != "cuda":
        raise RuntimeError("prefill attention runs only on CUDA tensors; there is no CPU path")
    if query.stride(-1) != 1:
        query = query.contiguous()
    if key.stride(-1) != 1:
        key = key.contiguous()
    if value.stride(-1) != 1:
        value = value.contiguous()
    batch, length, heads, _ = query.shape
    kv_heads = key.shape[2]
    device = query.device
    out = torch.empty((batch, length, heads, HEAD_DIM), dtype=torch.bfloat16, device=device)
    lse = torch.empty((batch, heads, length), dtype=torch.float32, device=device)
    if status is None:
        status = torch.zeros((1,), dtype=torch.int32, device=device)
    elif status.dtype != torch.int32 or status.numel() != 1 or status.device != device:
        raise ValueError("status must be a one-element int32 tensor on the inputs' device")
    args = native.PrefillArgs()
    native.fill(
        args,
        device=device.index or 0,
        batch=batch,
        seq_len=length,
        query_heads=heads,
        kv_heads=kv_heads,
        num_sink=num_sink,
        mode=mode,
        edges_per_row=edges_per_row,
        softmax_scale=float(softmax_scale),
        exact_slack=float(exact_slack),
        q_batch_stride=query.stride(0), q_row_stride=query.stride(1), q_head_stride=query.stride(2),
        k_batch_stride=key.stride(0), k_row_stride=key.stride(1), k_head_stride=key.stride(2),
        v_batch_stride=value.stride(0), v_row_stride=value.stride(1), v_head_stride=value.stride(2),
        o_batch_stride=out.stride(0), o_row_stride=out.stride(1), o_head_stride=out.stride(2),
        query=query.data_ptr(), key=key.data_ptr(), value=value.data_ptr(),
        output=out.data_ptr(), lse=lse.data_ptr(), status=status.data_ptr(),
    )
    return args, out, lse, status, (query, key, value)


def check_status(status: torch.Tensor) -> None:
    """Raise if a bounded wait inside the kernels ran out (the outputs are then invalid).

    Every entry point below checks its own status word after the launch, which synchronises
    with the stream.  A caller that wants to queue several calls without a host round trip
    passes its own ``status`` tensor (one int32, zero-initialised; the kernels OR their flags
    into it) and calls this function once at the end.  The check is skipped while the stream
    is being captured into a CUDA graph.
    """

    if torch.cuda.is_current_stream_capturing():
        return
    word = int(status.item())
    if word != 0:
        raise RuntimeError(
            f"prefill kernels reported device status {word:#x}: a bounded wait on a copy or "
            "tensor-core barrier ran out; the outputs of this call are invalid"
        )


def prefill_attention_topk(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    *,
    softmax_scale: float,
    num_sink: int = 10,
    status: torch.Tensor | None = None,
):
    """Causal grouped-query attention plus the reference's row-wise top-8 edges.

    Returns ``(out, lse, None, None, topk_val, topk_idx)`` with ``topk_val`` fp32 and
    ``topk_idx`` int32 of shape ``[B, Hq, S - (num_sink + 7), 8]`` (rows with fewer
    than eight eligible keys are omitted, as in the reference).
    """

    own_status = status is None
    rows = max(0, query.shape[1] - (num_sink + TOPK - 1)) if query.ndim == 4 else 0
    # a prompt with no row long enough for eight eligible keys: attention only, empty edge tensors
    args, out, lse, status, keep = _pack(
        query, key, value, softmax_scale=softmax_scale, num_sink=num_sink, mode=1 if rows else 0, status=status
    )
    batch, length, heads, _ = out.shape
    topk_val = torch.zeros((batch, heads, rows, TOPK), dtype=torch.float32, device=out.device)
    topk_idx = torch.zeros((batch, heads, rows, TOPK), dtype=torch.int32, device=out.device)
    if rows:
        args.topk_val = topk_val.data_ptr()
        args.topk_idx = topk_idx.data_ptr()
    native.call("ckv_prefill_topk", args, native.current_stream(out.device))
    if own_status:
        check_status(status)
    del keep
    return out, lse, None, None, topk_val, topk_idx


def prefill_attention_edges(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    *,
    softmax_scale: float,
    num_sink: int = 10,
    edges_per_row: int = 16,
    exact_slack: float = 1e-3,
    status: torch.Tensor | None = None,
):
    """Causal attention plus the exact top-``edges_per_row`` keys per KV head and row.

    The score of key ``j`` for row ``i`` is ``max over the query group of
    scale * (q_i . k_j)`` in fp32 (fixed summation order); keys are ranked by
    (score descending, index ascending) over ``num_sink <= j <= i``.  Returns
    ``(out, lse, edge_idx int32, edge_score fp32, rescanned)`` with edges of shape
    ``[B, Hkv, S - (num_sink + m - 1), m]``; ``rescanned`` counts the rows whose
    short list could not be proven complete and were re-ranked by a full scan.
    """

    if not 1 <= edges_per_row <= EXACT_KEEP:
        raise ValueError("edges_per_row must be in [1, 16]")
    own_status = status is None
    rows = max(0, query.shape[1] - (num_sink + edges_per_row - 1)) if query.ndim == 4 else 0
    # a prompt with no row long enough for `edges_per_row` eligible keys: attention only, empty edges
    args, out, lse, status, keep = _pack(
        query, key, value, softmax_scale=softmax_scale, num_sink=num_sink, mode=2 if rows else 0,
        edges_per_row=edges_per_row, exact_slack=exact_slack, status=status,
    )
    batch, length, heads, _ = out.shape
    kv_heads = keep[1].shape[2]
    group = heads // kv_heads
    device = out.device
    candidates = torch.zeros((batch, kv_heads, length, group, EXACT_KEEP + 1), dtype=torch.int64, device=device)
    edge_idx = torch.full((batch, kv_heads, rows, edges_per_row), -1, dtype=torch.int32, device=device)
    edge_score = torch.zeros((batch, kv_heads, rows, edges_per_row), dtype=torch.float32, device=device)
    flags = torch.zeros((batch, kv_heads, rows), dtype=torch.int32, device=device)
    rescan_list = torch.zeros((1 + batch * kv_heads * rows,), dtype=torch.int32, device=device)
    if rows:
        native.fill(
            args,
            candidates=candidates.data_ptr(),
            edge_idx=edge_idx.data_ptr(),
            edge_score=edge_score.data_ptr(),
            edge_flags=flags.data_ptr(),
            rescan_list=rescan_list.data_ptr(),
        )
    native.call("ckv_prefill_topk", args, native.current_stream(device))
    if own_status:
        check_status(status)
    del keep
    return out, lse, edge_idx, edge_score, flags


def prefill_attention(query, key, value, *, softmax_scale: float, status: torch.Tensor | None = None):
    """Causal grouped-query attention only: ``(out, lse)``."""

    own_status = status is None
    args, out, lse, status, keep = _pack(
        query, key, value, softmax_scale=softmax_scale, num_sink=0, mode=0, status=status
    )
    native.call("ckv_prefill_topk", args, native.current_stream(out.device))
    if own_status:
        check_status(status)
    del keep
    return out, lse


__all__ = ["check_status", "prefill_attention", "prefill_attention_edges", "prefill_attention_topk"]

"""Decode-path operators: same call signatures as the reference's kernel launchers.

``score_centroids``, ``select_weighted_descriptors_*``, ``score_and_select``
(reference ``community_kv/attention/kernels/centroid_selection.py:330-556``),
``segmented_attention`` / ``triton_segmented_attention``
(``segmented_attention.py:1016-1273``) and ``decode_layer``
(``community_kv/attention/decode.py:67-111``).  Each one validates its tensors
like the reference does and then makes exactly one call into the CUDA library.
Tensors may carry a leading batch axis (see ``community_kv_b200.state``).
"""

from __future__ import annotations

import os

import torch

from community_kv_b200 import native
from community_kv_b200.state import (
    ATTENTION_TILE,
    HEAD_DIM,
    CentroidSelectionWorkspace,
    DecodeDeltaChunks,
    DecodeLayerWorkspace,
    MutableGraphState,
    OnlineUpdateWorkspace,
    PackedSegments,
    PrefillCSR,
    SegmentedAttentionWorkspace,
)


def _require_cuda(*tensors: torch.Tensor) -> torch.device:
    device = tensors[0].device
    if device.type != "cuda":
        raise RuntimeError(
            "community_kv_b200 operators run only on CUDA tensors; there is no CPU path"
        )
    if any(tensor.device != device for tensor in tensors):
        raise ValueError("all operator tensors must share one device")
    return device


def _contiguous(name: str, tensor: torch.Tensor) -> torch.Tensor:
    if not tensor.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return tensor


def _score_args(
    args: native.LayerArgs,
    *,
    query: torch.Tensor,
    centroids: torch.Tensor,
    community_sizes: torch.Tensor,
    community_counts: torch.Tensor,
    workspace: CentroidSelectionWorkspace,
) -> None:
    batched = centroids.ndim == 4
    heads = workspace.kv_heads
    if query.ndim != (3 if batched else 2) or query.shape[-1] != HEAD_DIM or query.shape[-2] % heads:
        raise ValueError("query heads must divide into [KV head, group, 128]")
    group = query.shape[-2] // heads
    if not 1 <= group <= 16:
        raise ValueError("GQA group size must be in [1, 16]")
    lead = tuple(centroids.shape[:-3])
    if tuple(centroids.shape[-3:]) != (heads, workspace.community_capacity, HEAD_DIM) or tuple(
        workspace.scores.shape[:-2]
    ) != lead:
        raise ValueError("centroids have the wrong fixed capacity")
    if community_sizes.shape != centroids.shape[:-1]:
        raise ValueError("community_sizes must match centroid rows")
    if community_counts.shape != lead + (heads,):
        raise ValueError("community_counts must have one entry per KV head")
    if query.dtype != torch.bfloat16:
        raise TypeError("query must use BF16")
    if centroids.dtype not in (torch.float8_e4m3fn, torch.float32):
        raise TypeError("centroids must use FP8 E4M3 (the reference's layout) or FP32")
    if community_sizes.dtype != torch.int32:
        raise TypeError("community_sizes must use int32")
    if community_counts.dtype != torch.int32:
        raise TypeError("community_counts must use int32")
    native.fill(
        args,
        batch=lead[0] if lead else 1,
        retrieval_heads=heads,
        group_size=group,
        community_capacity=workspace.community_capacity,
        token_budget=workspace.token_budget,
        num_sink=workspace.num_sink,
        max_communities=workspace.max_communities,
        descriptor_capacity=workspace.communities.shape[-1],
        query=native.pointer(_contiguous("query", query)),
        centroids=native.pointer(_contiguous("centroids", centroids)),
        community_sizes=native.pointer(_contiguous("community_sizes", community_sizes)),
        community_counts=native.pointer(_contiguous("community_counts", community_counts)),
        score_cover=native.pointer(workspace.score_cover),
        scores=native.pointer(workspace.scores),
        communities=native.pointer(workspace.communities),
        cumulative_ends=native.pointer(workspace.cumulative_ends),
        descriptor_counts=native.pointer(workspace.descriptor_counts),
        tile_descriptors=native.pointer(workspace.tile_descriptors),
        threshold_state=native.pointer(workspace.native_threshold),
        positions=native.pointer(workspace.positions),
    )


def _graph_args(
    args: native.LayerArgs,
    *,
    csr: PrefillCSR,
    state: MutableGraphState,
    sink_positions: torch.Tensor,
    current_position: torch.Tensor,
) -> None:
    deltas = state.deltas
    if sink_positions.dtype != torch.int32 or current_position.dtype != torch.int32:
        raise TypeError("sink_positions and current_position must use int32")
    native.fill(
        args,
        graphs=state.graph_count,
        retrieval_heads=state.retrieval_head_count,
        community_capacity=state.community_capacity,
        token_capacity=state.token_communities.shape[-1],
        member_capacity=csr.member_positions.shape[-1],
        chunks_per_graph=deltas.chunk_capacity_per_graph,
        delta_position_capacity=deltas.position_capacity,
        sink_positions=native.pointer(sink_positions),
        retrieval_to_graph=native.pointer(state.retrieval_to_graph),
        retrieval_to_kv=native.pointer(state.retrieval_to_kv),
        member_offsets=native.pointer(_contiguous("member_offsets", csr.member_offsets)),
        member_positions=native.pointer(_contiguous("member_positions", csr.member_positions)),
        centroids=native.pointer(state.centroids),
        community_sizes=native.pointer(state.community_sizes),
        community_counts=native.pointer(state.community_counts),
        community_weight=native.pointer(state.community_weight),
        total_weight=native.pointer(state.total_weight),
        token_communities=native.pointer(state.token_communities),
        current_position=native.pointer(current_position),
        delta_positions=native.pointer(deltas.positions),
        chunk_start=native.pointer(deltas.chunk_start),
        chunk_capacity=native.pointer(deltas.chunk_capacity),
        chunk_size=native.pointer(deltas.chunk_size),
        chunk_next=native.pointer(deltas.chunk_next),
        chunk_previous=native.pointer(deltas.chunk_previous),
        community_head=native.pointer(deltas.community_head),
        community_tail=native.pointer(deltas.community_tail),
        delta_sizes=native.pointer(deltas.community_sizes),
        next_free_chunk=native.pointer(deltas.next_free_chunk),
        next_free_position=native.pointer(deltas.next_free_position),
    )


def _attention_args(
    args: native.LayerArgs,
    *,
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    softmax_scale: float,
    lam: float,
    workspace: SegmentedAttentionWorkspace,
    update: OnlineUpdateWorkspace | None,
    token_budget: int,
) -> None:
    batched = key.ndim == 4
    if key.ndim not in (3, 4) or value.shape != key.shape or key.shape[-1] != HEAD_DIM:
        raise ValueError("key and value must have shape [Hkv, S, 128]")
    if query.dtype != torch.bfloat16 or key.dtype != query.dtype or value.dtype != query.dtype:
        raise TypeError("query, key, and value must use BF16")
    if token_budget % ATTENTION_TILE:
        raise ValueError("token budget must be a multiple of 64")
    if key.stride(-1) != 1 or value.stride(-1) != 1:
        raise ValueError("key and value rows must be contiguous")
    if not 0.0 <= lam <= 1.0:
        raise ValueError("update_lam must be in [0, 1]")
    native.fill(
        args,
        group_size=workspace.group_size,
        splits=workspace.splits,
        token_budget=token_budget,
        sequence_capacity=key.shape[-2],
        softmax_scale=float(softmax_scale),
        lam=float(lam),
        key=native.pointer(key),
        value=native.pointer(value),
        key_batch_stride=key.stride(0) if batched else 0,
        key_head_stride=key.stride(-3),
        key_row_stride=key.stride(-2),
        value_batch_stride=value.stride(0) if batched else 0,
        value_head_stride=value.stride(-3),
        value_row_stride=value.stride(-2),
        query=native.pointer(_contiguous("query", query)),
        partials=native.pointer(workspace.partials),
        partial_topk=native.pointer(workspace.partial_topk_packed),
        output=native.pointer(workspace.output),
        lse=native.pointer(workspace.lse),
        topk_scores=native.pointer(workspace.topk_scores),
        topk_positions=native.pointer(workspace.topk_positions),
        status=native.pointer(workspace.status),
        flags=(0 if update is not None else native.FLAG_SKIP_UPDATE) | _layout_flags(),
        assigned=native.pointer(update.assigned_communities) if update is not None else None,
        overflow=native.pointer(update.overflow) if update is not None else None,
    )


def score_centroids(
    *,
    query: torch.Tensor,
    centroids: torch.Tensor,
    community_sizes: torch.Tensor,
    community_counts: torch.Tensor,
    workspace: CentroidSelectionWorkspace,
    exact: bool = False,
) -> torch.Tensor:
    """Score each contiguous query group against its centroid table (fp16 out).

    ``exact``: use the fixed-order CUDA-core sum for this call whatever the process-wide
    switch says (a CPU can reproduce it bit for bit).
    """

    args = native.LayerArgs()
    _score_args(
        args,
        query=query,
        centroids=centroids,
        community_sizes=community_sizes,
        community_counts=community_counts,
        workspace=workspace,
    )
    device = _require_cuda(query, centroids, community_sizes, community_counts, workspace.scores)
    # identity mappings are not read by the scoring kernel beyond make_unit()
    mapping = torch.arange(workspace.kv_heads, dtype=torch.int32, device=device)
    native.fill(
        args,
        device=device.index or 0,
        graphs=workspace.kv_heads,
        retrieval_to_graph=native.pointer(mapping),
        retrieval_to_kv=native.pointer(mapping),
        flags=(_layout_flags() & ~(native.FLAG_TENSOR_SCORES if exact else 0)) | _centroid_flag(centroids),
    )
    native.call("ckv_score_centroids", args, native.current_stream(device))
    return workspace.scores


def _select(
    *,
    community_sizes: torch.Tensor,
    community_counts: torch.Tensor,
    workspace: CentroidSelectionWorkspace,
    csr: PrefillCSR,
    state: MutableGraphState,
    sink_positions: torch.Tensor,
    current_position: torch.Tensor,
) -> PackedSegments:
    if community_sizes.shape != workspace.scores.shape:
        raise ValueError("community_sizes must match the score capacity")
    if community_sizes.dtype != torch.int32:
        raise TypeError("community_sizes must use int32")
    if community_counts.shape != workspace.scores.shape[:-1]:
        raise ValueError("community_counts must have one entry per KV head")
    if community_counts.dtype != torch.int32:
        raise TypeError("community_counts must use int32")
    device = _require_cuda(workspace.scores, community_sizes, community_counts)
    args = native.LayerArgs()
    _graph_args(
        args, csr=csr, state=state, sink_positions=sink_positions, current_position=current_position
    )
    native.fill(
        args,
        device=device.index or 0,
        batch=workspace.batch or 1,
        group_size=1,
        token_budget=workspace.token_budget,
        num_sink=workspace.num_sink,
        max_communities=workspace.max_communities,
        descriptor_capacity=workspace.communities.shape[-1],
        community_sizes=native.pointer(community_sizes),
        community_counts=native.pointer(community_counts),
        scores=native.pointer(workspace.scores),
        communities=native.pointer(workspace.communities),
        cumulative_ends=native.pointer(workspace.cumulative_ends),
        descriptor_counts=native.pointer(workspace.descriptor_counts),
        tile_descriptors=native.pointer(workspace.tile_descriptors),
        threshold_state=native.pointer(workspace.native_threshold),
        positions=native.pointer(workspace.positions),
    )
    native.call("ckv_select_descriptors", args, native.current_stream(device))
    return workspace.packed_segments()


def select_weighted_descriptors_native(**kwargs) -> PackedSegments:
    """Exact budgeted selection from the fp16 scores already in the workspace.

    Besides the reference's ``community_sizes``, ``community_counts`` and
    ``workspace`` it needs ``csr``, ``state``, ``sink_positions`` and
    ``current_position`` because the same kernel also resolves the selected
    members to cache rows.
    """

    return _select(**kwargs)


select_weighted_descriptors_cluster = select_weighted_descriptors_native
select_weighted_descriptors_auto = select_weighted_descriptors_native


def score_and_select(
    *,
    query: torch.Tensor,
    centroids: torch.Tensor,
    community_sizes: torch.Tensor,
    community_counts: torch.Tensor,
    workspace: CentroidSelectionWorkspace,
    csr: PrefillCSR,
    state: MutableGraphState,
    sink_positions: torch.Tensor,
    current_position: torch.Tensor,
) -> PackedSegments:
    score_centroids(
        query=query,
        centroids=centroids,
        community_sizes=community_sizes,
        community_counts=community_counts,
        workspace=workspace,
    )
    return _select(
        community_sizes=community_sizes,
        community_counts=community_counts,
        workspace=workspace,
        csr=csr,
        state=state,
        sink_positions=sink_positions,
        current_position=current_position,
    )


def _check_update(state: MutableGraphState, deltas: DecodeDeltaChunks, csr: PrefillCSR) -> None:
    if state.deltas is not deltas:
        raise ValueError("fused update must mutate the attention delta store")
    if deltas.community_capacity != csr.community_capacity:
        raise ValueError("delta chunks must match CSR community capacity")
    if state.head_dim != HEAD_DIM:
        raise ValueError("update state must use head_dim=128")


def segmented_attention(
    *,
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    csr: PrefillCSR,
    deltas: DecodeDeltaChunks,
    segments: PackedSegments,
    sink_positions: torch.Tensor,
    current_position: torch.Tensor,
    softmax_scale: float,
    workspace: SegmentedAttentionWorkspace,
    update_state: MutableGraphState,
    update_workspace: OnlineUpdateWorkspace | None,
    update_lam: float,
    positions: torch.Tensor | None = None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Gather the selected members' K/V rows and run exact split attention.

    ``update_workspace=None`` skips the online assignment (attention only).
    Returns ``(output, lse, topk_scores, topk_positions)``, aliases of the
    workspace tensors.
    """

    _check_update(update_state, deltas, csr)
    device = _require_cuda(query, key, value, segments.communities)
    heads = update_state.retrieval_head_count
    if query.shape[-2:] != (heads * workspace.group_size, HEAD_DIM):
        raise ValueError(
            f"query must have {workspace.group_size} [128] heads per retrieval head"
        )
    if positions is None:
        positions = torch.empty(
            segments.communities.shape[:-1] + (segments.token_budget,),
            dtype=torch.int32,
            device=device,
        )
    args = native.LayerArgs()
    _graph_args(
        args,
        csr=csr,
        state=update_state,
        sink_positions=sink_positions,
        current_position=current_position,
    )
    _attention_args(
        args,
        query=query,
        key=key,
        value=value,
        softmax_scale=softmax_scale,
        lam=update_lam,
        workspace=workspace,
        update=update_workspace,
        token_budget=segments.token_budget,
    )
    native.fill(
        args,
        device=device.index or 0,
        batch=key.shape[0] if key.ndim == 4 else 1,
        num_sink=segments.num_sink,
        descriptor_capacity=segments.communities.shape[-1],
        communities=native.pointer(segments.communities),
        cumulative_ends=native.pointer(segments.cumulative_ends),
        descriptor_counts=native.pointer(segments.descriptor_counts),
        tile_descriptors=native.pointer(segments.tile_descriptors),
        positions=native.pointer(positions),
    )
    native.call("ckv_segmented_attention", args, native.current_stream(device))
    return workspace.output, workspace.lse, workspace.topk_scores, workspace.topk_positions


triton_segmented_attention = segmented_attention


def segmented_attention_static(
    *,
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    csr: PrefillCSR,
    deltas: DecodeDeltaChunks,
    segments: PackedSegments,
    sink_positions: torch.Tensor,
    current_position: torch.Tensor,
    softmax_scale: float,
    workspace: SegmentedAttentionWorkspace,
    update_state: MutableGraphState,
    update_workspace: OnlineUpdateWorkspace | None,
    update_lam: float,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """``segmented_attention`` for hosts that must not allocate device memory.

    Meant for callers that live inside a fixed memory budget - a serving process
    whose pool is fully handed out, a plug-in running in memory it does not own -
    and therefore cannot provide (or let this package provide) scratch tensors.
    Only the outputs of ``workspace`` are used; the row positions, split partials
    and candidate lists stay in a fixed array inside the CUDA library.  Limits:
    at most 64 (sequence, head) units, budget 4096, 8 splits, group size 8
    (``NativeError`` beyond).  Calls share that one array, so two calls that may
    overlap on the GPU race; the first call on a device should come before any
    stream capture.  Results are identical to ``segmented_attention``.
    """

    _check_update(update_state, deltas, csr)
    device = _require_cuda(query, key, value, segments.communities)
    heads = update_state.retrieval_head_count
    if query.shape[-2:] != (heads * workspace.group_size, HEAD_DIM):
        raise ValueError(
            f"query must have {workspace.group_size} [128] heads per retrieval head"
        )
    args = native.LayerArgs()
    _graph_args(
        args,
        csr=csr,
        state=update_state,
        sink_positions=sink_positions,
        current_position=current_position,
    )
    _attention_args(
        args,
        query=query,
        key=key,
        value=value,
        softmax_scale=softmax_scale,
        lam=update_lam,
        workspace=workspace,
        update=update_workspace,
        token_budget=segments.token_budget,
    )
    native.fill(
        args,
        device=device.index or 0,
        batch=key.shape[0] if key.ndim == 4 else 1,
        num_sink=segments.num_sink,
        descriptor_capacity=segments.communities.shape[-1],
        communities=native.pointer(segments.communities),
        cumulative_ends=native.pointer(segments.cumulative_ends),
        descriptor_counts=native.pointer(segments.descriptor_counts),
        tile_descriptors=native.pointer(segments.tile_descriptors),
        positions=None,
        partials=None,
        partial_topk=None,
    )
    native.call("ckv_segmented_attention_static", args, native.current_stream(device))
    return workspace.output, workspace.lse, workspace.topk_scores, workspace.topk_positions


def tensor_scores_enabled() -> bool:
    """Centroid scoring on the tensor cores (the default); ``CKV_TENSOR_SCORES=0`` selects the
    fixed-order CUDA-core sum, which a CPU can reproduce bit for bit."""

    return os.environ.get("CKV_TENSOR_SCORES", "1") != "0"


def _centroid_flag(centroids: torch.Tensor) -> int:
    """An fp32 centroid table (not the reference's layout) is announced to the kernels by a flag."""

    return native.FLAG_FP32_CENTROIDS if centroids.dtype == torch.float32 else 0


def _layout_flags() -> int:
    """Process-wide switches read from the environment.

    ``CKV_TENSOR_SCORES=0``: score the centroids on the CUDA cores in one fixed summation
    order instead of on the tensor cores (``mma.m16n8k16``, which is also what the
    reference's ``tl.dot`` compiles to; the two may differ in a score's last fp16 bit).
    ``CKV_UNFUSED=1`` selects the four stand-alone kernels for ``ckv_decode_layer``
    instead of the single cluster launch (same results; a debugging and A/B-timing
    switch).  ``CKV_REFERENCE_DIVISION=1`` makes the running centroid mean divide like
    the reference's compiled Triton kernel (approximate ``div.full.f32``) instead of
    like its CPU test helper (IEEE division): the stored e4m3 centroid then matches the
    reference kernel bit for bit also when the exact quotient is a rounding tie.
    """

    flags = native.FLAG_UNFUSED if os.environ.get("CKV_UNFUSED") == "1" else 0
    if os.environ.get("CKV_REFERENCE_DIVISION") == "1":
        flags |= native.FLAG_REFERENCE_DIVISION
    if tensor_scores_enabled():
        flags |= native.FLAG_TENSOR_SCORES
    return flags


def build_layer_args(
    *,
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    csr: PrefillCSR,
    state: MutableGraphState,
    sink_positions: torch.Tensor,
    current_position: torch.Tensor,
    softmax_scale: float,
    lam: float,
    workspace: DecodeLayerWorkspace,
) -> native.LayerArgs:
    """Validate one layer's tensors and pack them for ``ckv_decode_layer``."""

    device = _require_cuda(query, key, value, state.centroids)
    _check_update(state, state.deltas, csr)
    args = native.LayerArgs()
    _score_args(
        args,
        query=query,
        centroids=state.centroids,
        community_sizes=state.community_sizes,
        community_counts=state.community_counts,
        workspace=workspace.selection,
    )
    _graph_args(
        args, csr=csr, state=state, sink_positions=sink_positions, current_position=current_position
    )
    _attention_args(
        args,
        query=query,
        key=key,
        value=value,
        softmax_scale=softmax_scale,
        lam=lam,
        workspace=workspace.attention,
        update=workspace.update,
        token_budget=workspace.selection.token_budget,
    )
    native.fill(args, device=device.index or 0)
    args.flags |= _centroid_flag(state.centroids)
    return args


def decode_layer(
    *,
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    csr: PrefillCSR,
    state: MutableGraphState,
    sink_positions: torch.Tensor,
    current_position: torch.Tensor,
    softmax_scale: float,
    lam: float,
    workspace: DecodeLayerWorkspace,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Run one complete layer transition: score, select, attend, assign."""

    args = build_layer_args(
        query=query,
        key=key,
        value=value,
        csr=csr,
        state=state,
        sink_positions=sink_positions,
        current_position=current_position,
        softmax_scale=softmax_scale,
        lam=lam,
        workspace=workspace,
    )
    native.call("ckv_decode_layer", args, native.current_stream(query.device))
    attention = workspace.attention
    return (
        attention.output,
        attention.lse,
        attention.topk_scores,
        attention.topk_positions,
        workspace.update.assigned_communities,
    )


class DeferredUpdate:
    """Runs the online graph update of a layer beside whatever follows its attention.

    Nothing downstream of a layer's attention output depends on that layer's online
    assignment (labels, sizes, centroid, delta chains): only the SAME layer's next decode
    step does.  ``launch`` therefore enqueues the layer's attention
    (``ckv_decode_layer`` with ``CKV_FLAG_SKIP_UPDATE``: scores, selection, attention,
    merged outputs, log-sum-exp and the eight neighbour candidates) on the caller's
    stream and the assignment (``ckv_online_update``) on a second stream, ordered after
    the attention by an event; the returned event marks the update as done and must be
    handed back as ``pending`` for the layer's next step.  Results are identical to the
    single call.  The split also works under CUDA-graph stream capture, where it becomes
    a side branch of the graph.
    """

    def __init__(self, device: torch.device) -> None:
        self.stream = torch.cuda.Stream(device)

    def launch(
        self,
        args: native.LayerArgs,
        *,
        pending: "torch.cuda.Event | None" = None,
    ) -> "torch.cuda.Event":
        device = self.stream.device
        main = torch.cuda.current_stream(device)
        if pending is not None:
            main.wait_event(pending)
        attend = native.LayerArgs.from_buffer_copy(args)
        attend.flags |= native.FLAG_SKIP_UPDATE
        native.call("ckv_decode_layer", attend, main.cuda_stream)
        attended = torch.cuda.Event()
        attended.record(main)
        self.stream.wait_event(attended)
        update = native.LayerArgs.from_buffer_copy(args)
        update.peer_count = 0          # the head outputs were already stored by the attention call
        update.peer_wait_flag = None
        native.call("ckv_online_update", update, self.stream.cuda_stream)
        done = torch.cuda.Event()
        done.record(self.stream)
        return done

    def synchronize(self) -> None:
        self.stream.synchronize()


def append_kv(
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    new_key: torch.Tensor,
    new_value: torch.Tensor,
    row: int | torch.Tensor,
) -> None:
    """``cache[..., row, :] = new[..., :]`` for both caches in one small launch.

    The caches are bf16 ``[..., rows, 128]`` (contiguous), the new rows bf16 ``[..., 128]``
    with the same leading shape; ``row`` is one index for all of them, an int32 tensor
    with one element (a device-side cursor shared by all of them, read by the kernel: no
    host round trip), or an int32 tensor with one index per leading entry (negative: skip).
    """

    if key_cache.shape != value_cache.shape or new_key.shape != new_value.shape:
        raise ValueError("key and value must have the same shapes")
    if key_cache.shape[-1] != HEAD_DIM or tuple(key_cache.shape[:-2]) != tuple(new_key.shape[:-1]):
        raise ValueError("caches must be [..., rows, 128] and the new rows [..., 128]")
    if not (key_cache.is_contiguous() and value_cache.is_contiguous()):
        raise ValueError("the caches must be contiguous")
    if key_cache.dtype != torch.bfloat16 or new_key.dtype != torch.bfloat16:
        raise TypeError("caches and new rows must use BF16")
    device = _require_cuda(key_cache, value_cache, new_key, new_value)
    units = new_key.numel() // HEAD_DIM
    index = None
    stride = 0
    if isinstance(row, torch.Tensor):
        if row.dtype != torch.int32 or row.numel() not in (1, units) or row.device != device:
            raise ValueError("row must be an int32 device tensor with one entry, or one per cache row to write")
        index = row.contiguous()
        stride = 0 if row.numel() == 1 else 1
    elif not 0 <= int(row) < key_cache.shape[-2]:
        raise ValueError("row is outside the cache")
    keep = (new_key.contiguous(), new_value.contiguous())
    status = native.library().ckv_append_kv(
        key_cache.data_ptr(), value_cache.data_ptr(), keep[0].data_ptr(), keep[1].data_ptr(), units,
        key_cache.shape[-2] * HEAD_DIM, native.pointer(index), stride, 0 if index is not None else int(row),
        native.current_stream(device),
    )
    if status:
        raise native.NativeError(native.library().ckv_status_string(status).decode())


__all__ = [
    "DeferredUpdate",
    "append_kv",
    "build_layer_args",
    "decode_layer",
    "score_and_select",
    "score_centroids",
    "segmented_attention",
    "segmented_attention_static",
    "select_weighted_descriptors_auto",
    "select_weighted_descriptors_cluster",
    "select_weighted_descriptors_native",
    "tensor_scores_enabled",
    "triton_segmented_attention",
]

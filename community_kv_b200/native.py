"""ctypes binding of ``libckv_b200.so`` (the C ABI declared in ``include/ckv_b200.h``).

There is no fallback: if the library is missing or an entry point reports an
error the call raises.  The library is built in-tree by
``community_kv_b200.build``.
"""

from __future__ import annotations

import ctypes
import functools
from typing import Any

import torch

from community_kv_b200.build import LIBRARY_PATH

_i32 = ctypes.c_int32
_i64 = ctypes.c_int64
_f32 = ctypes.c_float
_ptr = ctypes.c_void_p


MAX_PEERS = 7  # CKV_MAX_PEERS


class LayerArgs(ctypes.Structure):
    """Field-for-field mirror of ``struct ckv_layer_args``."""

    _fields_ = [
        ("device", _i32),
        ("batch", _i32),
        ("retrieval_heads", _i32),
        ("graphs", _i32),
        ("group_size", _i32),
        ("community_capacity", _i32),
        ("token_budget", _i32),
        ("num_sink", _i32),
        ("sequence_capacity", _i32),
        ("token_capacity", _i32),
        ("member_capacity", _i32),
        ("chunks_per_graph", _i32),
        ("delta_position_capacity", _i32),
        ("descriptor_capacity", _i32),
        ("max_communities", _i32),
        ("splits", _i32),
        ("flags", _i32),
        ("softmax_scale", _f32),
        ("lam", _f32),
        ("key_batch_stride", _i64),
        ("key_head_stride", _i64),
        ("key_row_stride", _i64),
        ("value_batch_stride", _i64),
        ("value_head_stride", _i64),
        ("value_row_stride", _i64),
        ("key", _ptr),
        ("value", _ptr),
        ("query", _ptr),
        ("sink_positions", _ptr),
        ("retrieval_to_graph", _ptr),
        ("retrieval_to_kv", _ptr),
        ("score_cover", _ptr),
        ("member_offsets", _ptr),
        ("member_positions", _ptr),
        ("centroids", _ptr),
        ("community_sizes", _ptr),
        ("community_counts", _ptr),
        ("community_weight", _ptr),
        ("total_weight", _ptr),
        ("token_communities", _ptr),
        ("current_position", _ptr),
        ("delta_positions", _ptr),
        ("chunk_start", _ptr),
        ("chunk_capacity", _ptr),
        ("chunk_size", _ptr),
        ("chunk_next", _ptr),
        ("chunk_previous", _ptr),
        ("community_head", _ptr),
        ("community_tail", _ptr),
        ("delta_sizes", _ptr),
        ("next_free_chunk", _ptr),
        ("next_free_position", _ptr),
        ("scores", _ptr),
        ("communities", _ptr),
        ("cumulative_ends", _ptr),
        ("descriptor_counts", _ptr),
        ("tile_descriptors", _ptr),
        ("threshold_state", _ptr),
        ("positions", _ptr),
        ("partials", _ptr),
        ("partial_topk", _ptr),
        ("output", _ptr),
        ("lse", _ptr),
        ("topk_scores", _ptr),
        ("topk_positions", _ptr),
        ("assigned", _ptr),
        ("overflow", _ptr),
        ("status", _ptr),
        ("kv_row_begin", _i32),
        ("kv_row_count", _i32),
        ("merged", _ptr),
        ("current_key", _ptr),
        ("peer_count", _i32),
        ("peer_wait_expected", _i32),
        ("peer_output", _ptr * MAX_PEERS),
        ("peer_flag", _ptr * MAX_PEERS),
        ("peer_done", _ptr),
        ("peer_wait_flag", _ptr),
        ("phase_times", _ptr),
        ("partial_unit_stride", _i64),
        ("partial_split_stride", _i64),
        ("topk_unit_stride", _i64),
        ("topk_split_stride", _i64),
        ("merged_topk", _ptr),
        ("forced_community", _ptr),
    ]


class PrefillArgs(ctypes.Structure):
    """Field-for-field mirror of ``struct ckv_prefill_args``."""

    _fields_ = [
        ("device", _i32),
        ("batch", _i32),
        ("seq_len", _i32),
        ("query_heads", _i32),
        ("kv_heads", _i32),
        ("num_sink", _i32),
        ("mode", _i32),
        ("edges_per_row", _i32),
        ("softmax_scale", _f32),
        ("exact_slack", _f32),
        ("q_batch_stride", _i64),
        ("q_row_stride", _i64),
        ("q_head_stride", _i64),
        ("k_batch_stride", _i64),
        ("k_row_stride", _i64),
        ("k_head_stride", _i64),
        ("v_batch_stride", _i64),
        ("v_row_stride", _i64),
        ("v_head_stride", _i64),
        ("o_batch_stride", _i64),
        ("o_row_stride", _i64),
        ("o_head_stride", _i64),
        ("query", _ptr),
        ("key", _ptr),
        ("value", _ptr),
        ("output", _ptr),
        ("lse", _ptr),
        ("topk_val", _ptr),
        ("topk_idx", _ptr),
        ("candidates", _ptr),
        ("edge_idx", _ptr),
        ("edge_score", _ptr),
        ("edge_flags", _ptr),
        ("status", _ptr),
        ("rescan_list", _ptr),
    ]


FLAG_SKIP_UPDATE = 1
STATIC_MAX_UNITS = 64
STATIC_MAX_BUDGET = 4096
STATIC_MAX_SPLITS = 8
STATIC_MAX_GROUP = 8
FLAG_ATTENTION_ONLY = 2
FLAG_UPDATE_ONLY = 4
# ckv_decode_layer: four stand-alone kernels instead of the single cluster launch
FLAG_UNFUSED = 8
FLAG_FP32_CENTROIDS = 64  # the centroid table is fp32 instead of e4m3 (four stand-alone kernels)
FLAG_TENSOR_SCORES = 32  # centroid scoring with mma.sync instead of the fixed CUDA-core order
FLAG_REFERENCE_DIVISION = 16  # centroid mean with the reference kernel's approximate division
DEV_WAIT_TIMEOUT = 1
PARTIAL_STRIDE = 132

ENTRY_POINTS = (
    "ckv_version",
    "ckv_status_string",
    "ckv_score_centroids",
    "ckv_select_descriptors",
    "ckv_segmented_attention",
    "ckv_decode_layer",
    "ckv_decode_layer_kernels",
    "ckv_attention_smem_bytes",
    "ckv_segmented_attention_static",
    "ckv_prefill_topk",
    "ckv_online_update",
    "ckv_wait_peers",
    "ckv_nearest_centroid",
    "ckv_append_kv",
    "ckv_merge_partials",
    "ckv_assemble_member_csr",
    "ckv_assemble_centroids",
    "ckv_assemble_modularity",
    "ckv_adjacency_raw_edges",
    "ckv_adjacency_scratch_bytes",
    "ckv_build_adjacency",
)


class NativeError(RuntimeError):
    """An entry point of the CUDA library returned a negative status."""


@functools.cache
def library() -> ctypes.CDLL:
    if not LIBRARY_PATH.exists():
        raise ImportError(
            f"{LIBRARY_PATH} is missing: build it with `python -m community_kv_b200.build`; "
            "this package has no CPU or framework fallback"
        )
    lib = ctypes.CDLL(str(LIBRARY_PATH))
    lib.ckv_version.restype = ctypes.c_int
    lib.ckv_status_string.restype = ctypes.c_char_p
    lib.ckv_status_string.argtypes = [ctypes.c_int]
    lib.ckv_attention_smem_bytes.restype = ctypes.c_int
    lib.ckv_attention_smem_bytes.argtypes = [ctypes.c_int]
    for name in (
        "ckv_score_centroids",
        "ckv_select_descriptors",
        "ckv_segmented_attention",
        "ckv_decode_layer",
        "ckv_segmented_attention_static",
        "ckv_online_update",
    ):
        function = getattr(lib, name)
        function.restype = ctypes.c_int
        function.argtypes = [ctypes.POINTER(LayerArgs), ctypes.c_void_p]
    lib.ckv_decode_layer_kernels.restype = ctypes.c_int
    lib.ckv_decode_layer_kernels.argtypes = [ctypes.POINTER(LayerArgs)]
    lib.ckv_append_kv.restype = ctypes.c_int
    lib.ckv_append_kv.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p,
                                  ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p]
    _p, _i, _l = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64
    lib.ckv_assemble_member_csr.restype = ctypes.c_int
    lib.ckv_assemble_member_csr.argtypes = [_p, _i, _i, _i, _i, _p, _p, _p, _i, _p]
    lib.ckv_assemble_centroids.restype = ctypes.c_int
    lib.ckv_assemble_centroids.argtypes = [_p, _p, _i, _i, _p, _l, _l, _p, _p, _i, _i, _i, _p, _p, _p]
    lib.ckv_assemble_modularity.restype = ctypes.c_int
    lib.ckv_assemble_modularity.argtypes = [_p, _i, _i, _p, _p, _p, _l, _i, _p, _p, _p]
    for name in ("ckv_adjacency_raw_edges", "ckv_adjacency_scratch_bytes"):
        getattr(lib, name).restype = ctypes.c_int64
        getattr(lib, name).argtypes = [_l, _l, _i, ctypes.c_double]
    lib.ckv_build_adjacency.restype = ctypes.c_int
    lib.ckv_build_adjacency.argtypes = [_p, _p, _p, _i, _l, _i, _i, ctypes.c_double, _p, _p, _p, _l, _p, _p, _l, _p]
    lib.ckv_nearest_centroid.restype = ctypes.c_int
    lib.ckv_nearest_centroid.argtypes = [ctypes.POINTER(LayerArgs), ctypes.c_void_p, ctypes.c_void_p]
    lib.ckv_wait_peers.restype = ctypes.c_int
    lib.ckv_wait_peers.argtypes = [ctypes.c_void_p, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p]
    lib.ckv_prefill_topk.restype = ctypes.c_int
    lib.ckv_prefill_topk.argtypes = [ctypes.POINTER(PrefillArgs), ctypes.c_void_p]
    return lib


def pointer(tensor: torch.Tensor | None) -> int | None:
    if tensor is None:
        return None
    return tensor.data_ptr()


def current_stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def call(name: str, args: ctypes.Structure, stream: int) -> None:
    status = getattr(library(), name)(ctypes.byref(args), ctypes.c_void_p(stream))
    if status != 0:
        message = library().ckv_status_string(status).decode()
        raise NativeError(f"{name} failed with status {status}: {message}")


def fill(args: ctypes.Structure, **values: Any) -> ctypes.Structure:
    for key, value in values.items():
        setattr(args, key, value)
    return args


__all__ = [
    "DEV_WAIT_TIMEOUT",
    "ENTRY_POINTS",
    "FLAG_ATTENTION_ONLY",
    "FLAG_SKIP_UPDATE",
    "FLAG_REFERENCE_DIVISION",
    "FLAG_TENSOR_SCORES",
    "FLAG_FP32_CENTROIDS",
    "FLAG_UNFUSED",
    "FLAG_UPDATE_ONLY",
    "LayerArgs",
    "MAX_PEERS",
    "NativeError",
    "PARTIAL_STRIDE",
    "PrefillArgs",
    "call",
    "current_stream",
    "fill",
    "library",
    "pointer",
]

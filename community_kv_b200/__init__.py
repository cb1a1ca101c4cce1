"""B200-native CommunityKV sparse-decode hot path behind the reference's API."""

from community_kv_b200.adapter import (
    ATTENTION_IMPLEMENTATION,
    CommunityKVAttention,
    HuggingFaceAttention,
)
from community_kv_b200.config import CommunityKVConfig, GraphAggregation, PartitionConfig
from community_kv_b200.ops import (
    decode_layer,
    score_and_select,
    score_centroids,
    segmented_attention,
    triton_segmented_attention,
)
from community_kv_b200.runtime import CommunityKVRuntime, DecodeRuntime, convert_prefill_tensors
from community_kv_b200.state import (
    DecodeDeltaChunks,
    DecodeLayerWorkspace,
    MutableGraphState,
    PackedSegments,
    PrefillCSR,
)

__all__ = [
    "ATTENTION_IMPLEMENTATION",
    "CommunityKVAttention",
    "CommunityKVConfig",
    "CommunityKVRuntime",
    "DecodeDeltaChunks",
    "DecodeLayerWorkspace",
    "DecodeRuntime",
    "GraphAggregation",
    "HuggingFaceAttention",
    "MutableGraphState",
    "PackedSegments",
    "PartitionConfig",
    "PrefillCSR",
    "convert_prefill_tensors",
    "decode_layer",
    "score_and_select",
    "score_centroids",
    "segmented_attention",
    "triton_segmented_attention",
]


def __getattr__(name: str):
    # The cache classes import transformers; load them on first use only.
    if name in ("StaticCache", "StaticCacheLayer"):
        from community_kv_b200 import cache

        return getattr(cache, name)
    if name == "prefill_attention_topk":
        from community_kv_b200.prefill import prefill_attention_topk

        return prefill_attention_topk
    raise AttributeError(name)

"""Public configuration objects, same names and meaning as the reference's.

Mirrors ``community_kv/config.py:9-70`` of the reference project: how query-head
edge lists are aggregated into graphs, the per-request decode settings, and the
prefill partition scheduling settings.
"""

from __future__ import annotations

import enum
from dataclasses import dataclass


class GraphAggregation(str, enum.Enum):
    """Which query heads share one token graph."""

    PER_QUERY_HEAD = "per_query_head"
    QUERY_GROUP = "query_group"
    LAYER_WISE = "layer_wise"

    def graph_count(self, *, query_heads: int, kv_heads: int) -> int:
        if min(query_heads, kv_heads) <= 0 or query_heads % kv_heads != 0:
            raise ValueError("query heads must divide evenly into KV-head groups")
        return {
            GraphAggregation.PER_QUERY_HEAD: query_heads,
            GraphAggregation.QUERY_GROUP: kv_heads,
            GraphAggregation.LAYER_WISE: 1,
        }[self]

    def retrieval_head_count(self, *, query_heads: int, kv_heads: int) -> int:
        graphs = self.graph_count(query_heads=query_heads, kv_heads=kv_heads)
        return graphs if graphs > kv_heads else kv_heads


@dataclass(frozen=True, slots=True)
class CommunityKVConfig:
    """Settings that stay fixed for the lifetime of one request."""

    token_budget: int = 4096
    num_sink: int = 10
    lam: float = 0.5
    aggregation: GraphAggregation = GraphAggregation.PER_QUERY_HEAD
    leiden_resolution: float = 1.0
    leiden_seed: int = 0
    # Not in the reference: how a decoded token picks its community.  "modularity" is the
    # reference's rule (largest modularity gain among the communities of the token's eight
    # strongest neighbours, a new community when no gain is positive); "nearest_centroid"
    # joins the live community whose centroid has the largest inner product with the token's
    # key (ties: smallest id) - one more centroid scan per layer and step.
    online_assignment: str = "modularity"
    # Not in the reference either: "fp32" keeps the centroid table unquantised (scores from the
    # fixed-order fp32 sum, running mean stored as it is; four stand-alone kernels per layer
    # call instead of the single cluster launch); "e4m3" is the reference's layout.
    centroid_dtype: str = "e4m3"

    def __post_init__(self) -> None:
        object.__setattr__(self, "aggregation", GraphAggregation(self.aggregation))
        problems = []
        if self.centroid_dtype not in ("e4m3", "fp32"):
            problems.append("centroid_dtype must be 'e4m3' or 'fp32'")
        if self.online_assignment not in ("modularity", "nearest_centroid"):
            problems.append("online_assignment must be 'modularity' or 'nearest_centroid'")
        if self.token_budget <= 0 or self.token_budget % 64 != 0:
            problems.append("token_budget must be a positive multiple of 64")
        elif self.num_sink < 0 or self.num_sink + 1 >= self.token_budget:
            problems.append("num_sink leaves no selected-token capacity")
        if not (0.0 <= self.lam <= 1.0):
            problems.append("lam must be in [0, 1]")
        if self.leiden_resolution <= 0:
            problems.append("leiden_resolution must be positive")
        if problems:
            raise ValueError(problems[0])


@dataclass(frozen=True, slots=True)
class PartitionConfig:
    """Where and how wide the host-side prefill partition jobs run."""

    devices: tuple[str, ...] = ()
    workers_per_device: int = 2

    def __post_init__(self) -> None:
        if self.workers_per_device <= 0:
            raise ValueError("workers_per_device must be positive")


__all__ = ["CommunityKVConfig", "GraphAggregation", "PartitionConfig"]

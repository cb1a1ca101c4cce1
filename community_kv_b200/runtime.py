"""Request runtime: prefill-state conversion, fixed-address layer state, decode.

Keeps the public surface of the reference's ``community_kv/runtime.py``:
``convert_prefill_tensors`` (``:85-234``), ``DecodeRuntime.prepare_layer`` /
``.decode`` / ``.assert_no_overflow`` (``:237-399``) and ``CommunityKVRuntime``
(``:402-614``).  Decode runs through the CUDA library; there is no other path.

Leiden partitioning stays on the host and is not implemented here:
``CommunityKVRuntime`` takes a ``partitioner`` callable that turns one layer's
prefill top-k edges into a partitioned layer (the reference's
``build_partitioned_layer`` has exactly that shape).  Synthetic or externally
computed partitions enter through ``DecodeRuntime.prepare_layer``.
"""

from __future__ import annotations

import ctypes

from dataclasses import dataclass
from types import TracebackType
from typing import Any, Callable, Mapping, Sequence

import torch

from community_kv_b200 import native, ops
from community_kv_b200.config import CommunityKVConfig, GraphAggregation, PartitionConfig
from community_kv_b200.state import (
    ATTENTION_TILE,
    HEAD_DIM,
    DecodeDeltaChunks,
    DecodeLayerWorkspace,
    MutableGraphState,
    PrefillCSR,
)


def _effective_token_budget(*, configured_budget: int, prefill_seq_len: int, num_sink: int) -> int:
    """Budget capped to the whole 64-token tiles a short prompt can fill."""

    whole_tiles = (prefill_seq_len + 1) // ATTENTION_TILE * ATTENTION_TILE
    budget = configured_budget if configured_budget < whole_tiles else whole_tiles
    if budget <= num_sink + 1:
        raise ValueError("prefill sequence is too short for the fixed 64-token decode kernel")
    return budget


@dataclass(slots=True)
class ConvertedPrefillState:
    """Validated decode state of one layer."""

    csr: PrefillCSR
    mutable: MutableGraphState
    current_position: torch.Tensor
    initial_community_counts: tuple[int, ...]
    prefill_seq_len: int
    decode_capacity: int
    group_size: int
    aggregation: GraphAggregation
    query_heads: int
    kv_heads: int


@dataclass(slots=True)
class DecodeLayerState:
    """Fixed-address state and workspaces of one transformer layer."""

    converted: ConvertedPrefillState
    workspace: DecodeLayerWorkspace
    sink_positions: torch.Tensor
    args: native.LayerArgs | None = None
    cache_key: tuple[int, ...] | None = None
    update_done: Any = None  # deferred update: event of the layer's last online assignment
    # nearest-centroid assignment variant: the community each graph's new token joins
    forced: torch.Tensor | None = None


def _pad_member_offsets(member_offsets: torch.Tensor, *, community_capacity: int) -> torch.Tensor:
    if member_offsets.dtype != torch.int32 or member_offsets.ndim != 2:
        raise TypeError("member_offsets must be a rank-two int32 tensor")
    width = member_offsets.shape[1]
    if width > community_capacity + 1:
        raise ValueError("member offsets exceed centroid community capacity")
    if width == community_capacity + 1:
        return member_offsets.contiguous()
    tail = member_offsets[:, -1:].expand(-1, community_capacity + 1 - width)
    return torch.cat((member_offsets, tail), dim=1).contiguous()


def convert_prefill_tensors(
    *,
    member_offsets: torch.Tensor,
    member_positions: torch.Tensor,
    num_communities: torch.Tensor,
    centroids: torch.Tensor,
    community_sizes: torch.Tensor,
    community_weight: torch.Tensor,
    total_weight: torch.Tensor,
    token_communities: torch.Tensor,
    retrieval_to_graph: torch.Tensor | None = None,
    retrieval_to_kv: torch.Tensor | None = None,
    prefill_seq_len: int,
    max_decode_tokens: int,
    group_size: int = 4,
    aggregation: GraphAggregation = GraphAggregation.PER_QUERY_HEAD,
    query_heads: int | None = None,
    kv_heads: int | None = None,
    centroid_dtype: torch.dtype = torch.float8_e4m3fn,
) -> ConvertedPrefillState:
    """Validate one layer's partition tensors and allocate its decode-delta pools.

    ``centroid_dtype`` (not in the reference, whose table is always e4m3): ``torch.float32``
    admits an fp32 centroid table (``CommunityKVConfig(centroid_dtype="fp32")``).
    """

    if centroids.ndim != 3 or centroids.shape[-1] != HEAD_DIM:
        raise ValueError("centroids must have shape [retrieval heads, communities, 128]")
    if centroids.dtype != centroid_dtype:
        raise TypeError("centroids must use FP8 E4M3" if centroid_dtype == torch.float8_e4m3fn
                        else f"centroids must use {centroid_dtype}")
    heads, capacity, _ = centroids.shape
    graphs = member_offsets.shape[0]
    if min(heads, graphs, capacity) <= 0:
        raise ValueError("prefill state must contain active graphs and centroids")
    if member_positions.dtype != torch.int32 or member_positions.ndim != 2:
        raise TypeError("member_positions must be a rank-two int32 tensor")
    if member_positions.shape[0] != graphs:
        raise ValueError("member positions must contain one row per graph")
    if num_communities.dtype != torch.int32:
        raise TypeError("num_communities must use int32")
    if num_communities.shape != (graphs,):
        raise ValueError("num_communities must contain one value per graph")
    if community_sizes.shape != (heads, capacity):
        raise ValueError("community_sizes must match centroids")
    if community_sizes.dtype != torch.int32:
        raise TypeError("community_sizes must use int32")
    if community_weight.shape != (graphs, capacity):
        raise ValueError("community_weight must have one row per graph")
    if community_weight.dtype != torch.float32:
        raise TypeError("community_weight must use float32")
    if total_weight.shape != (graphs,) or total_weight.dtype != torch.float32:
        raise TypeError("total_weight must be one float32 value per graph")
    if token_communities.dtype != torch.int32 or token_communities.ndim != 2:
        raise TypeError("token_communities must be a rank-two int32 tensor")
    if token_communities.shape[0] != graphs:
        raise ValueError("token_communities must contain one row per graph")
    if prefill_seq_len <= 0 or max_decode_tokens <= 0:
        raise ValueError("prefill and decode capacities must be positive")
    if not 1 <= group_size <= 16:
        raise ValueError("group_size must be in [1, 16]")
    aggregation = GraphAggregation(aggregation)
    if retrieval_to_graph is None or retrieval_to_kv is None:
        if heads != graphs:
            raise ValueError("aggregation mappings are required for non-identity state")
        retrieval_to_graph = torch.arange(heads, dtype=torch.int32, device=centroids.device)
        retrieval_to_kv = retrieval_to_graph
    for mapping in (retrieval_to_graph, retrieval_to_kv):
        if mapping.dtype != torch.int32 or mapping.shape != (heads,):
            raise TypeError("aggregation mappings must be int32 retrieval-head vectors")
    widest_kv = int(retrieval_to_kv.max()) + 1
    query_heads = heads * group_size if query_heads is None else query_heads
    kv_heads = widest_kv if kv_heads is None else kv_heads
    if query_heads != heads * group_size:
        raise ValueError("query-head count does not match retrieval-head geometry")
    if kv_heads <= 0 or widest_kv > kv_heads:
        raise ValueError("KV-head count does not cover retrieval mappings")
    if token_communities.shape[1] < prefill_seq_len + max_decode_tokens:
        raise ValueError("token_communities lacks requested decode headroom")
    device = centroids.device
    for tensor in (
        member_offsets,
        member_positions,
        num_communities,
        community_sizes,
        community_weight,
        total_weight,
        token_communities,
        retrieval_to_graph,
        retrieval_to_kv,
    ):
        if tensor.device != device:
            raise ValueError("all converted tensors must share one device")

    head_counts = num_communities[retrieval_to_graph.long()].contiguous()
    initial = tuple(int(v) for v in head_counts.cpu().tolist())
    if any(not 0 < count <= capacity for count in initial):
        raise ValueError("active community counts must fit centroid capacity")
    csr = PrefillCSR(
        member_offsets=_pad_member_offsets(member_offsets, community_capacity=capacity),
        member_positions=member_positions.contiguous(),
        community_counts=num_communities.clone(),
    )
    mutable = MutableGraphState(
        centroids=centroids.contiguous(),
        community_sizes=community_sizes.contiguous(),
        community_counts=head_counts.clone(),
        community_weight=community_weight.contiguous(),
        total_weight=total_weight.contiguous(),
        token_communities=token_communities.contiguous(),
        deltas=DecodeDeltaChunks.allocate(
            graph_count=graphs,
            community_capacity=capacity,
            max_decode_tokens=max_decode_tokens,
            device=device,
        ),
        retrieval_to_graph=retrieval_to_graph.contiguous(),
        retrieval_to_kv=retrieval_to_kv.contiguous(),
    )
    csr.validate()
    mutable.validate()
    return ConvertedPrefillState(
        csr=csr,
        mutable=mutable,
        current_position=torch.full((graphs,), prefill_seq_len, dtype=torch.int32, device=device),
        initial_community_counts=initial,
        prefill_seq_len=prefill_seq_len,
        decode_capacity=max_decode_tokens,
        group_size=group_size,
        aggregation=aggregation,
        query_heads=query_heads,
        kv_heads=kv_heads,
    )


class DecodeRuntime:
    """Fixed-address per-layer decode states; one CUDA-library call per layer and token."""

    def __init__(self, config: CommunityKVConfig, *, splits: int | None = None,
                 defer_update: bool = False, max_communities: int = 0) -> None:
        """``defer_update``: run each layer's online assignment on a second stream beside the
        work that follows the layer's attention (see ``ops.DeferredUpdate``); same results.
        ``max_communities`` (not in the reference): select at most that many communities per
        retrieval head under the token budget ("top-k communities"; 0 = the budget alone)."""

        if max_communities < 0:
            raise ValueError("max_communities must be nonnegative")
        self.config = config
        self.max_communities = max_communities
        self.splits = splits
        self.defer_update = defer_update
        self._deferred: ops.DeferredUpdate | None = None
        self.layers: dict[int, DecodeLayerState] = {}

    def reset(self) -> None:
        self.synchronize_updates()
        self.layers.clear()

    def synchronize_updates(self) -> None:
        """Wait for deferred online assignments (before the graph state is read on the host)."""

        if self._deferred is not None:
            self._deferred.synchronize()

    def prepare_partitioned_layer(self, state: Any) -> DecodeLayerState:
        """Install a partitioned layer (any object with the reference's ``PartitionedLayer`` fields)."""

        return self.prepare_layer(
            state.layer_idx,
            member_offsets=state.member_offsets,
            member_positions=state.member_positions,
            num_communities=state.community_counts,
            centroids=state.centroids,
            community_sizes=state.community_sizes,
            community_weight=state.community_weight,
            total_weight=state.total_weight,
            token_communities=state.token_communities,
            retrieval_to_graph=state.retrieval_to_graph,
            retrieval_to_kv=state.retrieval_to_kv,
            prefill_seq_len=state.prefill_seq_len,
            max_decode_tokens=state.token_communities.shape[1] - state.prefill_seq_len,
            group_size=state.query_heads // state.retrieval_to_graph.numel(),
            aggregation=state.aggregation,
            query_heads=state.query_heads,
            kv_heads=state.kv_heads,
        )

    def prepare_layer(self, layer_idx: int, **tensors: Any) -> DecodeLayerState:
        """Same keyword arguments as ``convert_prefill_tensors``."""

        if layer_idx in self.layers:
            raise ValueError(f"layer {layer_idx} is already prepared")
        tensors.setdefault(
            "centroid_dtype", torch.float32 if self.config.centroid_dtype == "fp32" else torch.float8_e4m3fn)
        converted = convert_prefill_tensors(**tensors)
        mutable = converted.mutable
        budget = _effective_token_budget(
            configured_budget=self.config.token_budget,
            prefill_seq_len=converted.prefill_seq_len,
            num_sink=self.config.num_sink,
        )
        device = mutable.centroids.device
        layer = DecodeLayerState(
            converted=converted,
            workspace=DecodeLayerWorkspace.allocate(
                retrieval_head_count=mutable.retrieval_head_count,
                graph_count=mutable.graph_count,
                group_size=converted.group_size,
                community_capacity=mutable.community_capacity,
                token_budget=budget,
                num_sink=self.config.num_sink,
                dtype=torch.bfloat16,
                device=device,
                score_community_counts=converted.initial_community_counts,
                score_headroom=converted.decode_capacity,
                splits=self.splits,
                max_communities=self.max_communities,
            ),
            sink_positions=torch.arange(self.config.num_sink, dtype=torch.int32, device=device),
        )
        self.layers[layer_idx] = layer
        return layer

    def decode(
        self,
        *,
        layer_idx: int,
        query: torch.Tensor,
        key: torch.Tensor,
        value: torch.Tensor,
        softmax_scale: float,
    ) -> torch.Tensor:
        layer = self.layers.get(layer_idx)
        if layer is None:
            raise RuntimeError(f"decode layer {layer_idx} is not prepared")
        if query.ndim != 4 or query.shape[0] != 1 or query.shape[2] != 1 or query.shape[3] != HEAD_DIM:
            raise ValueError("decode requires query shape [1, Hq, 1, 128]")
        heads = layer.converted.query_heads
        if query.shape[1] != heads:
            raise ValueError(f"decode expected {heads} query heads, found {query.shape[1]}")
        if key.ndim != 4 or key.shape[0] != 1 or value.shape != key.shape:
            raise ValueError("decode requires key/value shape [1, Hkv, S, 128]")
        if key.shape[1] != layer.converted.kv_heads:
            raise ValueError(
                f"decode expected {layer.converted.kv_heads} KV heads, found {key.shape[1]}"
            )
        flat_query = query[0, :, 0, :]
        if not flat_query.is_contiguous():
            flat_query = flat_query.contiguous()
        # The state and workspaces never move; the packed argument block is
        # rebuilt only when the caller hands in different K/V storage.
        cache_key = (key.data_ptr(), value.data_ptr(), *key.stride(), float(softmax_scale))
        if layer.args is None or layer.cache_key != cache_key:
            layer.args = ops.build_layer_args(
                query=flat_query,
                key=key[0],
                value=value[0],
                csr=layer.converted.csr,
                state=layer.converted.mutable,
                sink_positions=layer.sink_positions,
                current_position=layer.converted.current_position,
                softmax_scale=softmax_scale,
                lam=self.config.lam,
                workspace=layer.workspace,
            )
            layer.cache_key = cache_key
        layer.args.query = flat_query.data_ptr()
        if self.config.online_assignment == "nearest_centroid":
            self._nearest_centroid(layer, key[0])
        if self.defer_update:
            if self._deferred is None:
                self._deferred = ops.DeferredUpdate(query.device)
            layer.update_done = self._deferred.launch(layer.args, pending=layer.update_done)
        else:
            native.call("ckv_decode_layer", layer.args, native.current_stream(query.device))
        return layer.workspace.attention.output.view(1, 1, heads, HEAD_DIM)

    def _nearest_centroid(self, layer: DecodeLayerState, key: torch.Tensor) -> None:
        """The variant of the online assignment that is not in the reference: the token joins
        the live community whose centroid has the largest inner product with its key.

        One small launch (``ckv_nearest_centroid``) scores the key row of the token being
        decoded (already in the cache at the graph's cursor) against the head's centroid table -
        the fp16 value the scoring kernel gives a query group made of that key, in the fixed
        summation order, so that a CPU reproduces the choice bit for bit - and leaves the first
        maximum per leader head where the update reads it (``forced_community``).
        """

        mutable = layer.converted.mutable
        device = mutable.centroids.device
        if layer.forced is None:
            layer.forced = torch.full((mutable.graph_count,), -1, dtype=torch.int32, device=device)
        layer.args.forced_community = layer.forced.data_ptr()  # the block is rebuilt when the cache moves
        if layer.update_done is not None:
            # the previous step's deferred update still reads `forced`
            torch.cuda.current_stream(device).wait_event(layer.update_done)
        status = native.library().ckv_nearest_centroid(
            ctypes.byref(layer.args), ctypes.c_void_p(layer.forced.data_ptr()),
            ctypes.c_void_p(native.current_stream(device)),
        )
        if status:
            raise native.NativeError(native.library().ckv_status_string(status).decode())

    def assert_no_overflow(self) -> None:
        self.synchronize_updates()
        failures = {}
        for layer_idx, layer in self.layers.items():
            flags = layer.workspace.update.overflow
            if int(torch.count_nonzero(flags)):
                failures[layer_idx] = flags.cpu().tolist()
            if int(layer.workspace.attention.status[0]):
                failures[layer_idx] = f"device status {int(layer.workspace.attention.status[0])}"
        if failures:
            raise RuntimeError(f"decode state overflow: {failures}")


Partitioner = Callable[..., Any]


class CommunityKVRuntime:
    """Request lifecycle: prefill edges -> host partition -> fixed-address decode."""

    def __init__(
        self,
        *,
        config: CommunityKVConfig,
        partition: PartitionConfig,
        num_layers: int,
        max_decode_tokens: int,
        partitioner: Partitioner | None = None,
    ) -> None:
        if num_layers <= 0 or max_decode_tokens <= 0:
            raise ValueError("num_layers and max_decode_tokens must be positive")
        self.config = config
        self.partition = partition
        self.num_layers = num_layers
        self.max_decode_tokens = max_decode_tokens
        self.decode_runtime = DecodeRuntime(config)
        self.partitioner = partitioner
        self.partition_runtime = self  # the partition hand-off lives on this object
        self.resolutions: dict[int, float] = {}
        self._pending: dict[int, Any] = {}
        self._ready = False
        self._generation_cache: Any | None = None

    def __enter__(self) -> "CommunityKVRuntime":
        return self

    def __exit__(
        self,
        exc_type: type[BaseException] | None,
        exc_value: BaseException | None,
        traceback: TracebackType | None,
    ) -> None:
        self.close()

    def start_request(
        self,
        *,
        resolutions: Mapping[int, float] | Sequence[float] | None = None,
        max_decode_tokens: int | None = None,
    ) -> None:
        self._pending.clear()
        self.decode_runtime.reset()
        self._ready = False
        if max_decode_tokens is not None:
            if max_decode_tokens <= 0:
                raise ValueError("max_decode_tokens must be positive")
            self.max_decode_tokens = max_decode_tokens
        if resolutions is None:
            table: dict[int, float] = {}
        elif isinstance(resolutions, Mapping):
            table = {int(layer): float(value) for layer, value in resolutions.items()}
        else:
            if len(resolutions) != self.num_layers:
                raise ValueError("resolution vector must contain one value per layer")
            table = {layer: float(value) for layer, value in enumerate(resolutions)}
        if any(value <= 0 for value in table.values()):
            raise ValueError("all layer resolutions must be positive")
        self.resolutions = table

    def submit_prefill_layer(
        self,
        *,
        layer_idx: int,
        topk_indices: torch.Tensor,
        topk_scores: torch.Tensor,
        keys: torch.Tensor,
        completion_event: Any,
    ) -> None:
        """Hand one layer's prefill edges to the host partitioner."""

        if self.partitioner is None:
            raise RuntimeError(
                "no partitioner configured: Leiden partitioning is host-side and outside this "
                "package; pass partitioner=<callable returning a partitioned layer>"
            )
        if layer_idx in self._pending:
            raise ValueError(f"layer {layer_idx} was already submitted")
        if completion_event is not None:
            completion_event.synchronize()
        self._pending[layer_idx] = self.partitioner(
            layer_idx=layer_idx,
            topk_indices=topk_indices,
            topk_scores=topk_scores,
            keys=keys,
            num_sink=self.config.num_sink,
            lam=self.config.lam,
            leiden_resolution=self.resolutions.get(layer_idx, self.config.leiden_resolution),
            leiden_seed=self.config.leiden_seed,
            max_decode_tokens=self.max_decode_tokens,
            aggregation=self.config.aggregation,
        )

    def finish_prefill(self) -> None:
        if self._ready:
            return
        for layer_idx in sorted(self._pending):
            self.decode_runtime.prepare_partitioned_layer(self._pending[layer_idx])
        self._pending.clear()
        have = set(self.decode_runtime.layers)
        want = set(range(self.num_layers))
        if have != want:
            raise RuntimeError(
                "partitioned layer set is incomplete: "
                f"missing={sorted(want - have)}, extra={sorted(have - want)}"
            )
        self._ready = True
        if self._generation_cache is not None:
            self._generation_cache.enable_device_updates()

    def ensure_ready(self) -> None:
        if not self._ready:
            self.finish_prefill()

    def generate(
        self,
        model: Any,
        inputs: torch.Tensor | None = None,
        *,
        resolutions: Mapping[int, float] | Sequence[float] | None = None,
        **kwargs: Any,
    ) -> Any:
        """Greedy single-sequence generation with a managed static cache."""

        if inputs is not None and "input_ids" in kwargs:
            raise ValueError("pass input_ids either positionally or by keyword")
        input_ids = kwargs.get("input_ids", inputs)
        if not isinstance(input_ids, torch.Tensor) or input_ids.ndim != 2:
            raise ValueError("generate requires rank-two input_ids")
        if input_ids.shape[0] != 1:
            raise ValueError("CommunityKV generate currently requires batch size 1")
        if getattr(model.config, "_attn_implementation", None) != "community_kv":
            raise ValueError("model.config._attn_implementation must be 'community_kv'")
        refusals = {
            "past_key_values": "CommunityKV generate manages past_key_values",
            "cache_implementation": "CommunityKV generate manages the cache implementation",
            "assistant_model": "CommunityKV generate does not support assisted generation",
            "penalty_alpha": "CommunityKV generate does not support contrastive search",
        }
        for name, message in refusals.items():
            if kwargs.get(name) is not None:
                raise ValueError(message)
        if kwargs.get("do_sample") not in (None, False):
            raise ValueError("CommunityKV generate supports greedy decoding only")
        generation_config = kwargs.get(
            "generation_config", getattr(model, "generation_config", None)
        )

        def option(name: str, default: Any) -> Any:
            # an unset generation option reads as None in recent transformers releases
            value = kwargs[name] if name in kwargs else getattr(generation_config, name, default)
            return default if value is None else value

        if option("num_beams", 1) != 1:
            raise ValueError("CommunityKV generate does not support beam search")
        if option("num_return_sequences", 1) != 1:
            raise ValueError("CommunityKV generate supports one returned sequence per prompt")
        prompt_tokens = int(input_ids.shape[-1])
        max_new_tokens = option("max_new_tokens", None)
        if max_new_tokens is None:
            max_length = option("max_length", None)
            if max_length is None:
                raise ValueError("generate requires max_new_tokens or max_length")
            max_new_tokens = int(max_length) - prompt_tokens
        if isinstance(max_new_tokens, bool) or not isinstance(max_new_tokens, int) or max_new_tokens <= 0:
            raise ValueError("max_new_tokens must be a positive integer")
        model_layers = int(model.config.num_hidden_layers)
        if model_layers != self.num_layers:
            raise ValueError(f"runtime has {self.num_layers} layers but model has {model_layers}")
        if self._generation_cache is not None:
            raise RuntimeError("CommunityKV runtime is already generating")

        from community_kv_b200.cache import StaticCache

        cache = StaticCache(
            num_hidden_layers=self.num_layers, max_cache_len=prompt_tokens + max_new_tokens
        )
        self.start_request(resolutions=resolutions, max_decode_tokens=max(1, max_new_tokens - 1))
        call = dict(kwargs)
        call.update(past_key_values=cache, do_sample=False, num_beams=1, num_return_sequences=1)
        if hasattr(generation_config, "disable_compile"):
            call["disable_compile"] = True
        self._generation_cache = cache
        try:
            output = model.generate(**call) if inputs is None else model.generate(inputs, **call)
            self.finish_prefill()
            self.assert_no_overflow()
            return output
        finally:
            self._generation_cache = None

    def close(self) -> None:
        self._pending.clear()

    def shutdown(self) -> None:
        self.close()

    def assert_no_overflow(self) -> None:
        self.decode_runtime.assert_no_overflow()


__all__ = [
    "CommunityKVRuntime",
    "ConvertedPrefillState",
    "DecodeLayerState",
    "DecodeRuntime",
    "convert_prefill_tensors",
]

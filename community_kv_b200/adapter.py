"""Hugging Face attention plug-in.

Stands where the reference's ``community_kv/attention/adapter.py:19-91`` stands:
``CommunityKVAttention(runtime).register()`` puts one callable under the name
``"community_kv"`` into transformers' attention registry, and every attention module of
the model then calls it with ``(module, query, key, value, mask, scaling, ...)``.

A call is one of two things, told apart by the query length:

* **prefill** (more than one query position): ``ckv_prefill_topk`` in mode 1 - causal
  attention plus, per query head and row, the eight strongest keys under the reference's
  rule - on the caller's stream.  The edges and the layer's keys go to the runtime, which
  builds the layer's graph and partition from them beside the remaining layers' prefill;
  an event recorded behind the kernel tells it when they are valid.
* **decode** (one query position): one ``ckv_decode_layer`` call for the layer, i.e.
  centroid scores, community selection, gather + segmented attention, split merge and the
  online assignment of the new token.
"""

from __future__ import annotations

from typing import TYPE_CHECKING, Any

import torch

if TYPE_CHECKING:
    from community_kv_b200.runtime import CommunityKVRuntime

ATTENTION_IMPLEMENTATION = "community_kv"
_EDGES_PER_ROW = 8  # the reference's rule reports eight neighbours per row


class CommunityKVAttention:
    """The callable transformers dispatches to, bound to one request runtime."""

    IMPL_NAME = ATTENTION_IMPLEMENTATION

    def __init__(self, runtime: "CommunityKVRuntime") -> None:
        self.runtime = runtime

    def register(self) -> str:
        """Install ``forward`` in the registry; returns the implementation name to set on the model config."""

        from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS

        ALL_ATTENTION_FUNCTIONS[self.IMPL_NAME] = self.forward
        return self.IMPL_NAME

    # transformers' attention interface: [B, H, S, D] tensors in, ([B, S, H, D], weights) out
    def forward(
        self,
        module: torch.nn.Module,
        query: torch.Tensor,
        key: torch.Tensor,
        value: torch.Tensor,
        attention_mask: torch.Tensor | None,
        scaling: float,
        dropout: float = 0.0,
        **kwargs: Any,
    ) -> tuple[torch.Tensor, None]:
        layer = int(module.layer_idx)
        if query.shape[2] == 1:
            return self._decode(layer, query, key, value, float(scaling)), None
        return self._prefill(layer, query, key, value, float(scaling)), None

    def _prefill(self, layer: int, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                 scale: float) -> torch.Tensor:
        from community_kv_b200.prefill import prefill_attention_topk

        rows = query.shape[2]
        sinks = self.runtime.config.num_sink
        if rows < sinks + _EDGES_PER_ROW:
            raise ValueError("CommunityKV prefill is too short to build a graph")
        # the static cache hands in its whole capacity: only the prompt's rows take part
        prompt_key, prompt_value = key[:, :, :rows, :], value[:, :, :rows, :]
        out, _lse, _, _, edge_weight, edge_index = prefill_attention_topk(
            query.transpose(1, 2).contiguous(),
            prompt_key.transpose(1, 2).contiguous(),
            prompt_value.transpose(1, 2).contiguous(),
            softmax_scale=scale,
            num_sink=sinks,
        )
        with torch.cuda.device(key.device):
            edges_valid = torch.cuda.Event(enable_timing=False)
            edges_valid.record()
        self.runtime.submit_prefill_layer(
            layer_idx=layer,
            topk_indices=edge_index[0],
            topk_scores=edge_weight[0],
            keys=prompt_key[0],
            completion_event=edges_valid,
        )
        return out

    def _decode(self, layer: int, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                scale: float) -> torch.Tensor:
        self.runtime.ensure_ready()  # every layer's partition has been installed
        return self.runtime.decode_runtime.decode(
            layer_idx=layer, query=query, key=key, value=value, softmax_scale=scale
        )


HuggingFaceAttention = CommunityKVAttention

__all__ = ["ATTENTION_IMPLEMENTATION", "CommunityKVAttention", "HuggingFaceAttention"]

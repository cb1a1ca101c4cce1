"""Hugging Face attention plug-in (reference ``community_kv/attention/adapter.py:19-91``).

``CommunityKVAttention(runtime).register()`` installs ``forward`` under the name
``"community_kv"`` in transformers' attention registry.  Prefill calls
(query length > 1) run the fused causal attention + neighbour-edge kernel and
hand the edges to the runtime; decode calls run one fused layer transition.
"""

from __future__ import annotations

from typing import TYPE_CHECKING, Any

import torch

if TYPE_CHECKING:
    from community_kv_b200.runtime import CommunityKVRuntime

ATTENTION_IMPLEMENTATION = "community_kv"
_TOPK_WIDTH = 8


class CommunityKVAttention:
    IMPL_NAME = ATTENTION_IMPLEMENTATION

    def __init__(self, runtime: "CommunityKVRuntime") -> None:
        self.runtime = runtime

    def register(self) -> str:
        from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS

        ALL_ATTENTION_FUNCTIONS[self.IMPL_NAME] = self.forward
        return self.IMPL_NAME

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
        layer_idx = int(module.layer_idx)
        length = query.shape[2]
        if length > 1:
            if length < _TOPK_WIDTH + self.runtime.config.num_sink:
                raise ValueError("CommunityKV prefill is too short to build a graph")
            from community_kv_b200.prefill import prefill_attention_topk

            key = key[:, :, :length, :]
            value = value[:, :, :length, :]
            result = prefill_attention_topk(
                query.transpose(1, 2).contiguous(),
                key.transpose(1, 2).contiguous(),
                value.transpose(1, 2).contiguous(),
                softmax_scale=float(scaling),
                num_sink=self.runtime.config.num_sink,
            )
            with torch.cuda.device(key.device):
                done = torch.cuda.Event(enable_timing=False)
                done.record()
            self.runtime.submit_prefill_layer(
                layer_idx=layer_idx,
                topk_indices=result[5][0],
                topk_scores=result[4][0],
                keys=key[0],
                completion_event=done,
            )
            return result[0], None

        self.runtime.ensure_ready()
        output = self.runtime.decode_runtime.decode(
            layer_idx=layer_idx,
            query=query,
            key=key,
            value=value,
            softmax_scale=float(scaling),
        )
        return output, None


HuggingFaceAttention = CommunityKVAttention

__all__ = ["ATTENTION_IMPLEMENTATION", "CommunityKVAttention", "HuggingFaceAttention"]

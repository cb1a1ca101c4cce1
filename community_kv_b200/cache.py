"""Fixed-address BF16 key/value cache for Hugging Face ``generate``.

Same behaviour as the reference's ``community_kv/attention/cache.py:9-121``:
prefill appends with a host cursor; after ``enable_device_updates`` the cursor
lives on the device so that decode steps have no host round trip.  A decode step's
single new row goes in through one ``ckv_append_kv`` launch that reads the device
cursor itself (the reference runs ``arange`` + two ``index_copy_``, ``cache.py:39-47``).
"""

from __future__ import annotations

import torch
from transformers.cache_utils import Cache, StaticLayer


class StaticCacheLayer(StaticLayer):
    def __init__(self, max_cache_len: int) -> None:
        super().__init__(max_cache_len=max_cache_len)
        self.valid_length = 0
        self.device_updates = False
        self.cumulative_length = torch.zeros(1, dtype=torch.int32)

    def lazy_initialization(self, key_states: torch.Tensor, value_states: torch.Tensor) -> None:
        if torch.bfloat16 not in (key_states.dtype,) or value_states.dtype != torch.bfloat16:
            raise TypeError("CommunityKV cache requires BF16 K/V")
        super().lazy_initialization(key_states, value_states)
        self.valid_length = 0

    def update(self, key_states, value_states, *args, **kwargs):
        if not self.is_initialized:
            self.lazy_initialization(key_states, value_states)
        count = key_states.shape[-2]
        if self.device_updates:
            if count == 1 and key_states.is_cuda and self.keys.is_contiguous() and self.values.is_contiguous():
                from community_kv_b200 import ops

                ops.append_kv(self.keys, self.values, key_states[..., 0, :], value_states[..., 0, :],
                              self.cumulative_length)
                self.cumulative_length.add_(1)
                return self.keys, self.values
            rows = torch.arange(count, device=self.device) + self.cumulative_length
            self.cumulative_length.add_(count)
            self.keys.index_copy_(2, rows, key_states)
            self.values.index_copy_(2, rows, value_states)
            return self.keys, self.values
        stop = self.valid_length + count
        if stop > self.max_cache_len:
            raise ValueError(f"KV cache capacity exceeded: {stop} > {self.max_cache_len}")
        self.keys[:, :, self.valid_length : stop, :].copy_(key_states)
        self.values[:, :, self.valid_length : stop, :].copy_(value_states)
        self.valid_length = stop
        self.cumulative_length.fill_(stop)
        return self.keys, self.values

    def get_mask_sizes(self, query_length: int) -> tuple[int, int]:
        if self.device_updates:
            return self.max_cache_len, 0
        return min(self.valid_length + query_length, self.max_cache_len), 0

    def get_seq_length(self):
        if self.device_updates and self.is_initialized:
            return self.cumulative_length
        return self.valid_length if self.is_initialized else 0

    def enable_device_updates(self) -> None:
        if not self.is_initialized:
            raise RuntimeError("cache layer must be initialized before graph decode")
        with torch.inference_mode():
            self.cumulative_length.fill_(self.valid_length)
        self.device_updates = True

    def sync_valid_length(self) -> None:
        if self.is_initialized:
            self.valid_length = int(self.cumulative_length.item())

    def reset(self) -> None:
        if self.is_initialized:
            with torch.inference_mode():
                self.keys.zero_()
                self.values.zero_()
                self.cumulative_length.zero_()
        self.valid_length = 0
        self.device_updates = False


class StaticCache(Cache):
    def __init__(self, *, num_hidden_layers: int, max_cache_len: int) -> None:
        super().__init__(
            layers=[StaticCacheLayer(max_cache_len=max_cache_len) for _ in range(num_hidden_layers)]
        )

    def layer(self, layer_idx: int) -> StaticCacheLayer:
        layer = self.layers[layer_idx]
        if not isinstance(layer, StaticCacheLayer):
            raise TypeError(f"unexpected cache layer: {type(layer).__name__}")
        return layer

    def valid_length(self, layer_idx: int) -> int:
        return self.layer(layer_idx).valid_length

    def enable_device_updates(self) -> None:
        for index in range(len(self.layers)):
            self.layer(index).enable_device_updates()

    def sync_valid_lengths(self) -> None:
        for index in range(len(self.layers)):
            self.layer(index).sync_valid_length()


__all__ = ["StaticCache", "StaticCacheLayer"]

"""Fixed-address bf16 key/value cache for Hugging Face ``generate``.

Takes the place of the reference's ``community_kv/attention/cache.py:9-121`` and keeps its
surface (``StaticCache(num_hidden_layers=, max_cache_len=)``, ``layer``, ``valid_length``,
``enable_device_updates``, ``sync_valid_lengths``; per layer ``update``,
``get_mask_sizes``, ``get_seq_length``, ``reset``): the decode kernels read K/V rows in
place, so the storage never moves and rows are only ever appended.

Two phases.  While the prompt is prefilled the write cursor is a host integer.  Once
``enable_device_updates`` has been called the cursor is a one-element int32 tensor on the
device, and appending the row of a decoded token is ONE ``ckv_append_kv`` launch that reads
the cursor itself (the reference runs ``arange`` and two ``index_copy_``,
``cache.py:39-47``): no host round trip, and the step can be captured in a CUDA graph.
"""

from __future__ import annotations

import torch
from transformers.cache_utils import Cache, StaticLayer


class StaticCacheLayer(StaticLayer):
    """One layer's K and V, ``[B, Hkv, max_cache_len, 128]`` bf16 each."""

    def __init__(self, max_cache_len: int) -> None:
        super().__init__(max_cache_len=max_cache_len)
        self.valid_length = 0          # host cursor (prefill phase)
        self.device_updates = False    # True: the device cursor below is the one that counts
        self.cumulative_length = torch.zeros(1, dtype=torch.int32)

    # -- storage ------------------------------------------------------------------------------
    def lazy_initialization(self, key_states: torch.Tensor, value_states: torch.Tensor) -> None:
        for name, tensor in (("key", key_states), ("value", value_states)):
            if tensor.dtype != torch.bfloat16:
                raise TypeError(f"CommunityKV cache requires BF16 K/V ({name} states are {tensor.dtype})")
        super().lazy_initialization(key_states, value_states)
        self.valid_length = 0

    def reset(self) -> None:
        if self.is_initialized:
            with torch.inference_mode():
                for tensor in (self.keys, self.values, self.cumulative_length):
                    tensor.zero_()
        self.valid_length = 0
        self.device_updates = False

    # -- appending ----------------------------------------------------------------------------
    def update(self, key_states, value_states, *args, **kwargs):
        if not self.is_initialized:
            self.lazy_initialization(key_states, value_states)
        if self.device_updates:
            self._append_at_device_cursor(key_states, value_states)
        else:
            self._append_at_host_cursor(key_states, value_states)
        return self.keys, self.values

    def _append_at_host_cursor(self, key_states: torch.Tensor, value_states: torch.Tensor) -> None:
        begin = self.valid_length
        end = begin + key_states.shape[-2]
        if end > self.max_cache_len:
            raise ValueError(f"KV cache capacity exceeded: {end} > {self.max_cache_len}")
        self.keys.narrow(2, begin, end - begin).copy_(key_states)
        self.values.narrow(2, begin, end - begin).copy_(value_states)
        self.valid_length = end
        self.cumulative_length.fill_(end)

    def _append_at_device_cursor(self, key_states: torch.Tensor, value_states: torch.Tensor) -> None:
        count = key_states.shape[-2]
        single_row = count == 1 and key_states.is_cuda and self.keys.is_contiguous() and self.values.is_contiguous()
        if single_row:
            from community_kv_b200 import ops

            # the kernel reads the cursor; the cursor moves on behind it, in stream order
            ops.append_kv(self.keys, self.values, key_states[..., 0, :], value_states[..., 0, :],
                          self.cumulative_length)
        else:
            rows = self.cumulative_length + torch.arange(count, device=self.device)
            self.keys.index_copy_(2, rows, key_states)
            self.values.index_copy_(2, rows, value_states)
        self.cumulative_length.add_(count)

    # -- what the model asks about the cache ----------------------------------------------------
    def get_mask_sizes(self, query_length: int) -> tuple[int, int]:
        if self.device_updates:
            return self.max_cache_len, 0
        return min(self.valid_length + query_length, self.max_cache_len), 0

    def get_seq_length(self):
        if not self.is_initialized:
            return 0
        return self.cumulative_length if self.device_updates else self.valid_length

    # -- switching between the two cursors --------------------------------------------------------
    def enable_device_updates(self) -> None:
        if not self.is_initialized:
            raise RuntimeError("cache layer must be initialized before graph decode")
        with torch.inference_mode():
            self.cumulative_length.fill_(self.valid_length)
        self.device_updates = True

    def sync_valid_length(self) -> None:
        """Read the device cursor back (a host synchronisation)."""

        if self.is_initialized:
            self.valid_length = int(self.cumulative_length.item())


class StaticCache(Cache):
    """``num_hidden_layers`` cache layers of one capacity."""

    def __init__(self, *, num_hidden_layers: int, max_cache_len: int) -> None:
        super().__init__(layers=[StaticCacheLayer(max_cache_len=max_cache_len) for _ in range(num_hidden_layers)])

    def layer(self, layer_idx: int) -> StaticCacheLayer:
        found = self.layers[layer_idx]
        if not isinstance(found, StaticCacheLayer):
            raise TypeError(f"unexpected cache layer: {type(found).__name__}")
        return found

    def valid_length(self, layer_idx: int) -> int:
        return self.layer(layer_idx).valid_length

    def enable_device_updates(self) -> None:
        for index, _ in enumerate(self.layers):
            self.layer(index).enable_device_updates()

    def sync_valid_lengths(self) -> None:
        for index, _ in enumerate(self.layers):
            self.layer(index).sync_valid_length()


__all__ = ["StaticCache", "StaticCacheLayer"]

"""HiraCache / HiraCacheLayer / CacheOutput: the reference's Hugging Face cache
(cache/hira_cache.py:19-249) over the CUDA index.

Behaviour kept from the reference: the first `update` of a layer is the prefill and
builds the index (`indexer.build`), returning the raw prefill keys/values next to empty
queues; later updates append to a queue that is flushed into the index
(`indexer.update`) every `update_every` tokens; `update` returns `(CacheOutput, None)`,
so the model's attention forward must be the patched one (`hira_attention`).

Only `DeviceMode.CUDA_ONLY` is served: this build has no CPU path.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

import torch
from transformers.cache_utils import Cache, CacheLayerMixin

from ..indexer import CUDAIndexer
from ..searcher import CUDASearcher
from .hira_config import DeviceMode, HiraConfig


@dataclass
class CacheOutput:
    queued_keys: torch.Tensor
    queued_values: torch.Tensor
    prefill_keys: Optional[torch.Tensor]
    prefill_values: Optional[torch.Tensor]
    indexer: CUDAIndexer
    searcher: CUDASearcher


class HiraCacheLayer(CacheLayerMixin):
    """One layer; all KV heads (and batch items) of that layer share one index object."""

    def __init__(self, device_mode, update_every: int, indexer_kwargs: dict[str, Any],
                 searcher_kwargs: dict[str, Any]):
        super().__init__()
        self.device_mode = device_mode
        self.update_every = update_every
        self.indexer_kwargs = indexer_kwargs
        self.searcher_kwargs = searcher_kwargs
        self.indexer_cls = None
        self.searcher_cls = None
        if self.device_mode == DeviceMode.CUDA_ONLY:
            self.indexer_cls = CUDAIndexer
            self.searcher_cls = CUDASearcher
        else:
            raise NotImplementedError(
                f"Device mode {self.device_mode} not supported yet (this build runs DeviceMode.CUDA_ONLY only)")

    def lazy_initialization(self, key_states, value_states):
        self.dim = key_states.shape[-1]
        self.vdim = value_states.shape[-1]
        self.vdtype = value_states.dtype
        self._queue_k = self._queue_v = None
        self.B = key_states.shape[0]
        self.H_kv = key_states.shape[-3]
        self.dtype = key_states.dtype
        self.device = key_states.device
        self.indexer = self.indexer_cls(**self.indexer_kwargs)
        self.searcher = self.searcher_cls(**self.searcher_kwargs)
        self._reset_queue()
        self.keys = None    # no dense copies: the index holds keys and values
        self.values = None
        self.is_initialized = True

    def _reset_queue(self):
        """The queue of not-yet-indexed tokens is a pre-allocated buffer of `update_every` rows per
        head; `queued_keys` / `queued_values` are views of its filled part.  (The reference grows the
        queue by `torch.cat` on every token, cache/hira_cache.py:121-124.)"""
        if getattr(self, "_queue_k", None) is None:
            cap = max(1, int(self.update_every))
            self._queue_k = torch.empty((self.B, self.H_kv, cap, self.dim), dtype=self.dtype, device=self.device)
            self._queue_v = torch.empty((self.B, self.H_kv, cap, self.vdim), dtype=self.vdtype, device=self.device)
        self.queued_len = 0
        self.queued_keys = self._queue_k[:, :, :0]
        self.queued_values = self._queue_v[:, :, :0]

    def _enqueue(self, key_states: torch.Tensor, value_states: torch.Tensor):
        n = key_states.shape[-2]
        if self.queued_len + n > self._queue_k.shape[2]:     # more tokens at once than a flush period: make room
            cap = max(2 * self._queue_k.shape[2], self.queued_len + n)
            for name, src in (("_queue_k", self._queue_k), ("_queue_v", self._queue_v)):
                bigger = torch.empty(src.shape[:2] + (cap, src.shape[3]), dtype=src.dtype, device=src.device)
                bigger[:, :, : self.queued_len] = src[:, :, : self.queued_len]
                setattr(self, name, bigger)
        self._queue_k[:, :, self.queued_len:self.queued_len + n] = key_states
        self._queue_v[:, :, self.queued_len:self.queued_len + n] = value_states
        self.queued_len += n
        self.queued_keys = self._queue_k[:, :, : self.queued_len]
        self.queued_values = self._queue_v[:, :, : self.queued_len]

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor,
               cache_kwargs: dict[str, Any] | None = None, *args, **kwargs):
        if not self.is_initialized:
            self.lazy_initialization(key_states, value_states)
            self.indexer.build(key_states, value_states)
            self.indexed_len = key_states.shape[-2]
            return (
                CacheOutput(queued_keys=self.queued_keys, queued_values=self.queued_values,
                            prefill_keys=key_states, prefill_values=value_states,
                            indexer=self.indexer, searcher=self.searcher),
                None,
            )
        self._enqueue(key_states, value_states)
        if self.queued_len >= self.update_every:
            self.update_index()
        return (
            CacheOutput(queued_keys=self.queued_keys, queued_values=self.queued_values,
                        prefill_keys=None, prefill_values=None,
                        indexer=self.indexer, searcher=self.searcher),
            None,
        )

    def update_index(self):
        self.indexer.update(self.queued_keys, self.queued_values)
        self.indexed_len += self.queued_len
        self._reset_queue()

    def get_mask_sizes(self, cache_position):
        """Accepts the query length as an int (current transformers) or a cache_position
        tensor (the signature the reference was written against, cache/hira_cache.py:155-159)."""
        kv_offset = 0
        query_length = cache_position if isinstance(cache_position, int) else cache_position.shape[0]
        kv_length = self.get_seq_length() + query_length
        return kv_length, kv_offset

    def get_seq_length(self):
        if not self.is_initialized:
            return 0
        return self.indexed_len + self.queued_len

    def get_max_cache_shape(self):
        return -1

    def reset(self):
        if self.is_initialized:
            self.indexer = self.indexer_cls(**self.indexer_kwargs)
            self._reset_queue()
            self.is_initialized = False
        if hasattr(self, "cumulative_length"):
            self.cumulative_length = 0


class HiraCache(Cache):
    """Hugging Face `Cache` whose layers index their keys for range-searching attention."""

    def __init__(self, cache_config, hira_config: HiraConfig):
        self.device_mode = hira_config.device_mode
        self.update_every = hira_config.update_every
        self.hira_config = hira_config
        config = cache_config.get_text_config(decoder=True)
        layer_types = getattr(config, "layer_types", None)
        if layer_types is None:
            if getattr(config, "sliding_window", None) is not None:
                layer_types = ["sliding_attention"] * config.num_hidden_layers
            elif getattr(config, "attention_chunk_size", None) is not None:
                layer_types = ["chunked_attention"] * config.num_hidden_layers
            else:
                layer_types = ["full_attention"] * config.num_hidden_layers
        if hasattr(config, "num_kv_shared_layers"):
            layer_types = layer_types[: -config.num_kv_shared_layers]
        layers = [
            HiraCacheLayer(device_mode=self.device_mode, update_every=self.update_every,
                           indexer_kwargs=hira_config.get_indexer_kwargs(),
                           searcher_kwargs=hira_config.get_searcher_kwargs())
            for _ in layer_types
        ]
        super().__init__(layers=layers, offloading=False, offload_only_non_sliding=None)

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int,
               cache_kwargs: dict[str, Any] | None = None, *args, **kwargs):
        cache_output, _ = self.layers[layer_idx].update(key_states, value_states, cache_kwargs)
        return cache_output, None

"""The cache object the attention layer talks to (mirror of ``CustomDynamicCache``,
src/utils/cache.py:14-137, and of its CPU-offloading subclass :139-172).

Only the protocol the path uses is kept -- per-layer ``cache_kwargs``, ``meta``, ``record_kwargs``
(merge), ``update``, ``update_router_kcache``, ``get_kvcache``, ``get_router_kcache``,
``clear_kvcache`` -- implemented on plain dictionaries instead of HF ``DynamicCache`` internals
(which changed between transformers releases)."""
from __future__ import annotations

import torch


class SparseCache:
    def __init__(self):
        self.cache_kwargs = {}
        self.meta = {}
        self.key_cache = {}
        self.value_cache = {}
        self.router_key_cache = {}

    def record_kwargs(self, layer_idx, kwargs):
        if layer_idx in self.cache_kwargs:
            self.cache_kwargs[layer_idx].update(kwargs)
        else:
            self.cache_kwargs[layer_idx] = dict(kwargs)

    def get_layer_length(self):
        return len(self.cache_kwargs)

    def update(self, key_states, value_states, layer_idx, cache_kwargs=None):
        self.key_cache[layer_idx], self.value_cache[layer_idx] = key_states, value_states
        return key_states, value_states

    def update_router_kcache(self, key_states, layer_idx):
        self.router_key_cache[layer_idx] = key_states
        return key_states

    def get_kvcache(self, layer_idx):
        return self.key_cache[layer_idx], self.value_cache[layer_idx]

    def get_router_kcache(self, layer_idx):
        return self.router_key_cache.get(layer_idx)

    def clear_kvcache(self):
        self.key_cache, self.value_cache = {}, {}


class SparseCacheOnCPU(SparseCache):
    """Moves everything it is handed to host memory, as the stage-1 worker's cache does."""

    @staticmethod
    def _cpu(t):
        return t.cpu() if torch.is_tensor(t) and t.is_cuda else t

    def record_kwargs(self, layer_idx, kwargs):
        super().record_kwargs(layer_idx, {k: (self._cpu(v) if torch.is_tensor(v) and v.is_cuda else
                                              (v.clone() if torch.is_tensor(v) else v)) for k, v in kwargs.items()})

    def update(self, key_states, value_states, layer_idx, cache_kwargs=None):
        return super().update(self._cpu(key_states), self._cpu(value_states), layer_idx)

    def update_router_kcache(self, key_states, layer_idx):
        return super().update_router_kcache(self._cpu(key_states), layer_idx)


def create_cache():
    return SparseCache()

"""The cache object the attention layer talks to (mirror of ``CustomDynamicCache``,
src/utils/cache.py:14-137, and of its CPU-offloading subclass :139-172).

Only the protocol the path uses is kept -- per-layer ``cache_kwargs``, ``meta``, ``record_kwargs``
(merge), ``update``, ``update_router_kcache``, ``get_kvcache``, ``get_router_kcache``,
``clear_kvcache`` -- implemented on plain dictionaries instead of HF ``DynamicCache`` internals
(which changed between transformers releases)."""
from __future__ import annotations

import os

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


class SharedPooledCache:
    """One stage-1 block's pooled tensors in a shared-memory file, in the bank's own layouts.

    The reference's stage-1 worker hands its CPU cache object to the service through a ``multiprocessing.Queue``
    (src/prefill.py:124-131), i.e. pickles every pooled tensor and copies it twice.  Here the worker writes, per
    router layer, ``kv [C, 2, Hkv, D]`` (K then V per chunk) and ``rk [C, Hkv, D]`` once into a file under
    ``/dev/shm``; what travels through the queue is this small object (path, shapes, the per-layer ``cache_kwargs``
    with the template prefix and ``pooled_doc_ids``).  The receiver maps the file: ``kv_chunk_major`` / ``rk_chunk_major``
    give the mapped tensors for a straight copy into the bank, ``get_kvcache`` / ``get_router_kcache`` the
    reference-shaped ``[1, Hkv, C, D]`` views of the same bytes.  ``clear_kvcache`` (which the receive loop calls
    per block, src/msa_service.py:569) unmaps and removes the file."""

    def __init__(self, path: str, dtype: torch.dtype, n_kv_heads: int, head_dim: int, layer_chunks: dict, has_rk: dict,
                 cache_kwargs: dict, meta: dict):
        self.path, self.dtype, self.n_kv_heads, self.head_dim = path, dtype, n_kv_heads, head_dim
        self.layer_chunks, self.has_rk = dict(layer_chunks), dict(has_rk)
        self.cache_kwargs, self.meta = cache_kwargs, meta
        self._raw = None

    @staticmethod
    def _layer_bytes(c, h, d, esize, has_rk):
        return c * 2 * h * d * esize, (c * h * d * esize if has_rk else 0)

    @classmethod
    def write(cls, path: str, cache: SparseCache, router_layer_ids):
        """Move the pooled K / V / K_r of ``cache`` (``[1, Hkv, C, D]`` per router layer) into ``path``."""
        first_k = cache.key_cache[router_layer_ids[0]]
        dtype, h, d = first_k.dtype, first_k.shape[1], first_k.shape[3]
        layer_chunks, has_rk = {}, {}
        with open(path, "wb") as f:
            for layer in router_layer_ids:
                k, v = cache.get_kvcache(layer)
                rk = cache.get_router_kcache(layer)
                kv = torch.stack([k[0].permute(1, 0, 2), v[0].permute(1, 0, 2)], dim=1).contiguous().cpu()    # [C, 2, Hkv, D]
                f.write(kv.view(torch.uint8).numpy().tobytes() if kv.numel() else b"")
                if rk is not None:
                    f.write(rk[0].permute(1, 0, 2).contiguous().cpu().view(torch.uint8).numpy().tobytes())
                layer_chunks[layer], has_rk[layer] = int(k.shape[2]), rk is not None
            if f.tell() == 0:
                f.write(b"\0" * 16)
        meta = {k: v for k, v in cache.meta.items() if not str(k).startswith("_msa_b200_")}   # per-process scratch stays behind
        return cls(path, dtype, h, d, layer_chunks, has_rk, cache.cache_kwargs, meta)

    def __getstate__(self):
        state = dict(self.__dict__)
        state["_raw"] = None          # the mapping is per process
        return state

    def _map(self):
        if self._raw is None:
            self._raw = torch.from_file(self.path, shared=True, size=max(os.path.getsize(self.path), 1), dtype=torch.uint8)
        return self._raw

    def _offsets(self, layer_idx):
        esize = torch.empty((), dtype=self.dtype).element_size()
        off = 0
        for layer, c in self.layer_chunks.items():
            n_kv, n_rk = self._layer_bytes(c, self.n_kv_heads, self.head_dim, esize, self.has_rk[layer])
            if layer == layer_idx:
                return off, n_kv, n_rk, c
            off += n_kv + n_rk
        raise KeyError(layer_idx)

    def kv_chunk_major(self, layer_idx):
        off, n_kv, _, c = self._offsets(layer_idx)
        return self._map()[off:off + n_kv].view(self.dtype).view(c, 2, self.n_kv_heads, self.head_dim)

    def rk_chunk_major(self, layer_idx):
        off, n_kv, n_rk, c = self._offsets(layer_idx)
        if not n_rk:
            return None
        return self._map()[off + n_kv:off + n_kv + n_rk].view(self.dtype).view(c, self.n_kv_heads, self.head_dim)

    def get_kvcache(self, layer_idx):
        kv = self.kv_chunk_major(layer_idx)
        return kv[:, 0].permute(1, 0, 2).unsqueeze(0), kv[:, 1].permute(1, 0, 2).unsqueeze(0)

    def get_router_kcache(self, layer_idx):
        rk = self.rk_chunk_major(layer_idx)
        return None if rk is None else rk.permute(1, 0, 2).unsqueeze(0)

    def record_kwargs(self, layer_idx, kwargs):
        self.cache_kwargs.setdefault(layer_idx, {}).update(kwargs)

    def clear_kvcache(self):
        self._raw = None
        if os.path.exists(self.path):
            os.unlink(self.path)


def create_cache():
    return SparseCache()

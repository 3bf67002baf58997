"""Memory-Parallel service: the B200 counterpart of the reference's ``MSAService``.

Mirrors ``src/msa_service.py:1013-1314``.  The exchange pattern is redesigned for one NVSwitch
node (the reference issues seven collectives and five host synchronisations per routing
layer, :1105-1283):

  1. every rank folds its own queries (4x fewer bytes) and ONE all-gather lands every rank's
     folded queries in local HBM (reference: all-gather of unfolded, zero-padded q and mask);
  2. the fused kernel scores ALL ranks' queries against the local shard and selects the
     shard's top-k' per query;
  3. ONE all-gather of the candidates ``[3, B_all, k']`` (scores, local ids, global ids as planes of one buffer)
     replaces the two all-to-alls of candidates and the all-to-all of requests: every rank
     merges its own queries and knows each winner's owner;
  4. the requester reads the winners' K/V straight from the pinned host bank (every rank of
     the node maps every shard's bank), which removes the owner-side CPU gather and the
     variable-size all-to-all of payloads.
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from . import _cabi as A
from . import ops
from .memory import AttentionGeometry, Document, Memory, MemoryConfig, ModelConfig


class MemoryClientBase:
    """Interface the attention layer calls (src/msa_service.py:259-264)."""

    def get_template_prefix_kvcaches(self, layer_idx: int):
        raise NotImplementedError

    def doc_query(self, query_states: torch.Tensor, attention_mask: torch.Tensor, layer_idx: int):
        raise NotImplementedError


# ------------------------------------------------------------------------------------------
# Host-side pieces that do not touch a GPU (covered by the gloo tests)
# ------------------------------------------------------------------------------------------

def balanced_bucket_partition(docs: Sequence[Document], n_buckets: int) -> List[List[Document]]:
    """Greedy least-loaded partition of documents over ranks by chunk count, heaviest first
    (the reference's placement rule, src/msa_service.py:1452-1476)."""
    buckets: List[List[Document]] = [[] for _ in range(n_buckets)]
    loads = [0] * n_buckets
    for d in sorted(docs, key=lambda x: x.num_chunks, reverse=True):
        i = loads.index(min(loads))
        buckets[i].append(d)
        loads[i] += d.num_chunks
    return buckets


# Set to a list to collect a (start, end) pair of timing events around every all-gather (a profiled step);
# ``COLLECTIVE_PROBE_EXTERNAL`` makes them event-record nodes, so that they can be read after a CUDA-graph replay.
COLLECTIVE_PROBE: Optional[list] = None
COLLECTIVE_PROBE_EXTERNAL = False


def all_gather_cat(t: torch.Tensor, world: int, group=None) -> torch.Tensor:
    """All-gather equal-shaped tensors along a new leading rank axis ``[W, ...]``."""
    out = torch.empty((world,) + tuple(t.shape), dtype=t.dtype, device=t.device)
    if world == 1:
        out[0].copy_(t)
        return out
    probe = COLLECTIVE_PROBE
    if probe is not None:
        e0 = torch.cuda.Event(enable_timing=True, external=COLLECTIVE_PROBE_EXTERNAL)
        e0.record()
    dist.all_gather_into_tensor(out.view(-1), t.contiguous().view(-1), group=group)
    if probe is not None:
        e1 = torch.cuda.Event(enable_timing=True, external=COLLECTIVE_PROBE_EXTERNAL)
        e1.record()
        probe.append((e0, e1))
    return out


def build_directory(per_rank_doc_lens: Sequence[Sequence[int]]):
    """Node-wide document directory from every rank's ``doc_lens`` (slot 0 = dummy):
    ``(shard_doc_base[W], doc_chunk_offset[sum], doc_chunk_len[sum])`` as CPU tensors."""
    bases, offs, lens = [], [], []
    base = 0
    for ln in per_rank_doc_lens:
        ln = torch.as_tensor(list(ln), dtype=torch.long)
        bases.append(base)
        offs.append(torch.cumsum(torch.cat([torch.zeros(1, dtype=torch.long), ln[:-1]]), 0))
        lens.append(ln)
        base += ln.numel()
    return torch.tensor(bases, dtype=torch.long), torch.cat(offs), torch.cat(lens).to(torch.int32)


class SharedHostBank:
    """A shard's K/V bank in a POSIX shared-memory file so that every rank of the node can
    map and pin it.  ``create`` is called by the owner, ``open`` by the peers."""

    def __init__(self, path: str, shape, dtype: torch.dtype, create: bool):
        self.path, self.shape, self.dtype = path, tuple(shape), dtype
        n = 1
        for s in shape:
            n *= s
        self.nbytes = n * torch.empty((), dtype=dtype).element_size()
        if create:
            with open(path, "wb") as f:
                f.truncate(max(self.nbytes, 16))
        self._raw = torch.from_file(path, shared=True, size=max(self.nbytes, 16), dtype=torch.uint8)
        self.tensor = self._raw[: self.nbytes].view(dtype).view(self.shape)
        self.device_address = 0
        self._owner = create

    def register(self) -> int:
        import ctypes
        addr = ctypes.c_uint64(0)
        A.check(A.lib().msa_bank_register_host(self._raw.data_ptr(), max(self.nbytes, 16), ctypes.byref(addr)),
                "msa_bank_register_host")
        self.device_address = int(addr.value)
        return self.device_address

    def close(self):
        if self.device_address:
            A.lib().msa_bank_unregister_host(self._raw.data_ptr())
            self.device_address = 0
        if self._owner and os.path.exists(self.path):
            os.unlink(self.path)


# ------------------------------------------------------------------------------------------
class MSAService(Memory, MemoryClientBase):
    """One rank of the Memory-Parallel job (src/msa_service.py:1013-1314)."""

    def __init__(self, gpu_id: int, generate_config=None, model_config: Optional[ModelConfig] = None,
                 memory_config: Optional[MemoryConfig] = None, geometry: Optional[AttentionGeometry] = None,
                 world_size: Optional[int] = None, rank: Optional[int] = None, shard_top_k: Optional[int] = None,
                 group=None):
        super().__init__(gpu_id, generate_config, model_config, memory_config, geometry)
        if world_size is None:
            world_size = dist.get_world_size(group) if dist.is_initialized() else 1
        self.world_size = world_size
        self.rank = (dist.get_rank(group) if dist.is_initialized() else 0) if rank is None else rank
        self.group = group
        if world_size > 1 and not dist.is_initialized():
            raise A.MsaError("world_size > 1 needs an initialised torch.distributed process group (NCCL)")
        self.shard_top_k = shard_top_k or self.model_config.doc_top_k
        self.uniform_seqlen = False   # set when every rank is known to pass queries of equal length
        self._directory = None
        self._total_pinned = torch.zeros(1, dtype=torch.int64).pin_memory()
        self._status_pinned = torch.zeros(4, dtype=torch.int32).pin_memory()

    def setup_memory_client(self, model):
        """Inject this service into every module that has ``set_memory_client`` (:1057-1067)."""
        for _, module in model.named_modules():
            if callable(getattr(module, "set_memory_client", None)):
                module.set_memory_client(self)

    # ------------------------------------------------------------------ directory of all shards
    def publish_directory(self, peer_kv_addresses: Optional[dict] = None):
        """Build the node-wide directory the fetch kernel reads.  With one rank it is the local
        shard; with several, every rank contributes its ``doc_lens`` (all_gather_object) and
        ``peer_kv_addresses[layer]`` must list the device-visible address of every rank's bank
        (see ``SharedHostBank``)."""
        lens = self.block_desc.doc_lens_cpu.tolist()
        if self.world_size > 1:
            gathered = [None] * self.world_size
            dist.all_gather_object(gathered, lens, group=self.group)
        else:
            gathered = [lens]
        base, offs, ln = build_directory(gathered)
        kv_base = {}
        for layer in self.router_layer_ids:
            if peer_kv_addresses is not None:
                addrs = list(peer_kv_addresses[layer])
            else:
                if self.world_size > 1:
                    raise A.MsaError("publish_directory: peer_kv_addresses is required when world_size > 1")
                addrs = [self.blocks[layer].kv_device_address]
            kv_base[layer] = torch.tensor(addrs, dtype=torch.int64, device=self.device)
        self._directory = (base.to(self.device), offs.to(self.device), ln.to(self.device), kv_base)

    def share_host_banks(self, tag: str, shm_dir: str = "/dev/shm"):
        """Move this rank's K/V banks into shared-memory files, map and pin every peer's files, and
        publish the node-wide directory.  Collective: every rank calls it after building its shard."""
        g = self.geometry
        sizes = [self.block_desc.chunks()]
        if self.world_size > 1:
            sizes = [None] * self.world_size
            dist.all_gather_object(sizes, self.block_desc.chunks(), group=self.group)
        path = lambda w, layer: os.path.join(shm_dir, f"msa_b200_{tag}_r{w}_l{layer}.bank")
        shape = lambda w: (sizes[w], 2, g.num_key_value_heads, g.head_dim)
        own = {}
        for layer in self.router_layer_ids:
            blk = self.blocks[layer]
            bank = SharedHostBank(path(self.rank, layer), shape(self.rank), blk.kv.dtype, create=True)
            bank.tensor.copy_(blk.kv)
            blk.kv = bank.tensor
            own[layer] = bank
        if self.world_size > 1:
            dist.barrier(group=self.group)
        self._shared_banks, addresses = [], {}
        for layer in self.router_layer_ids:
            banks = [own[layer] if w == self.rank else
                     SharedHostBank(path(w, layer), shape(w), self.blocks[layer].kv.dtype, create=False)
                     for w in range(self.world_size)]
            addresses[layer] = [b.register() for b in banks]
            self.blocks[layer].kv_device_address = addresses[layer][self.rank]
            self._shared_banks.extend(banks)
        self.publish_directory(peer_kv_addresses=addresses)

    def close_host_banks(self):
        """Unpin and (for the owner) unlink the shared banks.  Collective when world_size > 1."""
        torch.cuda.synchronize(self.device)
        if self.world_size > 1:
            dist.barrier(group=self.group)
        for b in getattr(self, "_shared_banks", []):
            b.close()
        self._shared_banks = []

    # ------------------------------------------------------------------ the layer-facing call
    def _gather_querys(self, query_states: torch.Tensor, query_mask: torch.Tensor, l2_normalize: bool = False,
                       all_valid: bool = False):
        """Fold local queries, agree on the padded length, all-gather (:1088-1131).
        Returns ``(q_folded_all[W*B*s_pad, Hkv*D], row_bias_all, s_pad, B)``."""
        b, hq, s, d = query_states.shape
        qr = self.query_reduce_method
        s_common = s
        if self.world_size > 1 and qr == "max" and not self.uniform_seqlen:
            lens = all_gather_cat(torch.tensor([s], device=self.device, dtype=torch.long), self.world_size, self.group)
            s_common = int(lens.max().item())
        s_pad = ops.route_s_pad(s_common, qr)
        qf, bias, _ = ops.fold_queries(query_states, query_mask, self.num_key_value_groups, query_reduce=qr,
                                       s_pad=s_pad, l2_normalize=l2_normalize)
        if self.world_size > 1:
            qf = all_gather_cat(qf, self.world_size, self.group).view(-1, qf.shape[1])
            if all_valid and s == s_pad:
                # every rank's mask is all ones and nothing is padded: the gathered bias is zero, no collective needed
                key = (self.world_size * b * s_pad,)
                cached = self.__dict__.get("_zero_bias")
                if cached is None or cached.shape != key:
                    cached = self._zero_bias = torch.zeros(key, dtype=torch.float32, device=self.device)
                bias = cached
            else:
                bias = all_gather_cat(bias, self.world_size, self.group).view(-1)
        return qf, bias, s_pad, b

    def route(self, query_states: torch.Tensor, query_mask: torch.Tensor, layer_idx: int, l2_normalize: bool = False,
              all_valid: bool = False):
        """Steps 1-4 of ``doc_query`` (:1149-1191): returns the merged winners of this rank's own
        queries ``(scores[B,k], local_ids[B,k] (-1 invalid), global_ids[B,k], owner_rank[B,k])``.
        ``l2_normalize``: the queries are raw projections; normalise every head inside the fold kernel
        (what the layer does with ``F.normalize`` before calling ``doc_query`` in cosine mode).
        ``all_valid``: the caller guarantees that every rank's ``query_mask`` is all ones (a decode step), which
        saves the all-gather of the row bias."""
        b, hq, s, d = query_states.shape
        scale = self.scaling if self.scaling > 0 else 1.0
        n_all = self.world_size * b
        if self.head_reduce_method == "max":
            return self._route_unfolded(query_states, query_mask, layer_idx, l2_normalize, scale)
        if s == 1 and self.chunk_reduce_method == "max" and self.blocks[layer_idx].rk_blocked is not None:
            self.prepare_table(n_all)      # decode step over blocked keys (table path): the reset overlaps fold + all-gather
        qf, bias, s_pad, _ = self._gather_querys(query_states, query_mask, l2_normalize, all_valid)
        if self.world_size > 1:
            # the selection writes straight into one buffer (scores, local ids, global ids as planes), ONE
            # all-gather moves it, and the merge reads the gathered planes in place
            k_eff = min(self.shard_top_k, self.block_desc.nr_docs + 1)
            cb = self.__dict__.get("_cand_buf")
            if cb is None or tuple(cb[0].shape) != (3, n_all, k_eff):
                cb = self._cand_buf = ops.candidate_buffer(n_all, k_eff, self.device)
            self.score_folded(layer_idx, qf, bias, n_all, s_pad, hq, self.shard_top_k, scale=scale, out=cb[1:])
            sc, li, gi = ops.candidate_views(all_gather_cat(cb[0], self.world_size, self.group))   # [W, B_all, k']
        else:
            sc, li, gi = self.score_folded(layer_idx, qf, bias, n_all, s_pad, hq, self.shard_top_k, scale=scale)
            sc, li, gi = sc.unsqueeze(0), li.unsqueeze(0), gi.unsqueeze(0)
        return ops.topk_merge(sc, li, gi, self.model_config.doc_top_k, seq_offset=self.rank * b, n_seq=b)

    def _route_unfolded(self, query_states, query_mask, layer_idx: int, l2_normalize: bool, scale: float):
        """``route`` for head_reduce "max": a max over heads cannot be folded into one contraction, so the
        UNFOLDED queries and their masks are all-gathered (padded to the longest query, as the reference does,
        :1088-1131) and scored per head."""
        b, hq, s, d = query_states.shape
        if l2_normalize:
            query_states = torch.nn.functional.normalize(query_states, p=2, dim=-1)
        mask = query_mask.reshape(b, s)
        if self.world_size > 1:
            s_common = s
            if not self.uniform_seqlen:
                lens = all_gather_cat(torch.tensor([s], device=self.device, dtype=torch.long), self.world_size, self.group)
                s_common = int(lens.max().item())
            if s_common > s:
                query_states = torch.nn.functional.pad(query_states, (0, 0, 0, s_common - s))
                mask = torch.nn.functional.pad(mask, (0, s_common - s), value=False)
            q_all = all_gather_cat(query_states.contiguous(), self.world_size, self.group).view(-1, hq, s_common, d)
            m_all = all_gather_cat(mask.to(torch.uint8).contiguous(), self.world_size, self.group).view(-1, s_common)
            k_eff = min(self.shard_top_k, self.block_desc.nr_docs + 1)
            n_all = self.world_size * b
            cb = self.__dict__.get("_cand_buf")
            if cb is None or tuple(cb[0].shape) != (3, n_all, k_eff):
                cb = self._cand_buf = ops.candidate_buffer(n_all, k_eff, self.device)
            self.score_unfolded(layer_idx, q_all, m_all, self.shard_top_k, scale=scale, out=cb[1:])
            sc, li, gi = ops.candidate_views(all_gather_cat(cb[0], self.world_size, self.group))
        else:
            sc, li, gi = self.score_unfolded(layer_idx, query_states, mask, self.shard_top_k, scale=scale)
            sc, li, gi = sc.unsqueeze(0), li.unsqueeze(0), gi.unsqueeze(0)
        return ops.topk_merge(sc, li, gi, self.model_config.doc_top_k, seq_offset=self.rank * b, n_seq=b)

    def fetch(self, winner_local: torch.Tensor, winner_rank: torch.Tensor, layer_idx: int,
              max_entries: Optional[int] = None, max_ctas: int = 0):
        """Steps 5-8 of ``doc_query`` (:1193-1312): K/V of the winners from the pinned host banks.
        Returns ``(final_k[Hkv, sumN, D], final_v, n_sel[B])``.  By default one 8-byte read-back sizes
        the result (the reference synchronises five times here).  With ``max_entries`` the outputs
        are allocated for that many entries instead, nothing is read back and the call never blocks
        the host: ``(final_k[Hkv, max_entries, D], final_v, n_sel[B], total[1])``.  ``max_ctas`` caps the
        gather's grid (see ``ops.gather_run``): leave 0 next to prefill kernels, 24 inside a decode step."""
        if self._directory is None:
            self.publish_directory()
        base, offs, ln, kv_base = self._directory
        g = self.geometry
        blk = self.blocks[layer_idx]
        chunk_bytes = 2 * g.num_key_value_heads * g.head_dim * blk.kv.element_size()
        plan, n_sel, total = ops.gather_plan(winner_local, winner_rank, self.world_size, base, offs, ln,
                                             kv_base[layer_idx], chunk_bytes, total_host=None, status=self._status)
        if max_entries is not None:
            k, v = ops.gather_run(plan, blk.kv.dtype, g.num_key_value_heads, g.head_dim, max_entries, max_ctas)
            return k, v, n_sel, total
        # one read-back sizes the result; the status words of this layer's routing and plan ride along
        self._total_pinned.copy_(total, non_blocking=True)
        self._status_pinned.copy_(self._status, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        self._raise_on_status(self._status_pinned.tolist())
        n = int(self._total_pinned.item())
        k, v = ops.gather_run(plan, blk.kv.dtype, g.num_key_value_heads, g.head_dim, n, max_ctas)
        return k, v, n_sel

    def fetch_into(self, winner_local: torch.Tensor, winner_rank: torch.Tensor, layer_idx: int, k_cache: torch.Tensor,
                   v_cache: torch.Tensor, first_position: int, room: int, max_ctas: int = 0,
                   resident: Optional[torch.Tensor] = None):
        """``fetch`` for a decode loop: the winners' K/V go straight into positions ``first_position ..
        first_position + room`` of ``[B, Hkv, L, D]`` caches, sample b's entries into row b (no packed staging
        buffer, no copies afterwards, no read-back).  A sample whose documents hold more than ``room`` entries
        is cut; one that holds fewer leaves the tail of its segment as it was.  ``resident`` (int64 ``[B, k]``, -1
        before the first step, the caller's for this layer's segment): documents a sample selected again keep their
        entries and only the new ones are read from the host (``ops.gather_plan``).  Returns ``n_sel[B]`` (entries
        valid per sample, on the device)."""
        if self._directory is None:
            self.publish_directory()
        base, offs, ln, kv_base = self._directory
        g = self.geometry
        blk = self.blocks[layer_idx]
        chunk_bytes = 2 * g.num_key_value_heads * g.head_dim * blk.kv.element_size()
        plan, n_sel, _ = ops.gather_plan(winner_local, winner_rank, self.world_size, base, offs, ln, kv_base[layer_idx],
                                         chunk_bytes, sample_stride=room, status=self._status, resident=resident)
        ops.gather_run(plan, blk.kv.dtype, g.num_key_value_heads, g.head_dim, room, max_ctas,
                       out=(k_cache, v_cache, first_position))
        return n_sel

    def doc_query(self, query_states: torch.Tensor, query_mask: torch.Tensor, layer_idx: int):
        """src/msa_service.py:1133-1314.  query_states ``[B, Hq, S, D]`` (already L2-normalised in
        cosine mode), query_mask ``[B, S]`` bool.  Returns ``(final_k[Hkv, sumN, D], final_v,
        final_scores[B, k] float32, num_selected_chunks_per_sample[B], final_selected_doc_ids[B, k])``.
        A sample's entries are ordered by (owner rank, local doc id, chunk) as in the reference.
        Winners whose score is <= -1e9 select nothing."""
        scores, local, glob, rank = self.route(query_states, query_mask, layer_idx)
        k, v, n_sel = self.fetch(local, rank, layer_idx)
        return k, v, scores, n_sel, glob

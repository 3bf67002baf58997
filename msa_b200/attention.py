"""``MemorySparseAttention``: the B200 counterpart of the reference's attention layer for inference.

Mirrors ``src/msa/memory_sparse_attention.py:20-405`` (constructor, ``set_memory_client``,
``forward`` dispatch on the stage recorded in the cache, the three inference branches).  Same
constructor arguments, same module / parameter names (so a reference checkpoint's state dict
loads), same cache protocol (``cache_kwargs`` / ``meta`` / ``record_kwargs`` / ``update`` /
``update_router_kcache``).

What runs where (every attention of the path is one of this package's kernels; no library attention call):
  * stage 1: projections, norms and RoPE stay PyTorch as in the reference; chunk bookkeeping, the
    intra-document causal attention and all pooling run on this package's kernels.  In bf16 with
    head_dim 128: documents of 128 tokens and more go to the tcgen05 attention kernel (blocks with masked
    tokens inside documents: over each document's span of memory with a bitmap of the tokens that take
    part; K, V, K_r pooled by the pooling kernel), blocks of shorter documents to the mma.sync kernel
    that takes the K / V chunk means in the same pass; fp32 and other head sizes: the general CUDA-core
    attention kernel + the pooling kernel;
  * stage 2: routing, merge and fetch happen inside ``memory_client.doc_query`` (this package's
    ``MSAService``); one kernel assembles [template | retrieved | query] into the left-padded
    compact cache (allocated with room to append in place) and the prefill attention kernel reads it
    there (bf16 / head_dim 128: the tcgen05 kernel when every sequence's question tokens are one run of
    consecutive tokens, as left- or right-padded questions are, the mma.sync kernel otherwise; other
    dtypes and head sizes: the general kernel);
  * decode: this package's flash-decode kernel, in-place append, no ``torch.cat`` / ``repeat_kv``;
    the multi-token, non-causal segments of ``qa_mode`` are appended by one kernel and attended by the
    prefill kernels without their causal mask.
The training forward (``_forward``) is out of scope and raises.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F
from transformers.models.qwen3.modeling_qwen3 import Qwen3Attention, apply_rotary_pos_emb

from . import _cabi as A
from . import ops

class MemorySparseAttention(Qwen3Attention):
    #: extra cache positions reserved for tokens appended during decode
    decode_reserve = 512

    def __init__(self, config, layer_idx: int):
        super().__init__(config=config, layer_idx=layer_idx)
        A.lib()  # no kernels, no layer
        mc = config.msa_config
        self.layer_idx = layer_idx
        self.top_k_docs = mc.top_k_docs
        self.pooling_kernel_size = mc.pooling_kernel_size
        ridx = mc.router_layer_idx
        self.router_layer_idx = list(range(config.num_hidden_layers)) if ridx == "all" else [int(i) for i in ridx.split(",")]
        self.is_router_layer = self.layer_idx in self.router_layer_idx
        self.head_reduce_method = mc.head_reduce_method
        self.query_reduce_method = mc.query_reduce_method
        self.chunk_reduce_method = mc.chunk_reduce_method
        self.decouple_pooling_mode = mc.decouple_pooling_mode
        self.aux_loss_method = mc.aux_loss_method
        self.decouple_router = mc.decouple_router
        if self.is_router_layer and self.decouple_router:
            self.router_k_proj = nn.Sequential(
                nn.Linear(config.hidden_size, config.num_key_value_heads * self.head_dim, bias=False))
            self.router_q_proj = nn.Sequential(
                nn.Linear(config.hidden_size, config.num_attention_heads * self.head_dim, bias=False))
        self.num_kv_heads = config.num_key_value_heads
        self.template_prefix_kcache = None
        self.template_prefix_vcache = None
        self.memory_client = None

    def set_memory_client(self, memory_client):
        self.memory_client = memory_client

    def forward(self, hidden_states, doc_ids, attention_mask=None, position_embeddings=None, past_key_value=None,
                **kwargs):
        if self.training:
            raise NotImplementedError("msa_b200.MemorySparseAttention implements the inference branches only")
        if past_key_value is None:
            raise Exception("error!")  # the reference's message (memory_sparse_attention.py:97)
        return self.forward_with_kvcache_for_batch_parrallel(hidden_states, doc_ids, attention_mask,
                                                             position_embeddings, past_key_value, **kwargs)

    # ------------------------------------------------------------------------------------
    def forward_with_kvcache_for_batch_parrallel(self, hidden_states, doc_ids, attention_mask=None,
                                                 position_embeddings=None, past_key_value=None, **kwargs):
        bsz, q_len, _ = hidden_states.shape
        hidden_shape = (bsz, q_len, -1, self.head_dim)
        query_states = self.q_norm(self.q_proj(hidden_states).view(hidden_shape)).transpose(1, 2)
        key_states = self.k_norm(self.k_proj(hidden_states).view(hidden_shape)).transpose(1, 2)
        value_states = self.v_proj(hidden_states).view(hidden_shape).transpose(1, 2)
        cos, sin = position_embeddings
        query_states, key_states = apply_rotary_pos_emb(query_states, key_states, cos, sin)
        stage = past_key_value.cache_kwargs[self.layer_idx]["stage"]
        if stage == "prefill_stage1":
            return self._stage1(hidden_states, doc_ids, attention_mask, past_key_value, query_states, key_states,
                                value_states)
        if stage == "prefill_stage2":
            return self._stage2(hidden_states, doc_ids, attention_mask, past_key_value, query_states, key_states,
                                value_states)
        return self._decode(attention_mask, past_key_value, query_states, key_states, value_states)

    # ------------------------------------------------------------------------------------ stage 1
    def _bookkeeping(self, doc_ids, attention_mask, cache):
        """Chunk tables of this block; computed once and shared by every layer through cache.meta."""
        key = (doc_ids.data_ptr(), tuple(doc_ids.shape))
        hit = cache.meta.get("_msa_b200_bookkeeping")
        if hit is None or hit[0] != key:
            tok, off, pooled = ops.chunk_bookkeeping(doc_ids, attention_mask, self.pooling_kernel_size)
            hit = (key, tok, off, pooled)
            cache.meta["_msa_b200_bookkeeping"] = hit
        return hit[1], hit[2], hit[3]

    def _segments(self, doc_ids, attention_mask, cache):
        """Token lists and segment offsets of the document tokens and of the template tokens of this block
        (one segment per (row, document) run / per row), the longest segment and whether every segment is a
        run of consecutive tokens; computed once and shared by every layer."""
        prev = cache.meta.get("_msa_b200_attn_status")
        if prev is not None and int(prev[0].item()) != 0:
            raise A.MsaError("a bounded barrier wait ran out inside doc_attn_tc_kernel (stage-1 attention output invalid)")
        key = (doc_ids.data_ptr(), attention_mask.data_ptr(), tuple(doc_ids.shape))
        hit = cache.meta.get("_msa_b200_segments")
        if hit is None or hit[0] != key:
            s = doc_ids.shape[1]
            valid = attention_mask == 1

            def table(mask, ids):
                tok = torch.nonzero(mask.flatten()).flatten()
                if tok.numel() == 0:
                    return tok.to(torch.int32), torch.zeros(1, dtype=torch.int32, device=tok.device), 0, True
                gid = (tok // s) * (int(ids.max().item()) + 2) + ids.flatten()[tok]
                _, counts = torch.unique_consecutive(gid, return_counts=True)
                off = F.pad(counts.cumsum(0), (1, 0))
                first, last = tok[off[:-1]], tok[off[1:] - 1]
                runs = bool(((last - first == counts - 1) & (first // s == last // s)).all().item())
                return tok.to(torch.int32), off.to(torch.int32), int(counts.max().item()), runs
            listed = (doc_ids > 0) & valid
            docs = table(listed, doc_ids)
            spans = None
            if not docs[3] and docs[0].numel() > 0:      # masked tokens inside documents: spans + bitmap for the tcgen05 kernel
                spans = ops.document_spans(docs[0], docs[1]) + (ops.token_bitmap(listed),)
            hit = (key, docs, table((doc_ids == -2) & valid, torch.zeros_like(doc_ids)), spans)
            cache.meta["_msa_b200_segments"] = hit
        return hit[1], hit[2], hit[3]

    def _valid_runs(self, valid, cache):
        """Device flags ``[2]`` int32: whether the valid tokens of every row are one run of consecutive tokens (what the
        tcgen05 context kernel takes), and the status word of the earlier tensor-core attention launches.  The caller
        reads them back together with whatever else it needs on the host."""
        s = valid.shape[1]
        idx = torch.arange(s, device=valid.device).unsqueeze(0)
        first = torch.where(valid, idx, s).amin(dim=1)
        last = torch.where(valid, idx, -1).amax(dim=1)
        runs = (((last - first + 1) == valid.sum(dim=1)) | (last < 0)).all().to(torch.int32)
        status = cache.meta.setdefault("_msa_b200_attn_status", torch.zeros(4, dtype=torch.int32, device=valid.device))
        return torch.stack([runs, status[0]])

    @staticmethod
    def _check_attn_status(word):
        if word != 0:
            raise A.MsaError("a bounded barrier wait ran out inside doc_attn_tc_kernel (attention output invalid)")

    def _stage1(self, hidden_states, doc_ids, attention_mask, cache, query_states, key_states, value_states):
        """src/msa/memory_sparse_attention.py:137-243."""
        bsz, q_len, _ = hidden_states.shape
        device, dtype = hidden_states.device, hidden_states.dtype
        hidden_shape = (bsz, q_len, -1, self.head_dim)
        n_heads = self.config.num_attention_heads
        tensor_cores = dtype == torch.bfloat16 and self.head_dim == 128
        if self.is_router_layer and bsz != 1:
            raise A.MsaError("stage 1 pools one block per call (the reference's worker uses batch size 1)")

        # intra-document and template causal attention (:216-241)
        attn_output = torch.zeros((bsz, q_len, n_heads * self.head_dim), device=device, dtype=dtype)
        pooled_k = pooled_v = pooled_rk = pooled_doc_ids = None
        (tok_d, off_d, max_d, runs_d), (tok_t, off_t, max_t, _), spans = self._segments(doc_ids, attention_mask, cache)
        tc_ok = tensor_cores and max_d >= 128 and ops.doc_attention_tc_supported(query_states, key_states, value_states)
        if tc_ok and runs_d:
            # unmasked documents: attention on the tcgen05 kernel (K and V are pooled by the pooling kernel below)
            status = cache.meta.setdefault("_msa_b200_attn_status", torch.zeros(4, dtype=torch.int32, device=device))
            ops.doc_attention_tc(query_states, key_states, value_states, tok_d, off_d, max_d, out=attn_output,
                                 scale=self.scaling, status=status)
        elif tc_ok and spans is not None:
            # masked tokens inside documents: the same kernel over each document's span of memory with a bitmap of
            # the tokens that take part (masked rows of attn_output stay zero)
            status = cache.meta.setdefault("_msa_b200_attn_status", torch.zeros(4, dtype=torch.int32, device=device))
            ops.doc_attention_tc_masked(query_states, key_states, value_states, spans[0], spans[1], spans[2], spans[3],
                                        out=attn_output, scale=self.scaling, status=status)
        elif tensor_cores and self.is_router_layer and self.pooling_kernel_size % 32 == 0:
            # K and V are pooled from the tiles the attention kernel stages anyway
            tok, off, pooled_doc_ids = self._bookkeeping(doc_ids, attention_mask, cache)
            _, pooled_k, pooled_v = ops.doc_attention_pool(
                query_states, key_states, value_states, tok, off_d, max_d, out=attn_output, chunk_offsets=off,
                pool_size=self.pooling_kernel_size, head_major_out=True, scale=self.scaling)
        else:   # bf16 / 128 without pooling here, or any other dtype / head size on the general kernel
            ops.doc_attention_pool(query_states, key_states, value_states, tok_d, off_d, max_d, out=attn_output,
                                   scale=self.scaling)
        ops.doc_attention_pool(query_states, key_states, value_states, tok_t, off_t, max_t, out=attn_output,
                               scale=self.scaling)

        if self.is_router_layer:
            tok, off, pooled_doc_ids = self._bookkeeping(doc_ids, attention_mask, cache)
            if pooled_k is None:
                pooled_k = ops.pool_chunks(key_states, off, tok, head_major_out=True)
                pooled_v = ops.pool_chunks(value_states, off, tok, head_major_out=True)
            cosine = self.aux_loss_method == "INFONCE"
            if self.decouple_router:
                r_k_raw = self.router_k_proj(hidden_states).view(hidden_shape).transpose(1, 2)
                pooled_rk = ops.pool_chunks(r_k_raw, off, tok, l2_normalize=cosine, head_major_out=True)
            elif cosine:
                pooled_rk = F.normalize(pooled_k, p=2, dim=-1)
        n_template = int((doc_ids == -2).sum())
        kw = {"template_prefix_kcache": key_states[:, :, :n_template],
              "template_prefix_vcache": value_states[:, :, :n_template]}
        if self.is_router_layer:
            pooled_k, pooled_v = cache.update(pooled_k, pooled_v, self.layer_idx)
            kw.update({"doc_id_bias": doc_ids.shape[1], "pooled_doc_ids": pooled_doc_ids,
                       "prefill_stage1_kvcache_size": pooled_k.shape[2]})
            if pooled_rk is not None:
                cache.update_router_kcache(pooled_rk, self.layer_idx)
        cache.record_kwargs(self.layer_idx, kw)
        return self.o_proj(attn_output), None

    def _stage2(self, hidden_states, doc_ids, attention_mask, cache, query_states, key_states, value_states):
        """src/msa/memory_sparse_attention.py:245-359."""
        bsz, q_len, _ = hidden_states.shape
        device, dtype = hidden_states.device, hidden_states.dtype
        hidden_shape = (bsz, q_len, -1, self.head_dim)
        n_heads, n_kv, d = self.config.num_attention_heads, self.config.num_key_value_heads, self.head_dim
        cache_kwargs = cache.cache_kwargs[self.layer_idx]
        if self.memory_client is not None:
            if self.template_prefix_kcache is None:
                tk, tv = self.memory_client.get_template_prefix_kvcaches(self.layer_idx)
                self.template_prefix_kcache, self.template_prefix_vcache = tk.to(device), tv.to(device)
            template_k, template_v = self.template_prefix_kcache, self.template_prefix_vcache
        else:
            template_k = cache_kwargs["template_prefix_kcache"].to(device)
            template_v = cache_kwargs["template_prefix_vcache"].to(device)

        final_k = final_v = None
        if self.is_router_layer:
            routing_q = (self.router_q_proj(hidden_states).view(hidden_shape).transpose(1, 2)
                         if self.decouple_router else query_states)
            if self.aux_loss_method == "INFONCE":
                routing_q = F.normalize(routing_q, p=2, dim=-1)
            query_mask = (doc_ids == 0) & (attention_mask == 1)
            final_k, final_v, final_scores, n_sel, final_ids = self.memory_client.doc_query(routing_q, query_mask,
                                                                                          self.layer_idx)
            if cache.meta.get("require_recall_topk", False):
                ids, scores = final_ids.cpu().tolist(), final_scores.cpu().tolist()
                cache_kwargs["recall_topk"] = [{"topk_doc_ids": ids[i], "score": scores[i]} for i in range(bsz)]
        else:
            n_sel = torch.zeros(bsz, dtype=torch.long, device=device)

        # One kernel builds the left-padded compact cache (reference :299-351) in storage with room to
        # append decode tokens; attention then reads it in place (bf16 / head_dim 128: own kernel).
        valid_q = attention_mask == 1
        num_q = valid_q.sum(dim=1)
        t_len = template_k.shape[2]
        kv_lengths = t_len + n_sel + num_q
        tc = dtype == torch.bfloat16 and d == 128
        if tc:   # one read-back for the cache size, the run check and the status of earlier launches
            max_kv, runs, word = torch.cat([kv_lengths.max().reshape(1).to(torch.int32), self._valid_runs(valid_q, cache)]).tolist()
            self._check_attn_status(word)
            tc = bool(runs)
        else:
            max_kv = int(kv_lengths.max())
        reserve = int(cache.meta.get("max_generate_tokens", self.decode_reserve))
        k_store, v_store, kv_start, kv_len, q_tok, n_valid, _ = ops.assemble_context(
            template_k, template_v, final_k, None if final_v is None else final_v.to(device), n_sel, key_states,
            value_states, valid_q, max_kv, reserve)
        left_pad_mask = torch.arange(max_kv, device=device).unsqueeze(0) >= (max_kv - kv_lengths.unsqueeze(1))
        # question tokens that form one run per sequence (left / right padding): tcgen05 kernel; else mma.sync
        status = cache.meta["_msa_b200_attn_status"] if tc else None
        attn_output = ops.sparse_prefill_attn(query_states, k_store, v_store, kv_start, kv_len, q_tok, n_valid, self.scaling,
                                              q_runs=tc, status=status)
        cache_kwargs.update({
            "compacked_key_cache": k_store[:, :, :max_kv], "compacked_value_cache": v_store[:, :, :max_kv],
            "kv_lengths": kv_lengths, "attention_mask": left_pad_mask,
            "_msa_b200_store": (k_store, v_store, kv_start, kv_len),
        })
        cache.record_kwargs(self.layer_idx, cache_kwargs)
        return self.o_proj(attn_output), None

    # ------------------------------------------------------------------------------------ decode
    def _decode(self, attention_mask, cache, query_states, key_states, value_states):
        """src/msa/memory_sparse_attention.py:361-405."""
        cache_kwargs = cache.cache_kwargs[self.layer_idx]
        if "compacked_key_cache" not in cache_kwargs:
            raise ValueError("compact KV cache not found: did prefill stage 2 run?")
        bsz, n_heads, q_len, d = query_states.shape
        store = cache_kwargs.get("_msa_b200_store")
        cur_len = cache_kwargs["compacked_key_cache"].shape[2]
        if store is None or cur_len + q_len > store[0].shape[2]:
            store = self._adopt_cache(cache_kwargs, q_len)
        k_store, v_store, kv_start, kv_len = store
        # one token per sequence, all of them real: the flash-decode kernel.  A caller that feeds masked single tokens
        # (samples that wait in the interleave loop) says so in meta["step_all_valid"]; those steps, like qa_mode
        # segments, go through the segment path, which stores only the unmasked tokens.
        if q_len == 1 and not cache.meta.get("qa_mode", False) and cache.meta.get("step_all_valid", True):
            out = ops.sparse_decode_attn(query_states[:, :, 0], k_store, v_store, kv_len, key_states[:, :, 0],
                                         value_states[:, :, 0], kv_start=kv_start)
            attn_output = out.view(bsz, 1, n_heads * d)
            kv_len = kv_len + 1
            cache_kwargs["kv_lengths"] = cache_kwargs["kv_lengths"] + 1
        else:
            # qa_mode segments (:375-380): every token of the segment attends, without a causal mask, to the cache
            # and to the segment's own unmasked tokens.  One kernel appends the unmasked tokens in place (kv_len
            # grows by their number; masked tokens are never attended to, so they are not stored and a sequence's
            # valid entries stay one contiguous run), the prefill kernel attends without its causal mask.
            valid = attention_mask.reshape(bsz, q_len) == 1
            q_tok, num_q, _ = ops.append_segment(key_states, value_states, valid, k_store, v_store, kv_start, kv_len)
            # segments of 16 tokens and more whose unmasked tokens form one run per sequence: tcgen05 kernel
            tc = q_len >= 16 and query_states.dtype == torch.bfloat16 and d == 128
            if tc:
                runs, word = self._valid_runs(valid, cache).tolist()
                self._check_attn_status(word)
                tc = bool(runs)
            status = cache.meta["_msa_b200_attn_status"] if tc else None
            attn_output = ops.sparse_prefill_attn(query_states, k_store, v_store, kv_start, kv_len, q_tok, num_q,
                                                  self.scaling, causal=False, q_runs=tc, status=status)
            pos = torch.arange(cur_len + q_len, device=k_store.device).unsqueeze(0)
            cache_kwargs["attention_mask"] = (pos >= kv_start.unsqueeze(1)) & (pos < (kv_start + kv_len).unsqueeze(1))
            cache_kwargs["kv_lengths"] = kv_len.to(cache_kwargs["kv_lengths"].dtype)
        cache_kwargs["compacked_key_cache"] = k_store[:, :, :cur_len + q_len]
        cache_kwargs["compacked_value_cache"] = v_store[:, :, :cur_len + q_len]
        cache_kwargs["_msa_b200_store"] = (k_store, v_store, kv_start, kv_len)
        cache.record_kwargs(self.layer_idx, cache_kwargs)
        return self.o_proj(attn_output), None

    def _adopt_cache(self, cache_kwargs, q_len):
        """Take over a compact cache that was built elsewhere (or has run out of room): copy it once
        into storage with spare positions; from then on tokens are appended in place."""
        ck, cv = cache_kwargs["compacked_key_cache"], cache_kwargs["compacked_value_cache"]
        b, h, cur, d = ck.shape
        cap = cur + max(q_len, self.decode_reserve)
        k_store = torch.zeros((b, h, cap, d), dtype=ck.dtype, device=ck.device)
        v_store = torch.zeros((b, h, cap, d), dtype=cv.dtype, device=cv.device)
        k_store[:, :, :cur], v_store[:, :, :cur] = ck, cv
        prev = cache_kwargs.get("_msa_b200_store")
        if prev is not None:      # our own storage, out of room: positions and lengths stay what they are
            return k_store, v_store, prev[2], prev[3]
        kv_len = cache_kwargs["kv_lengths"].to(torch.int32)
        return k_store, v_store, (cur - kv_len).to(torch.int32), kv_len      # a left-padded cache of the reference

"""Generate the golden fixtures of this folder from the EverMind-AI/MSA reference itself.

Run in a container that has the reference checked out (read-only is fine):

    python tests/golden/make_golden.py --reference /path/to/MSA

The reference is imported unmodified.  Two names removed from transformers 5.x are
injected into ``transformers.cache_utils`` so that ``src/utils/cache.py:11`` imports (only
its unused quantized cache needs them), ``flash_attn_varlen_func`` (third party, CUDA only)
is replaced by an SDPA loop with bottom-right-aligned causal masking, and on a GPU-less box
``torch.cuda.current_stream`` is stubbed (``src/msa_service.py:1272`` synchronises it).
Everything is fp32 on the CPU.  Inputs AND outputs are stored, so the tests that consume
the ``.npz`` files need neither the reference nor this script.
"""
import argparse
import os
import sys
from types import SimpleNamespace

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def import_reference(path):
    sys.path.insert(0, path)
    import transformers.cache_utils as cu
    for n in ("QuantoQuantizedCache", "QuantizedCacheConfig"):
        if not hasattr(cu, n):
            setattr(cu, n, type(n, (), {}))
    import src.msa_service as svc
    import src.msa.memory_sparse_attention as msa_layer
    from src.msa.configuration_msa import MSAConfig
    return svc, msa_layer, MSAConfig


def save(name, **arrays):
    out = {}
    for k, v in arrays.items():
        if torch.is_tensor(v):
            v = v.detach().cpu().numpy()
        out[k] = np.asarray(v)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print("wrote", name, {k: v.shape for k, v in out.items()})


def make_memory(svc, chunks_per_doc, global_ids, rk, k, v, top_k, reduce=("mean", "max", "max"),
                cls=None, slice_chunks=16):
    cls = cls or svc.Memory
    docs = [svc.Document(doc="", doc_id=g, num_chunks=n) for g, n in zip(global_ids, chunks_per_doc)]
    m = object.__new__(cls)
    m.device = "cpu"
    m.gpu_id = 0
    m.router_layer_ids = [0]
    m.head_reduce_method, m.query_reduce_method, m.chunk_reduce_method = reduce
    m.model_config = SimpleNamespace(doc_top_k=top_k)
    m.block_desc = svc.BlockDesc()
    m.block_desc.init_docs(docs, "cpu")
    m.block_desc.pool_ids = torch.repeat_interleave(torch.arange(1, len(docs) + 1), torch.tensor(chunks_per_doc))
    m.blocks = {0: svc.BlockData(k=k, v=v, rk=rk)}
    m._generate_slice(slice_chunks)
    return m


def gen_pooling(svc, msa_layer):
    g = torch.Generator().manual_seed(101)
    p = 16
    doc_lens = [50, 16, 33, 1, 64]
    t_template = 3
    ids = [-2] * t_template
    for i, n in enumerate(doc_lens):
        ids += [i + 1] * n
    doc_ids = torch.tensor([ids])
    t = doc_ids.shape[1]
    attention_mask = torch.ones_like(doc_ids)
    h, d = 2, 128
    k = torch.randn(1, h, t, d, generator=g)
    v = torch.randn(1, h, t, d, generator=g)
    # the reference's inline bookkeeping (memory_sparse_attention.py:138-163), executed verbatim
    max_doc_id = int(doc_ids.max().item())
    mask = (doc_ids > 0) & (attention_mask == 1)
    doc_indices = torch.nonzero(mask, as_tuple=False)
    gdi = doc_indices[:, 0] * (max_doc_id + 1) + doc_ids[mask]
    _, counts = torch.unique_consecutive(gdi, return_counts=True)
    offsets = torch.zeros(counts.shape[0] + 1, dtype=counts.dtype)
    offsets[1:] = counts.cumsum(0)
    ranks = torch.arange(gdi.shape[0]) - torch.repeat_interleave(offsets[:-1], counts)
    gci = gdi * ((t // p) + 1) + ranks // p
    pk, pv = msa_layer.MemorySparseAttention.sequence_pooling_kv(None, k, v, doc_indices, gci)
    save("pooling_ragged", doc_ids=doc_ids, attention_mask=attention_mask, pooling_kernel_size=p,
         key_states=k, value_states=v, pooled_k=pk, pooled_v=pv)


def sdpa_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p=0.0, causal=True):
    outs = []
    for i in range(cu_seqlens_q.shape[0] - 1):
        qs, qe = int(cu_seqlens_q[i]), int(cu_seqlens_q[i + 1])
        ks, ke = int(cu_seqlens_k[i]), int(cu_seqlens_k[i + 1])
        qi, ki, vi = q[qs:qe].transpose(0, 1), k[ks:ke].transpose(0, 1), v[ks:ke].transpose(0, 1)
        if ki.shape[0] != qi.shape[0]:
            rep = qi.shape[0] // ki.shape[0]
            ki, vi = ki.repeat_interleave(rep, 0), vi.repeat_interleave(rep, 0)
        lq, lk = qe - qs, ke - ks
        m = torch.ones(lq, lk, dtype=torch.bool).tril(diagonal=lk - lq)
        att = (qi @ ki.transpose(-1, -2)) / qi.shape[-1] ** 0.5
        att = att.masked_fill(~m, float("-inf")).softmax(-1)
        outs.append((att @ vi).transpose(0, 1))
    return torch.cat(outs, 0)


class StubCache:
    def __init__(self):
        self.cache_kwargs, self.meta, self.kv, self.rk = {}, {}, {}, {}

    def record_kwargs(self, layer, kw):
        self.cache_kwargs.setdefault(layer, {}).update(kw)

    def update(self, k, v, layer, cache_kwargs=None):
        self.kv[layer] = (k, v)
        return k, v

    def update_router_kcache(self, k, layer):
        self.rk[layer] = k
        return k


def gen_layer(svc, msa_layer, MSAConfig):
    """Stage-1 and decode branches of the reference layer at small model sizes."""
    from transformers.models.qwen3.modeling_qwen3 import Qwen3RotaryEmbedding, apply_rotary_pos_emb
    msa_layer.flash_attn_varlen_func = sdpa_varlen
    torch.manual_seed(202)
    hq, hkv, d = 4, 2, 16
    cfg = MSAConfig(
        msa_config=dict(router_layer_idx="0", aux_loss=False, aux_loss_method="INFONCE", decouple_router=True,
                        top_k_docs=2, pooling_kernel_size=8, head_reduce_method="mean",
                        query_reduce_method="max", chunk_reduce_method="max", decouple_pooling_mode="mean"),
        hidden_size=hq * d, num_attention_heads=hq, num_key_value_heads=hkv, head_dim=d,
        num_hidden_layers=1, intermediate_size=64, vocab_size=32, max_position_embeddings=512)
    cfg._attn_implementation = "eager"
    layer = msa_layer.MemorySparseAttention(cfg, 0).eval()
    with torch.no_grad():
        layer.o_proj.weight.copy_(torch.eye(hq * d))
    rope = Qwen3RotaryEmbedding(cfg)

    # ---- stage 1
    doc_lens = [20, 8, 13]
    ids, pos = [-2, -2, -2], [0, 1, 2]
    for i, n in enumerate(doc_lens):
        ids += [i + 1] * n
        pos += list(range(n))
    doc_ids = torch.tensor([ids])
    position_ids = torch.tensor([pos])
    t = doc_ids.shape[1]
    hidden = torch.randn(1, t, hq * d)
    attention_mask = torch.ones(1, t, dtype=torch.long)
    cos, sin = rope(hidden, position_ids)
    cache = StubCache()
    cache.record_kwargs(0, {"stage": "prefill_stage1"})
    with torch.no_grad():
        layer(hidden, doc_ids, attention_mask, (cos, sin), cache)
        shape = (1, t, -1, d)
        qs = layer.q_norm(layer.q_proj(hidden).view(shape)).transpose(1, 2)
        ks = layer.k_norm(layer.k_proj(hidden).view(shape)).transpose(1, 2)
        vs = layer.v_proj(hidden).view(shape).transpose(1, 2)
        pre_rope_k = ks.clone()
        qs, ks = apply_rotary_pos_emb(qs, ks, cos, sin)
        rks = layer.router_k_proj(hidden).view(shape).transpose(1, 2)
    kw = cache.cache_kwargs[0]
    save("layer_stage1", doc_ids=doc_ids, attention_mask=attention_mask, position_ids=position_ids,
         pooling_kernel_size=8, rope_theta=float(getattr(cfg, "rope_theta", 0.0) or cfg.rope_parameters["rope_theta"]),
         cos=cos, sin=sin, pre_rope_k=pre_rope_k, key_states=ks, value_states=vs, router_k_states=rks,
         pooled_k=cache.kv[0][0], pooled_v=cache.kv[0][1], pooled_rk=cache.rk[0],
         pooled_doc_ids=kw["pooled_doc_ids"], template_k=kw["template_prefix_kcache"],
         template_v=kw["template_prefix_vcache"])

    # ---- decode: two steps over a left-padded compact cache
    b, max_l = 3, 11
    kv_lengths = torch.tensor([11, 7, 4])
    ck = torch.randn(b, hkv, max_l, d)
    cv = torch.randn(b, hkv, max_l, d)
    cache = StubCache()
    cache.record_kwargs(0, {"stage": "generate", "compacked_key_cache": ck.clone(), "compacked_value_cache": cv.clone(),
                            "kv_lengths": kv_lengths.clone(),
                            "attention_mask": torch.arange(max_l).unsqueeze(0) >= (max_l - kv_lengths.unsqueeze(1))})
    steps = {}
    for step in range(2):
        hidden = torch.randn(b, 1, hq * d)
        position_ids = (kv_lengths + step).view(b, 1)
        cos, sin = rope(hidden, position_ids)
        with torch.no_grad():
            out, _ = layer(hidden, torch.full((b, 1), -1), torch.ones(b, 1, dtype=torch.long), (cos, sin), cache)
            shape = (b, 1, -1, d)
            qs = layer.q_norm(layer.q_proj(hidden).view(shape)).transpose(1, 2)
            ks = layer.k_norm(layer.k_proj(hidden).view(shape)).transpose(1, 2)
            vs = layer.v_proj(hidden).view(shape).transpose(1, 2)
            qs, ks = apply_rotary_pos_emb(qs, ks, cos, sin)
        steps[f"q{step}"], steps[f"k{step}"], steps[f"v{step}"], steps[f"out{step}"] = qs, ks, vs, out
    save("layer_decode", cache_k=ck, cache_v=cv, kv_lengths=kv_lengths, **steps)


def gen_layer_decode_qa(svc, msa_layer, MSAConfig):
    """The decode branch of the reference layer in qa_mode (memory_sparse_attention.py:375-380): a multi-token segment
    with masked tokens (left padding and a finished sequence), then a one-token step in which one sequence is masked,
    then another segment.  Every token of a step attends, without a causal mask, to the cache and to the step's own
    unmasked tokens."""
    from transformers.models.qwen3.modeling_qwen3 import Qwen3RotaryEmbedding
    torch.manual_seed(707)
    hq, hkv, d = 4, 2, 16
    cfg = MSAConfig(
        msa_config=dict(router_layer_idx="0", aux_loss=False, aux_loss_method="INFONCE", decouple_router=True,
                        top_k_docs=2, pooling_kernel_size=8, head_reduce_method="mean",
                        query_reduce_method="max", chunk_reduce_method="max", decouple_pooling_mode="mean"),
        hidden_size=hq * d, num_attention_heads=hq, num_key_value_heads=hkv, head_dim=d,
        num_hidden_layers=1, intermediate_size=64, vocab_size=32, max_position_embeddings=512)
    cfg._attn_implementation = "eager"
    layer = msa_layer.MemorySparseAttention(cfg, 0).eval()
    rope = Qwen3RotaryEmbedding(cfg)
    b, max_l = 3, 9
    kv_lengths = torch.tensor([9, 6, 3])
    ck, cv = torch.randn(b, hkv, max_l, d), torch.randn(b, hkv, max_l, d)
    cache = StubCache()
    cache.meta["qa_mode"] = True
    cache.record_kwargs(0, {"stage": "generate", "compacked_key_cache": ck.clone(), "compacked_value_cache": cv.clone(),
                            "kv_lengths": kv_lengths.clone(),
                            "attention_mask": torch.arange(max_l).unsqueeze(0) >= (max_l - kv_lengths.unsqueeze(1))})
    arrays = {"w__" + k: v for k, v in layer.state_dict().items()}
    arrays.update(hq=hq, hkv=hkv, d=d, cache_k=ck, cache_v=cv, kv_lengths=kv_lengths,
                  rope_theta=float(getattr(cfg, "rope_theta", 0.0) or cfg.rope_parameters["rope_theta"]))
    masks = [torch.tensor([[0, 0, 1, 1, 1], [1, 1, 1, 1, 1], [0, 0, 0, 0, 0]]),      # left padding; a finished sequence
             torch.tensor([[1], [0], [1]]),
             torch.tensor([[1, 1, 1], [0, 1, 1], [0, 0, 1]])]
    pos = kv_lengths.clone()
    for step, am in enumerate(masks):
        q_len = am.shape[1]
        hidden = torch.randn(b, q_len, hq * d)
        position_ids = pos.view(b, 1) + (am.cumsum(1) - 1).clamp(min=0)
        with torch.no_grad():
            out, _ = layer(hidden, torch.full((b, q_len), -1), am, rope(hidden, position_ids), cache)
        pos = pos + am.sum(1)
        arrays.update({f"s{step}_hidden": hidden, f"s{step}_attention_mask": am, f"s{step}_position_ids": position_ids,
                       f"s{step}_out": out})
    arrays.update(final_mask=cache.cache_kwargs[0]["attention_mask"], final_cache_k=cache.cache_kwargs[0]["compacked_key_cache"],
                  n_steps=len(masks))
    save("layer_decode_qa", **arrays)


def gen_layer_e2e(svc, msa_layer, MSAConfig):
    """One reference layer through the whole path: stage 1 (encode a block, pool), a reference
    MSAService built from that stage-1 cache (one gloo rank), stage 2 (route, fetch, assemble,
    prefill attention, compact cache) for a left-padded batch, then two decode steps.  The layer's
    weights are stored so that the same module can be rebuilt without the reference."""
    import torch.distributed as dist
    from transformers.models.qwen3.modeling_qwen3 import Qwen3RotaryEmbedding
    msa_layer.flash_attn_varlen_func = sdpa_varlen
    torch.manual_seed(505)
    hq, hkv, d, top_k, pool = 4, 2, 16, 2, 8
    cfg = MSAConfig(
        msa_config=dict(router_layer_idx="0", aux_loss=False, aux_loss_method="INFONCE", decouple_router=True,
                        top_k_docs=top_k, pooling_kernel_size=pool, head_reduce_method="mean",
                        query_reduce_method="max", chunk_reduce_method="max", decouple_pooling_mode="mean"),
        hidden_size=hq * d, num_attention_heads=hq, num_key_value_heads=hkv, head_dim=d,
        num_hidden_layers=1, intermediate_size=64, vocab_size=32, max_position_embeddings=512)
    cfg._attn_implementation = "eager"
    layer = msa_layer.MemorySparseAttention(cfg, 0).eval()
    rope = Qwen3RotaryEmbedding(cfg)
    arrays = {"w__" + k: v for k, v in layer.state_dict().items()}
    arrays.update(hq=hq, hkv=hkv, d=d, top_k=top_k, pooling_kernel_size=pool,
                  rope_theta=float(getattr(cfg, "rope_theta", 0.0) or cfg.rope_parameters["rope_theta"]))

    # ---- stage 1: template head + 5 ragged documents
    doc_lens = [20, 8, 13, 30, 5]
    gids = [40, 41, 42, 43, 44]
    ids, pos = [-2, -2, -2], [0, 1, 2]
    for i, n in enumerate(doc_lens):
        ids += [i + 1] * n
        pos += list(range(n))
    doc_ids, position_ids = torch.tensor([ids]), torch.tensor([pos])
    t = doc_ids.shape[1]
    hidden = torch.randn(1, t, hq * d)
    am = torch.ones(1, t, dtype=torch.long)
    cache1 = StubCache()
    cache1.record_kwargs(0, {"stage": "prefill_stage1"})
    with torch.no_grad():
        out1, _ = layer(hidden, doc_ids, am, rope(hidden, position_ids), cache1)
    kw = cache1.cache_kwargs[0]
    arrays.update(s1_hidden=hidden, s1_doc_ids=doc_ids, s1_attention_mask=am, s1_position_ids=position_ids,
                  s1_out=out1, s1_pooled_k=cache1.kv[0][0], s1_pooled_v=cache1.kv[0][1], s1_pooled_rk=cache1.rk[0],
                  s1_pooled_doc_ids=kw["pooled_doc_ids"], s1_template_k=kw["template_prefix_kcache"],
                  s1_template_v=kw["template_prefix_vcache"], doc_global_ids=gids)

    # ---- the reference service over that bank (single rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29613")
    dist.init_process_group("gloo", rank=0, world_size=1)
    if not torch.cuda.is_available():
        torch.cuda.current_stream = lambda *a, **k: SimpleNamespace(synchronize=lambda: None)
    chunks = [(n + pool - 1) // pool for n in doc_lens]
    service = make_memory(svc, chunks, gids, cache1.rk[0], cache1.kv[0][0], cache1.kv[0][1], top_k=top_k,
                          cls=svc.MSAService)
    service.block_desc.pool_ids = kw["pooled_doc_ids"]
    service._generate_slice(16)
    service.world_size, service.num_key_value_groups, service.scaling = 1, hq // hkv, -1.0
    service.template_prefix_kvcache = {0: (kw["template_prefix_kcache"], kw["template_prefix_vcache"])}
    layer.set_memory_client(service)

    # ---- stage 2: two prompts, left padded; question tokens 0, template tail -2, response head -1
    rows = [[0] * 9 + [-2, -2] + [-1], [0] * 5 + [-2, -2] + [-1]]
    width = max(len(r) for r in rows)
    d2 = torch.tensor([[0] * (width - len(r)) + r for r in rows])
    a2 = torch.tensor([[0] * (width - len(r)) + [1] * len(r) for r in rows])
    p0 = 3 + top_k
    p2 = torch.tensor([[p0] * (width - len(r)) + list(range(p0, p0 + len(r))) for r in rows])
    hidden2 = torch.randn(2, width, hq * d)
    cache2 = StubCache()
    cache2.meta["require_recall_topk"] = True
    cache2.record_kwargs(0, {"stage": "prefill_stage2"})
    with torch.no_grad():
        out2, _ = layer(hidden2, d2, a2, rope(hidden2, p2), cache2)
    kw2 = cache2.cache_kwargs[0]
    arrays.update(s2_hidden=hidden2, s2_doc_ids=d2, s2_attention_mask=a2, s2_position_ids=p2, s2_out=out2,
                  s2_cache_k=kw2["compacked_key_cache"], s2_cache_v=kw2["compacked_value_cache"],
                  s2_kv_lengths=kw2["kv_lengths"], s2_mask=kw2["attention_mask"],
                  s2_recall_ids=[r["topk_doc_ids"] for r in kw2["recall_topk"]],
                  s2_recall_scores=[r["score"] for r in kw2["recall_topk"]])

    # ---- decode: two steps on the cache stage 2 left behind
    cache2.record_kwargs(0, {"stage": "generate"})
    next_pos = p2[:, -1:] + 1
    for step in range(2):
        h = torch.randn(2, 1, hq * d)
        with torch.no_grad():
            o, _ = layer(h, torch.full((2, 1), -1), torch.ones(2, 1, dtype=torch.long), rope(h, next_pos + step), cache2)
        arrays.update({f"dec{step}_hidden": h, f"dec{step}_position_ids": next_pos + step, f"dec{step}_out": o})
    arrays.update(dec_final_cache_k=cache2.cache_kwargs[0]["compacked_key_cache"],
                  dec_final_kv_lengths=cache2.cache_kwargs[0]["kv_lengths"])
    dist.destroy_process_group()
    save("layer_e2e", **arrays)


def _bf16_bits(t):
    """A tensor of bf16-representable fp32 values as its bf16 bit patterns (uint16): half the bytes, no loss."""
    return t.detach().to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def gen_layer_attn128(svc, msa_layer, MSAConfig):
    """The reference layer at the head size the tensor-core attention kernels take (head_dim 128, 8 q / 2 kv heads,
    pooling 64): stage 1 on a block of unmasked documents (one of at least 128 tokens), stage 1 on a block with masked
    tokens INSIDE documents, and stage 2 of a left-padded batch over the first block's bank.  Weights and hidden
    states are rounded to bf16 BEFORE the reference (fp32, CPU) consumes them, so a bf16 implementation sees the
    very same numbers.  The attention outputs are stored as they enter ``o_proj`` (a forward pre-hook)."""
    import torch.distributed as dist
    from transformers.models.qwen3.modeling_qwen3 import Qwen3RotaryEmbedding
    msa_layer.flash_attn_varlen_func = sdpa_varlen
    torch.manual_seed(606)
    hq, hkv, d, top_k, pool, hidden_size = 8, 2, 128, 2, 64, 128
    cfg = MSAConfig(
        msa_config=dict(router_layer_idx="0", aux_loss=False, aux_loss_method="INFONCE", decouple_router=True,
                        top_k_docs=top_k, pooling_kernel_size=pool, head_reduce_method="mean",
                        query_reduce_method="max", chunk_reduce_method="max", decouple_pooling_mode="mean"),
        hidden_size=hidden_size, num_attention_heads=hq, num_key_value_heads=hkv, head_dim=d,
        num_hidden_layers=1, intermediate_size=64, vocab_size=32, max_position_embeddings=1024)
    cfg._attn_implementation = "eager"
    layer = msa_layer.MemorySparseAttention(cfg, 0).eval()
    layer.to(torch.bfloat16).to(torch.float32)             # bf16-representable weights
    rope = Qwen3RotaryEmbedding(cfg)
    pre = {}
    layer.o_proj.register_forward_pre_hook(lambda mod, args: pre.__setitem__("x", args[0].detach().clone()))
    arrays = {"wbits__" + k: _bf16_bits(v) for k, v in layer.state_dict().items()}
    arrays.update(hq=hq, hkv=hkv, d=d, top_k=top_k, pooling_kernel_size=pool, hidden_size=hidden_size,
                  rope_theta=float(getattr(cfg, "rope_theta", 0.0) or cfg.rope_parameters["rope_theta"]))

    def block(doc_lens, drop):
        ids, pos = [-2, -2, -2], [0, 1, 2]
        for i, n in enumerate(doc_lens):
            ids += [i + 1] * n
            pos += list(range(n))
        doc_ids, position_ids = torch.tensor([ids]), torch.tensor([pos])
        t = doc_ids.shape[1]
        hidden = torch.randn(1, t, hidden_size).to(torch.bfloat16).to(torch.float32)
        am = torch.ones(1, t, dtype=torch.long)
        for x in drop:
            am[0, 3 + x] = 0
        cache = StubCache()
        cache.record_kwargs(0, {"stage": "prefill_stage1"})
        with torch.no_grad():
            out, _ = layer(hidden, doc_ids, am, rope(hidden, position_ids), cache)
        return dict(hidden=hidden, doc_ids=doc_ids, am=am, pos=position_ids, out=out, pre=pre["x"], cache=cache)

    # ---- stage 1, block A: unmasked documents (the first and the last are at least 128 tokens long)
    a = block([128, 70, 150], [])
    kw = a["cache"].cache_kwargs[0]
    arrays.update(a_hidden_bits=_bf16_bits(a["hidden"]), a_doc_ids=a["doc_ids"], a_attention_mask=a["am"],
                  a_position_ids=a["pos"], a_attn=a["pre"], a_pooled_k=a["cache"].kv[0][0], a_pooled_v=a["cache"].kv[0][1],
                  a_pooled_rk=a["cache"].rk[0], a_pooled_doc_ids=kw["pooled_doc_ids"])
    # ---- stage 1, block B: masked tokens inside both documents
    b = block([140, 64], [5, 6, 70, 71, 72, 139, 150])
    kwb = b["cache"].cache_kwargs[0]
    arrays.update(b_hidden_bits=_bf16_bits(b["hidden"]), b_doc_ids=b["doc_ids"], b_attention_mask=b["am"],
                  b_position_ids=b["pos"], b_attn=b["pre"], b_pooled_k=b["cache"].kv[0][0], b_pooled_v=b["cache"].kv[0][1],
                  b_pooled_rk=b["cache"].rk[0], b_pooled_doc_ids=kwb["pooled_doc_ids"])

    # ---- the reference service over block A's bank (one gloo rank), then stage 2
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29614")
    dist.init_process_group("gloo", rank=0, world_size=1)
    if not torch.cuda.is_available():
        torch.cuda.current_stream = lambda *a_, **k_: SimpleNamespace(synchronize=lambda: None)
    gids = [70, 71, 72]
    chunks = torch.unique_consecutive(kw["pooled_doc_ids"], return_counts=True)[1].tolist()
    service = make_memory(svc, chunks, gids, a["cache"].rk[0], a["cache"].kv[0][0], a["cache"].kv[0][1], top_k=top_k,
                          cls=svc.MSAService)
    service.block_desc.pool_ids = kw["pooled_doc_ids"]
    service._generate_slice(16)
    service.world_size, service.num_key_value_groups, service.scaling = 1, hq // hkv, -1.0
    service.template_prefix_kvcache = {0: (kw["template_prefix_kcache"], kw["template_prefix_vcache"])}
    layer.set_memory_client(service)
    rows = [[0] * 70 + [-2, -2] + [-1], [0] * 21 + [-2, -2] + [-1]]
    width = max(len(r) for r in rows)
    d2 = torch.tensor([[0] * (width - len(r)) + r for r in rows])
    a2 = torch.tensor([[0] * (width - len(r)) + [1] * len(r) for r in rows])
    p0 = 3 + top_k
    p2 = torch.tensor([[p0] * (width - len(r)) + list(range(p0, p0 + len(r))) for r in rows])
    full = make_memory(svc, chunks, gids, a["cache"].rk[0], a["cache"].kv[0][0], a["cache"].kv[0][1], top_k=3)
    full.block_desc.pool_ids = kw["pooled_doc_ids"]
    full._generate_slice(16)
    qmask = ((d2 == 0) & (a2 == 1)).view(2, 1, 1, width, 1)
    for seed in range(700, 800):
        # the top-2 choice among the three documents must not be a near tie that a bf16 run could flip: draw the
        # prompts until the second and third scores are at least 0.008 apart (bf16 scores are good to ~1e-4 here)
        gen = torch.Generator().manual_seed(seed)
        hidden2 = torch.randn(2, width, hidden_size, generator=gen).to(torch.bfloat16).to(torch.float32)
        with torch.no_grad():
            rq = torch.nn.functional.normalize(layer.router_q_proj(hidden2).view(2, width, hq, d).transpose(1, 2), dim=-1)
            all_scores, _, _ = full.prefill_stage2(0, rq.reshape(2, hkv, hq // hkv, width, d), qmask)
        if float((all_scores[:, 1] - all_scores[:, 2]).min()) > 0.008:
            break
    else:
        raise RuntimeError("no seed gives a clear top-2")
    cache2 = StubCache()
    cache2.meta["require_recall_topk"] = True
    cache2.record_kwargs(0, {"stage": "prefill_stage2"})
    with torch.no_grad():
        out2, _ = layer(hidden2, d2, a2, rope(hidden2, p2), cache2)
    kw2 = cache2.cache_kwargs[0]
    arrays.update(doc_global_ids=gids, s2_hidden_bits=_bf16_bits(hidden2), s2_doc_ids=d2, s2_attention_mask=a2,
                  s2_position_ids=p2, s2_attn=pre["x"], s2_cache_k=kw2["compacked_key_cache"],
                  s2_cache_v=kw2["compacked_value_cache"], s2_kv_lengths=kw2["kv_lengths"], s2_mask=kw2["attention_mask"],
                  s2_recall_ids=[r["topk_doc_ids"] for r in kw2["recall_topk"]],
                  s2_recall_scores=[r["score"] for r in kw2["recall_topk"]], s2_all_doc_scores=all_scores, s2_seed=seed)
    dist.destroy_process_group()
    save("layer_attn128", **arrays)


def gen_routing(svc):
    g = torch.Generator().manual_seed(303)
    chunks = [4, 1, 3, 8, 2, 8, 8, 5, 1, 7]          # ragged documents, 47 chunks, cut into 2 slices
    gids = [900 + 7 * i for i in range(len(chunks))]
    c = sum(chunks)
    hkv, grp, d = 8, 4, 128
    rk = torch.randn(1, hkv, c, d, generator=g)
    q = torch.randn(3, hkv, grp, 6, d, generator=g)
    mask = torch.ones(3, 1, 1, 6, 1, dtype=torch.bool)
    mask[1, 0, 0, 4:, 0] = False        # right padding
    mask[2] = False                     # a sample with no routing token at all
    arrays = dict(rk=rk[0], q=q, mask=mask.view(3, 6), chunks_per_doc=chunks, global_ids=gids, top_k=4)
    for name, reduce, cosine in [
        ("mean_max_max", ("mean", "max", "max"), False),
        ("cosine", ("mean", "max", "max"), True),
        ("max_max_max", ("max", "max", "max"), False),
        ("mean_mean_max", ("mean", "mean", "max"), False),
        ("mean_last_max", ("mean", "last", "max"), False),
        ("mean_max_mean", ("mean", "max", "mean"), False),
    ]:
        # the cosine case L2-normalises both sides first, as the layer does when
        # aux_loss_method == "INFONCE" (memory_sparse_attention.py:192-194, 264-265)
        qq = torch.nn.functional.normalize(q, dim=-1) if cosine else q
        rr = torch.nn.functional.normalize(rk, dim=-1) if cosine else rk
        m = make_memory(svc, chunks, gids, rr, rr, rr, top_k=4, reduce=reduce)
        s, li, gi = m.prefill_stage2(0, qq, mask)
        assert len(m.slice_desc) == 2      # tail under 1024 chunks is merged (msa_service.py:665-670)
        arrays.update({name + "__scores": s, name + "__local_ids": li, name + "__global_ids": gi})
    # fewer documents than k: k' = min(k, N + 1), the dummy document shows up among the winners
    m = make_memory(svc, chunks[:2], gids[:2], rk[:, :, :5], rk[:, :, :5], rk[:, :, :5], top_k=4)
    s, li, gi = m.prefill_stage2(0, q, mask)
    arrays.update({"k_gt_docs__scores": s, "k_gt_docs__local_ids": li, "k_gt_docs__global_ids": gi})
    save("route_cases", **arrays)


def _rank_main(rank, world, ref_path, payload, ret):
    import torch.distributed as dist
    svc, _, _ = import_reference(ref_path)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29611")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    if not torch.cuda.is_available():
        torch.cuda.current_stream = lambda *a, **k: SimpleNamespace(synchronize=lambda: None)
    p = payload[rank]
    s = make_memory(svc, p["chunks"], p["gids"], p["rk"], p["k"], p["v"], top_k=payload["top_k"], cls=svc.MSAService,
                    slice_chunks=16)
    s.gpu_id = rank
    s.world_size = world
    s.num_key_value_groups = payload["groups"]
    s.scaling = -1.0
    out = s.doc_query(p["q"], p["mask"], 0)
    ret[rank] = [o.clone() for o in out]
    dist.barrier()
    dist.destroy_process_group()


def gen_front_end(ref_path):
    """Engine request preparation (``MSAEngine._prepare_template`` / ``_apply_template`` / ``_apply_template_regenerate``
    / ``generate``, src/msa_service.py:1703-1906) and the Memory-Interleave loop (``MSAGenerationMixin._sample``,
    src/msa/generate.py:23-354), both run from the reference's own code with a character tokenizer and a scripted
    model (tests/fake_text.py).  Stored as JSON: what each GPU would be sent, and every forward call the loop made."""
    import json
    import queue
    import threading
    sys.path.insert(0, os.path.join(HERE, "..", ".."))
    from tests import fake_text as F
    import src.msa_service as svc
    from src.msa.generate import MSAGenerationMixin
    from src.utils.tools import RequestLimiter

    tok = F.CharTokenizer()
    out = {"requests": [], "interleave": []}

    # ---- engine: template + request preparation (no processes: the worker queues are plain queues)
    def make_engine(world, top_k):
        e = object.__new__(svc.MSAEngine)
        e.generate_config = SimpleNamespace(world=world, devices=list(range(world)), template=F.TEMPLATE, max_batch_size=0,
                                            max_seq_len=0, max_query_seq_len=0)
        e.model_config = SimpleNamespace(doc_top_k=top_k)
        e.tokenizer = tok
        e.worker_qs = {g: queue.Queue() for g in range(world)}
        e.limiter = RequestLimiter(4)
        e.requests, e.msg_id = {}, 0
        e.lock = threading.Lock()
        e._prepare_template()
        return e

    regen = ("<regenerate>" + F.QUESTION_HEAD + "what is it" + "\nPlease return all documents related to the question\n"
             "<|im_start|>[3]<|object_ref_end|>[3]. gamma doc\n<|object_ref_end|>[1]<|object_ref_end|>[1]. alpha doc\n<|object_ref_end|>")
    for world, top_k, prompts in [(2, 16, ["short", "a longer prompt here", "mid one"]),
                                  (1, 4, ["only one"]),
                                  (4, 16, ["p%d " % i * (i + 1) for i in range(6)]),
                                  (2, 16, ["plain question", regen])]:
        e = make_engine(world, top_k)
        e.generate(list(prompts), userdata="u", require_recall_topk=True, callback=lambda *a: None)
        reqs = [e.worker_qs[g].get_nowait() for g in range(world)]
        stub = e.requests[e.msg_id]
        out["requests"].append({
            "world": world, "top_k": top_k, "prompts": prompts, "nr_dummy": stub.nr_dummy,
            "tail_input_ids": e.prompt_tail_input_ids, "tail_doc_ids": e.tail_doc_ids,
            "per_gpu": [{"msg_id": r.msg_id, "seq_id": r.seq_id, "prompts": r.prompts, "input_ids": r.input_ids,
                         "attention_mask": r.attention_mask, "doc_ids": r.doc_ids, "positions": r.positions,
                         "require_recall_topk": r.require_recall_topk} for r in reqs]})

    # ---- GenerateStub.respond: merge of the per-GPU responses
    got = {}
    stub = svc.GenerateStub(msg_id=7, userdata="ud", nr_dummy=1, responses=[], callback=lambda t, r, u: got.update(t=t, r=r, u=u))
    stub.responses.append(svc.GenerateResponse(msg_id=7, seq_id=1, gpu_id=1, generated_texts=["c", "d"], recall_topk={18: [{"x": 3}]}))
    stub.responses.append(svc.GenerateResponse(msg_id=7, seq_id=0, gpu_id=0, generated_texts=["a", "b"], recall_topk={18: [{"x": 1}], 19: [{"x": 2}]}))
    stub.respond()
    out["respond"] = {"texts": got["t"], "recall": {str(k): v for k, v in got["r"].items()}, "userdata": got["u"]}

    # ---- the interleave loop, driven directly (``_sample`` with the helpers of GenerationMixin it calls replaced by
    # the few lines they amount to for a decoder-only model with a custom cache)
    class Scripted(MSAGenerationMixin):
        def __init__(self, lm):
            self.lm, self.config = lm, lm.config

        def _has_unfinished_sequences(self, this_peer_finished, synced_gpus, device=None):
            return not bool(this_peer_finished)

        def _get_initial_cache_position(self, input_ids, model_kwargs):
            model_kwargs["cache_position"] = torch.arange(input_ids.shape[1])
            return model_kwargs

        def _update_model_kwargs_for_generation(self, outputs, model_kwargs, is_encoder_decoder=False):
            model_kwargs["past_key_values"] = outputs.past_key_values
            am = model_kwargs["attention_mask"]
            model_kwargs["attention_mask"] = torch.cat([am, am.new_ones((am.shape[0], 1))], dim=-1)
            model_kwargs["cache_position"] = model_kwargs["cache_position"][-1:] + 1
            return model_kwargs

        def __call__(self, **kw):
            kw.pop("return_dict", None)
            return self.lm.forward(**kw)

    for name, prompts, scripts in F.INTERLEAVE_CASES:
        e = make_engine(1, 16)
        e.generate(list(prompts), callback=lambda *a: None)
        req = e.worker_qs[0].get_nowait()
        lm = F.ScriptedLM(scripts, tok)
        cache = F.StubCache()
        cache.meta.update({"require_recall_topk": False, "qa_mode": True, "max_generate_tokens": 64, "tokenizer": tok,
                           "idx_to_doc": F.IDX_TO_DOC, "pattern": r"\[(\d+)\]", "response_string": ["" for _ in prompts]})
        for layer in range(lm.config.num_hidden_layers):
            cache.record_kwargs(layer, {"stage": "prefill_stage2"})
        gen_cfg = SimpleNamespace(_pad_token_tensor=torch.tensor(tok.pad_token_id), output_attentions=False,
                                  output_hidden_states=False, output_scores=False, output_logits=False,
                                  return_dict_in_generate=False, do_sample=False, prefill_chunk_size=None)
        eos = torch.tensor([tok.eos_token_id])

        class Eos:
            eos_token_id = eos

            def __call__(self, ids, scores):
                return torch.isin(ids[:, -1], eos)

        class Criteria(list):
            def __call__(self, ids, scores):
                return self[0](ids, scores)

        seqs = Scripted(lm)._sample(
            torch.LongTensor(req.input_ids), logits_processor=lambda ids, logits: logits, stopping_criteria=Criteria([Eos()]),
            generation_config=gen_cfg, synced_gpus=False, streamer=None,
            attention_mask=torch.LongTensor(req.attention_mask), doc_ids=torch.LongTensor(req.doc_ids), use_cache=True,
            position_ids=torch.LongTensor(req.positions), past_key_values=cache)
        out["interleave"].append({
            "name": name, "prompts": prompts, "scripts": scripts, "sequences": seqs.tolist(),
            "response_string": cache.meta["response_string"],
            "calls": [{k: (v.tolist() if torch.is_tensor(v) else v) for k, v in c.items()} for c in lm.calls]})
        print("interleave", name, "calls", len(lm.calls), "sequence length", seqs.shape[1], cache.meta["response_string"])
    with open(os.path.join(HERE, "front_end.json"), "w") as f:
        json.dump(out, f)
    print("wrote front_end.json")


def gen_doc_query(ref_path):
    import torch.multiprocessing as mp
    g = torch.Generator().manual_seed(404)
    world, hkv, grp, d, top_k = 2, 8, 4, 128, 3
    chunk_lists = [[3, 1, 4, 2, 5, 2], [2, 6, 1, 3, 3]]
    payload = {"top_k": top_k, "groups": grp}
    gid = 10
    for r in range(world):
        c = sum(chunk_lists[r])
        gids = list(range(gid, gid + len(chunk_lists[r])))
        gid += len(chunk_lists[r])
        # ranks with different query lengths.  Both are >= the group count (4): doc_query trims
        # the gathered queries with [:, :, :seqlen, :] (msa_service.py:1155), which indexes the
        # GROUP axis of [B, Hkv, G, S, D], so a query shorter than G silently loses groups there.
        s_len = 5 if r == 0 else 4
        q = torch.nn.functional.normalize(torch.randn(2, hkv * grp, s_len, d, generator=g), dim=-1)
        mask = torch.ones(2, s_len, dtype=torch.bool)
        if r == 0:
            mask[1, 3:] = False
        payload[r] = dict(chunks=chunk_lists[r], gids=gids,
                          rk=torch.nn.functional.normalize(torch.randn(1, hkv, c, d, generator=g), dim=-1),
                          k=torch.randn(1, hkv, c, d, generator=g), v=torch.randn(1, hkv, c, d, generator=g),
                          q=q, mask=mask)
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_rank_main, args=(world, ref_path, payload, ret), nprocs=world, join=True)
    arrays = dict(world=world, top_k=top_k, groups=grp)
    for r in range(world):
        p = payload[r]
        fk, fv, fs, nsel, wg = ret[r]
        arrays.update({f"r{r}_chunks": p["chunks"], f"r{r}_gids": p["gids"], f"r{r}_rk": p["rk"][0],
                       f"r{r}_k": p["k"][0], f"r{r}_v": p["v"][0], f"r{r}_q": p["q"], f"r{r}_mask": p["mask"],
                       f"r{r}_final_k": fk, f"r{r}_final_v": fv, f"r{r}_final_scores": fs,
                       f"r{r}_num_selected": nsel, f"r{r}_winner_global_ids": wg})
    save("doc_query_w2", **arrays)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--only", default="", help="run one generator only, e.g. front_end")
    a = ap.parse_args()
    svc, msa_layer, MSAConfig = import_reference(a.reference)
    if a.only == "front_end":
        gen_front_end(a.reference)
        sys.exit(0)
    gen_pooling(svc, msa_layer)
    gen_layer(svc, msa_layer, MSAConfig)
    gen_routing(svc)
    gen_layer_e2e(svc, msa_layer, MSAConfig)
    gen_layer_attn128(svc, msa_layer, MSAConfig)
    gen_layer_decode_qa(svc, msa_layer, MSAConfig)
    gen_front_end(a.reference)
    gen_doc_query(a.reference)

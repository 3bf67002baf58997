"""The attention-layer mirror against the REFERENCE layer run end to end (tests/golden/layer_e2e.npz:
stage 1 -> bank -> stage 2 -> two decode steps, produced by the reference's own modules with the
weights stored alongside)."""
import numpy as np
import pytest
import torch

from tests.util import T, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def e2e(golden):
    from transformers.models.qwen3.modeling_qwen3 import Qwen3RotaryEmbedding
    from msa_b200.attention import MemorySparseAttention
    from msa_b200.configuration import MSAConfig
    g = golden("layer_e2e")
    hq, hkv, d = int(g["hq"]), int(g["hkv"]), int(g["d"])
    cfg = MSAConfig(
        msa_config=dict(router_layer_idx="0", aux_loss=False, aux_loss_method="INFONCE", decouple_router=True,
                        top_k_docs=int(g["top_k"]), pooling_kernel_size=int(g["pooling_kernel_size"]),
                        head_reduce_method="mean", query_reduce_method="max", chunk_reduce_method="max",
                        decouple_pooling_mode="mean"),
        hidden_size=hq * d, num_attention_heads=hq, num_key_value_heads=hkv, head_dim=d, num_hidden_layers=1,
        intermediate_size=64, vocab_size=32, max_position_embeddings=512)
    cfg._attn_implementation = "eager"
    layer = MemorySparseAttention(cfg, 0).eval()
    layer.load_state_dict({k[3:]: T(v) for k, v in g.items() if k.startswith("w__")})
    layer.to(DEV)
    rope = Qwen3RotaryEmbedding(cfg).to(DEV)
    return g, cfg, layer, rope


def test_layer_stage1_stage2_decode_match_reference(e2e):
    from msa_b200.cache import SparseCache, SparseCacheOnCPU
    from msa_b200.memory import AttentionGeometry, Document, ModelConfig
    from msa_b200.service import MSAService
    g, cfg, layer, rope = e2e
    hq, hkv, d, top_k, pool = int(g["hq"]), int(g["hkv"]), int(g["d"]), int(g["top_k"]), int(g["pooling_kernel_size"])

    # ---------------- stage 1
    cache1 = SparseCacheOnCPU()
    cache1.record_kwargs(0, {"stage": "prefill_stage1"})
    hidden = T(g["s1_hidden"]).to(DEV)
    with torch.no_grad():
        out1, _ = layer(hidden, T(g["s1_doc_ids"]).to(DEV), T(g["s1_attention_mask"]).to(DEV),
                        rope(hidden, T(g["s1_position_ids"]).to(DEV)), cache1)
    kw = cache1.cache_kwargs[0]
    assert rel_err(out1, T(g["s1_out"])) < 1e-5
    pk, pv = cache1.get_kvcache(0)
    assert rel_err(pk, T(g["s1_pooled_k"])) < 1e-5 and rel_err(pv, T(g["s1_pooled_v"])) < 1e-5
    assert rel_err(cache1.get_router_kcache(0), T(g["s1_pooled_rk"])) < 1e-5
    assert torch.equal(kw["pooled_doc_ids"], T(g["s1_pooled_doc_ids"]))
    assert rel_err(kw["template_prefix_kcache"], T(g["s1_template_k"])) < 1e-6
    assert kw["prefill_stage1_kvcache_size"] == T(g["s1_pooled_k"]).shape[2] and kw["doc_id_bias"] == hidden.shape[1]

    # ---------------- the service, fed with the stage-1 worker's META payload
    chunks = torch.unique_consecutive(kw["pooled_doc_ids"], return_counts=True)[1].tolist()
    docs = [Document(doc_id=int(i), num_chunks=n) for i, n in zip(g["doc_global_ids"], chunks)]
    geo = AttentionGeometry(num_hidden_layers=1, num_attention_heads=hq, num_key_value_heads=hkv, head_dim=d,
                            dtype=torch.float32)
    svc = MSAService(0, None, ModelConfig(doc_top_k=top_k, pooling_kernel_size=pool, router_layer_idx="0"), None, geo,
                     world_size=1, rank=0)
    svc.generate_blocks(docs, metas=[{"past_key_values": cache1, "nr_docs": len(docs), "chunk_sizes": chunks,
                                      "doc_ids": [dd.doc_id for dd in docs], "nr_chunks": chunks}])
    assert torch.equal(svc.block_desc.pool_ids.cpu(), T(g["s1_pooled_doc_ids"]))
    svc.setup_memory_client(layer)
    assert layer.memory_client is svc

    # ---------------- stage 2
    cache2 = SparseCache()
    cache2.meta["require_recall_topk"] = True
    cache2.meta["max_generate_tokens"] = 8
    cache2.record_kwargs(0, {"stage": "prefill_stage2"})
    hidden2 = T(g["s2_hidden"]).to(DEV)
    with torch.no_grad():
        out2, _ = layer(hidden2, T(g["s2_doc_ids"]).to(DEV), T(g["s2_attention_mask"]).to(DEV),
                        rope(hidden2, T(g["s2_position_ids"]).to(DEV)), cache2)
    svc.check_status()
    kw2 = cache2.cache_kwargs[0]
    am = T(g["s2_attention_mask"]).bool()
    assert rel_err(out2.cpu()[am], T(g["s2_out"])[am]) < 1e-5      # padded positions are unspecified
    assert torch.equal(kw2["kv_lengths"].cpu(), T(g["s2_kv_lengths"]))
    assert torch.equal(kw2["attention_mask"].cpu(), T(g["s2_mask"]))
    assert rel_err(kw2["compacked_key_cache"], T(g["s2_cache_k"])) < 1e-5
    assert rel_err(kw2["compacked_value_cache"], T(g["s2_cache_v"])) < 1e-5
    assert [r["topk_doc_ids"] for r in kw2["recall_topk"]] == g["s2_recall_ids"].tolist()
    assert np.allclose([r["score"] for r in kw2["recall_topk"]], g["s2_recall_scores"], atol=1e-4)

    # ---------------- decode, two steps, appended in place
    cache2.record_kwargs(0, {"stage": "generate"})
    store_ptr = kw2["_msa_b200_store"][0].data_ptr()
    for step in range(2):
        h = T(g[f"dec{step}_hidden"]).to(DEV)
        with torch.no_grad():
            o, _ = layer(h, torch.full((2, 1), -1, device=DEV), torch.ones(2, 1, dtype=torch.long, device=DEV),
                         rope(h, T(g[f"dec{step}_position_ids"]).to(DEV)), cache2)
        assert rel_err(o, T(g[f"dec{step}_out"])) < 1e-5
    kw2 = cache2.cache_kwargs[0]
    assert kw2["_msa_b200_store"][0].data_ptr() == store_ptr          # no reallocation, no torch.cat
    assert torch.equal(kw2["kv_lengths"].cpu(), T(g["dec_final_kv_lengths"]))
    assert rel_err(kw2["compacked_key_cache"], T(g["dec_final_cache_k"])) < 1e-5


def test_training_forward_is_rejected(e2e):
    g, cfg, layer, rope = e2e
    layer.train()
    try:
        with pytest.raises(NotImplementedError):
            layer(torch.zeros(1, 2, 64, device=DEV), torch.zeros(1, 2, dtype=torch.long, device=DEV))
    finally:
        layer.eval()


def test_qa_mode_decode_segments_match_reference_layer(golden):
    """The layer mirror's decode branch in qa_mode (multi-token, non-causal segments with masked tokens; reference:
    src/msa/memory_sparse_attention.py:375-380) against the reference layer's own outputs.  fp32, head_dim 16: the
    segment append kernel and the general attention kernel.  Rows of masked tokens are unspecified in the reference
    (it computes them and nobody reads them) and zero here."""
    from transformers.models.qwen3.modeling_qwen3 import Qwen3RotaryEmbedding
    from msa_b200.attention import MemorySparseAttention
    from msa_b200.cache import SparseCache
    from msa_b200.configuration import MSAConfig
    g = golden("layer_decode_qa")
    hq, hkv, d = int(g["hq"]), int(g["hkv"]), int(g["d"])
    cfg = MSAConfig(
        msa_config=dict(router_layer_idx="0", aux_loss=False, aux_loss_method="INFONCE", decouple_router=True,
                        top_k_docs=2, pooling_kernel_size=8, head_reduce_method="mean", query_reduce_method="max",
                        chunk_reduce_method="max", decouple_pooling_mode="mean"),
        hidden_size=hq * d, num_attention_heads=hq, num_key_value_heads=hkv, head_dim=d, num_hidden_layers=1,
        intermediate_size=64, vocab_size=32, max_position_embeddings=512)
    cfg._attn_implementation = "eager"
    layer = MemorySparseAttention(cfg, 0).eval()
    layer.load_state_dict({k[3:]: T(v) for k, v in g.items() if k.startswith("w__")})
    layer.to(DEV)
    rope = Qwen3RotaryEmbedding(cfg).to(DEV)
    ck, cv, lens = T(g["cache_k"]).to(DEV), T(g["cache_v"]).to(DEV), T(g["kv_lengths"]).to(DEV)
    max_l = ck.shape[2]
    cache = SparseCache()
    cache.meta["qa_mode"] = True
    cache.record_kwargs(0, {"stage": "generate", "compacked_key_cache": ck.clone(), "compacked_value_cache": cv.clone(),
                            "kv_lengths": lens.clone(),
                            "attention_mask": torch.arange(max_l, device=DEV).unsqueeze(0) >= (max_l - lens.unsqueeze(1))})
    valid_total = lens.clone()
    for step in range(int(g["n_steps"])):
        hidden, am = T(g[f"s{step}_hidden"]).to(DEV), T(g[f"s{step}_attention_mask"]).to(DEV)
        b, q_len = am.shape
        with torch.no_grad():
            out, _ = layer(hidden, torch.full((b, q_len), -1, device=DEV), am,
                           rope(hidden, T(g[f"s{step}_position_ids"]).to(DEV)), cache)
        valid = (am == 1).cpu()
        assert rel_err(out.cpu()[valid], T(g[f"s{step}_out"])[valid]) < 1e-5
        valid_total = valid_total + am.sum(1)
        kw = cache.cache_kwargs[0]
        # the store keeps only unmasked entries, one contiguous run per sequence
        assert torch.equal(kw["attention_mask"].sum(1), valid_total)
        assert torch.equal(kw["kv_lengths"], valid_total)
    # same entries as the reference's cache, in the same order, once its masked slots are dropped
    kw = cache.cache_kwargs[0]
    ref_k, ref_m = T(g["final_cache_k"]), T(g["final_mask"]).bool()
    got_k, got_m = kw["compacked_key_cache"].cpu(), kw["attention_mask"].cpu()
    for i in range(ref_k.shape[0]):
        assert rel_err(got_k[i][:, got_m[i]], ref_k[i][:, ref_m[i]]) < 1e-6

"""The oracle restatement against outputs of the reference's own code (tests/golden/*.npz,
produced by tests/golden/make_golden.py).  CPU only."""
import numpy as np
import pytest
import torch

from oracle import msa_oracle as O


def T(x):
    return torch.from_numpy(np.asarray(x))


def test_bookkeeping_and_pooling_match_reference(golden):
    g = golden("pooling_ragged")
    p = int(g["pooling_kernel_size"])
    doc_indices, gci, pooled_doc_ids, lengths = O.chunk_bookkeeping(T(g["doc_ids"]), T(g["attention_mask"]), p)
    assert lengths.tolist() == [16, 16, 16, 2, 16, 16, 16, 1, 1, 16, 16, 16, 16]
    assert pooled_doc_ids.tolist() == [1, 1, 1, 1, 2, 3, 3, 3, 4, 5, 5, 5, 5]
    pk, pv = O.sequence_pooling_kv(T(g["key_states"]), T(g["value_states"]), doc_indices, gci)
    # same formula, same fp32 op order: bit-exact
    assert torch.equal(pk, T(g["pooled_k"])) and torch.equal(pv, T(g["pooled_v"]))
    # and the cumsum-difference agrees with the exact mean norm-wise to fp32 accuracy
    k_docs = T(g["key_states"])[doc_indices[:, 0], :, doc_indices[:, 1]]
    exact = O.pool_chunks_exact(k_docs, lengths)
    rel = (pk.double() - exact).norm() / exact.norm()
    assert rel < 1e-6


def test_stage1_layer_outputs(golden):
    g = golden("layer_stage1")
    p = int(g["pooling_kernel_size"])
    doc_ids, am = T(g["doc_ids"]), T(g["attention_mask"])
    doc_indices, gci, pooled_doc_ids, lengths = O.chunk_bookkeeping(doc_ids, am, p)
    assert torch.equal(pooled_doc_ids, T(g["pooled_doc_ids"]))
    assert lengths.tolist() == [8, 8, 4, 8, 8, 5]
    # RoPE restatement against the keys the reference produced (positions restart per doc)
    cos, sin = O.rope_cos_sin(T(g["position_ids"]), 16, float(g["rope_theta"]))
    assert torch.allclose(cos, T(g["cos"]), atol=1e-6) and torch.allclose(sin, T(g["sin"]), atol=1e-6)
    k_rot = O.rope_rotate_half(T(g["pre_rope_k"]), cos.unsqueeze(1), sin.unsqueeze(1))
    assert torch.allclose(k_rot, T(g["key_states"]), atol=1e-6)
    pk, pv = O.sequence_pooling_kv(T(g["key_states"]), T(g["value_states"]), doc_indices, gci)
    assert torch.equal(pk.transpose(0, 1).unsqueeze(0), T(g["pooled_k"]))
    assert torch.equal(pv.transpose(0, 1).unsqueeze(0), T(g["pooled_v"]))
    rk_docs = T(g["router_k_states"])[doc_indices[:, 0], :, doc_indices[:, 1]]
    prk = O.l2_normalize(O.pool_chunks_cumsum(rk_docs, lengths).transpose(0, 1).unsqueeze(0))
    assert torch.equal(prk, T(g["pooled_rk"]))
    n_t = int((doc_ids == -2).sum())
    assert torch.equal(T(g["key_states"])[:, :, :n_t], T(g["template_k"]))


CASES = {
    "mean_max_max": ("mean", "max", "max"),
    "cosine": ("mean", "max", "max"),
    "max_max_max": ("max", "max", "max"),
    "mean_mean_max": ("mean", "mean", "max"),
    "mean_last_max": ("mean", "last", "max"),
    "mean_max_mean": ("mean", "max", "mean"),
}


@pytest.mark.parametrize("name", list(CASES))
def test_routing_matches_reference(golden, name):
    g = golden("route_cases")
    q, rk = T(g["q"]), T(g["rk"])
    if name == "cosine":
        q, rk = O.l2_normalize(q), O.l2_normalize(rk)
    chunks = g["chunks_per_doc"].tolist()
    pool_ids = torch.repeat_interleave(torch.arange(1, len(chunks) + 1), torch.tensor(chunks))
    table = torch.tensor([0] + g["global_ids"].tolist())
    h, qr, cr = CASES[name]
    s, li, gi = O.prefill_stage2(q, T(g["mask"]), rk, pool_ids, table, int(g["top_k"]),
                                 head_reduce=h, query_reduce=qr, chunk_reduce=cr, slice_chunks=7)
    ref_s = T(g[name + "__scores"])
    valid = ref_s > -1e9
    assert torch.allclose(s[valid], ref_s[valid], atol=1e-5, rtol=1e-5)
    assert torch.equal(li[valid], T(g[name + "__local_ids"])[valid])
    assert torch.equal(gi[valid], T(g[name + "__global_ids"])[valid])
    # the sample without any routing token scores finfo.min everywhere
    assert (s[2] == torch.finfo(torch.float32).min).all() or name == "mean_mean_max"


def test_routing_k_larger_than_docs(golden):
    g = golden("route_cases")
    pool_ids = torch.tensor([1, 1, 1, 1, 2])
    table = torch.tensor([0] + g["global_ids"].tolist()[:2])
    s, li, gi = O.prefill_stage2(T(g["q"]), T(g["mask"]), T(g["rk"])[:, :5], pool_ids, table, 4)
    assert s.shape == (3, 3)                      # k' = min(k, N + 1)
    ref_s = T(g["k_gt_docs__scores"])
    assert torch.allclose(s[:2], ref_s[:2], atol=1e-5)
    assert torch.equal(li[:2], T(g["k_gt_docs__local_ids"])[:2])
    assert (li[:2, -1] == 0).all()                # the dummy document comes last


def test_doc_query_two_ranks(golden):
    g = golden("doc_query_w2")
    w, top_k, grp = int(g["world"]), int(g["top_k"]), int(g["groups"])
    shards = [O.Shard(T(g[f"r{r}_k"]), T(g[f"r{r}_v"]), T(g[f"r{r}_rk"]),
                      g[f"r{r}_chunks"].tolist(), g[f"r{r}_gids"].tolist()) for r in range(w)]
    qs = [T(g[f"r{r}_q"]) for r in range(w)]
    ms = [T(g[f"r{r}_mask"]) for r in range(w)]
    outs = O.doc_query_world(qs, ms, shards, top_k, grp)
    for r, (fk, fv, fs, nsel, wg) in enumerate(outs):
        assert torch.allclose(fs, T(g[f"r{r}_final_scores"]), atol=1e-5)
        assert torch.equal(wg, T(g[f"r{r}_winner_global_ids"]))
        assert torch.equal(nsel, T(g[f"r{r}_num_selected"]))
        assert torch.equal(fk, T(g[f"r{r}_final_k"]))
        assert torch.equal(fv, T(g[f"r{r}_final_v"]))


def _attn128_states(g, prefix, weights, geo):
    from tests.util import from_bf16_bits
    hidden = from_bf16_bits(g[prefix + "_hidden_bits"])
    cos, sin = O.rope_cos_sin(T(g[prefix + "_position_ids"]), geo["d"], geo["theta"])
    return hidden, O.qwen3_attention_states(hidden, weights, cos, sin, geo["hq"], geo["hkv"], geo["d"])


@pytest.mark.parametrize("block", ["a", "b"])
def test_stage1_attention_restatement_matches_reference_layer(golden, block):
    """oracle.stage1_doc_attention against the attention output the reference layer fed to o_proj, at head_dim 128:
    block a = unmasked documents, block b = masked tokens inside documents; plus the pooled K / V / K_r."""
    from tests.util import attn128_case
    g = golden("layer_attn128")
    weights, geo = attn128_case(g)
    hidden, (q, k, v) = _attn128_states(g, block, weights, geo)
    doc_ids, am = T(g[block + "_doc_ids"]), T(g[block + "_attention_mask"])
    out = O.stage1_doc_attention(q, k, v, doc_ids, am)
    ref = T(g[block + "_attn"])
    assert float((out - ref).norm() / ref.norm()) < 1e-5
    assert float(ref[0][am[0] == 0].abs().sum()) == 0 and float(out[0][am[0] == 0].abs().sum()) == 0
    doc_indices, gci, pooled_doc_ids, lengths = O.chunk_bookkeeping(doc_ids, am, geo["pool"])
    assert torch.equal(pooled_doc_ids, T(g[block + "_pooled_doc_ids"]))
    pk, pv = O.sequence_pooling_kv(k, v, doc_indices, gci)
    assert float((pk.transpose(0, 1).unsqueeze(0) - T(g[block + "_pooled_k"])).abs().max()) < 1e-5
    assert float((pv.transpose(0, 1).unsqueeze(0) - T(g[block + "_pooled_v"])).abs().max()) < 1e-5


def test_stage2_attention_restatement_matches_reference_layer(golden):
    """oracle.stage2_context_attention (context assembly, bottom-right causal attention, left-padded compact cache)
    against the reference layer's stage 2 over block a's bank, the routing included (oracle.doc_query_world)."""
    from tests.util import attn128_case, from_bf16_bits
    g = golden("layer_attn128")
    weights, geo = attn128_case(g)
    _, (qa, ka, va) = _attn128_states(g, "a", weights, geo)
    doc_ids_a, am_a = T(g["a_doc_ids"]), T(g["a_attention_mask"])
    doc_indices, gci, pooled_doc_ids, lengths = O.chunk_bookkeeping(doc_ids_a, am_a, geo["pool"])
    chunks = torch.unique_consecutive(pooled_doc_ids, return_counts=True)[1].tolist()
    shard = O.Shard(T(g["a_pooled_k"])[0], T(g["a_pooled_v"])[0], T(g["a_pooled_rk"])[0], chunks, g["doc_global_ids"].tolist())
    hidden2, (q, k, v) = _attn128_states(g, "s2", weights, geo)
    d2, a2 = T(g["s2_doc_ids"]), T(g["s2_attention_mask"])
    b, s = d2.shape
    rq = torch.nn.functional.linear(hidden2, weights["router_q_proj.0.weight"]).view(b, s, geo["hq"], geo["d"]).transpose(1, 2)
    rq = O.l2_normalize(rq)
    (fk, fv, fs, n_sel, wg), = O.doc_query_world([rq], [(d2 == 0) & (a2 == 1)], [shard], geo["top_k"], geo["hq"] // geo["hkv"])
    assert wg.tolist() == g["s2_recall_ids"].tolist()
    assert torch.allclose(fs, T(g["s2_recall_scores"]).float(), atol=1e-5)
    n_t = int((doc_ids_a == -2).sum())
    out, ck, cv, lens = O.stage2_context_attention(q, k, v, ka[:, :, :n_t], va[:, :, :n_t], fk, fv, a2 == 1, n_sel)
    assert torch.equal(lens, T(g["s2_kv_lengths"]))
    assert float((ck - T(g["s2_cache_k"])).abs().max()) < 1e-5 and float((cv - T(g["s2_cache_v"])).abs().max()) < 1e-5
    ref = T(g["s2_attn"])
    valid = a2 == 1
    assert float((out[valid] - ref[valid]).norm() / ref[valid].norm()) < 1e-5
    assert float(ref[~valid].abs().sum()) == 0


def test_decode_matches_reference_layer(golden):
    g = golden("layer_decode")
    ck, cv, lens = T(g["cache_k"]), T(g["cache_v"]), T(g["kv_lengths"])
    for step in range(2):
        q, k, v = T(g[f"q{step}"]), T(g[f"k{step}"]), T(g[f"v{step}"])
        out = O.decode_attention(q, ck, cv, lens, k, v)
        assert torch.allclose(out, T(g[f"out{step}"]), atol=2e-6, rtol=1e-5)
        ck, cv, lens = torch.cat([ck, k], 2), torch.cat([cv, v], 2), lens + 1


def test_qa_mode_decode_segments_match_reference_layer(golden):
    """oracle.decode_segment_attention against the reference layer's decode branch in qa_mode: two multi-token
    segments and a one-token step, with left padding, a masked step and a finished sequence."""
    g = golden("layer_decode_qa")
    hq, hkv, d = int(g["hq"]), int(g["hkv"]), int(g["d"])
    weights = {k[3:]: T(v) for k, v in g.items() if k.startswith("w__")}
    ck, cv, lens = T(g["cache_k"]), T(g["cache_v"]), T(g["kv_lengths"])
    mask = torch.arange(ck.shape[2]).unsqueeze(0) >= (ck.shape[2] - lens.unsqueeze(1))
    for step in range(int(g["n_steps"])):
        hidden, am = T(g[f"s{step}_hidden"]), T(g[f"s{step}_attention_mask"])
        cos, sin = O.rope_cos_sin(T(g[f"s{step}_position_ids"]), d, float(g["rope_theta"]))
        q, k, v = O.qwen3_attention_states(hidden, weights, cos, sin, hq, hkv, d)
        out, ck, cv, mask = O.decode_segment_attention(q, ck, cv, mask, k, v, am == 1)
        out = torch.nn.functional.linear(out, weights["o_proj.weight"])
        ref = T(g[f"s{step}_out"])
        valid = am == 1
        assert torch.allclose(out[valid], ref[valid], atol=2e-6, rtol=1e-5)
    assert torch.equal(mask, T(g["final_mask"]))
    assert torch.allclose(ck, T(g["final_cache_k"]), atol=1e-6)

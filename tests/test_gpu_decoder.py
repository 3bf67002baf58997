"""The config-5 decode loop (msa_b200.decoder.SparseDecodeModel) against a plain PyTorch fp32
restatement of the same step built on the oracle's decode attention: same random weights, same
synthetic caches, two steps, no routing service (router layers are covered by the service tests)."""

import pytest
import torch
import torch.nn.functional as F

from oracle import msa_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _reference_step(m, tokens, kv_len, positions, k_cache, v_cache):
    s = m.s
    f32 = lambda t: t.float().cpu()
    x = f32(m.embed)[tokens]
    ang = positions.float().unsqueeze(-1) * f32(m.inv_freq)
    emb = torch.cat([ang, ang], -1)
    cos, sin = emb.cos().to(torch.bfloat16).float().unsqueeze(1), emb.sin().to(torch.bfloat16).float().unsqueeze(1)
    nq, nkv, d, B = s.n_q_heads, s.n_kv_heads, s.head_dim, tokens.shape[0]
    for l, p in enumerate(m.layers):
        h = F.rms_norm(x, (s.hidden,), f32(p["w_in"]), s.rms_eps)
        qkv = h @ f32(p["w_qkv"])
        q = F.rms_norm(qkv[:, : nq * d].view(B, nq, d), (d,), f32(p["q_norm"]), s.rms_eps)
        k = F.rms_norm(qkv[:, nq * d:(nq + nkv) * d].view(B, nkv, d), (d,), f32(p["k_norm"]), s.rms_eps)
        v = qkv[:, (nq + nkv) * d:(nq + 2 * nkv) * d].view(B, nkv, d)
        q, k = O.rope_rotate_half(q, cos, sin), O.rope_rotate_half(k, cos, sin)
        L = int(kv_len[0])
        # the oracle wants a left-padded cache of exactly the valid length
        att = O.decode_attention(q.unsqueeze(2), k_cache[l][:, :, :L], v_cache[l][:, :, :L], kv_len.long(),
                                 k.unsqueeze(2), v.unsqueeze(2))[:, 0]
        k_cache[l] = torch.cat([k_cache[l][:, :, :L], k.unsqueeze(2)], 2)
        v_cache[l] = torch.cat([v_cache[l][:, :, :L], v.unsqueeze(2)], 2)
        x = x + att @ f32(p["w_o"])
        h = F.rms_norm(x, (s.hidden,), f32(p["w_post"]), s.rms_eps)
        gu = h @ f32(p["w_gate_up"])
        x = x + (F.silu(gu[:, : s.ffn]) * gu[:, s.ffn:]) @ f32(p["w_down"])
    x = F.rms_norm(x, (s.hidden,), f32(m.w_final), s.rms_eps)
    return x @ f32(m.lm_head)


def test_decode_step_matches_fp32_restatement():
    from msa_b200.decoder import DecoderShape, SparseDecodeModel
    shape = DecoderShape(num_layers=3, hidden=256, n_q_heads=8, n_kv_heads=2, head_dim=128, ffn=512, vocab=1000)
    m = SparseDecodeModel(shape, None, [], batch=3, local_ctx=70, max_new=8, retrieved_entries=16, device=DEV, seed=5)
    k_ref = [c.float().cpu() for c in m.k_cache]
    v_ref = [c.float().cpu() for c in m.v_cache]
    tokens, kv_len, positions = m.tokens.cpu(), m.kv_len.cpu(), m.positions.cpu()
    for step in range(2):
        # capture the model's own logits by re-running its last matmul is not possible from outside:
        # compare the argmax it feeds back and, through a hook on lm_head, the logits themselves
        logits_ref = _reference_step(m, tokens, kv_len, positions, k_ref, v_ref)
        nxt = m.step().cpu()
        top2 = logits_ref.topk(2, dim=-1).values
        clear = (top2[:, 0] - top2[:, 1]) > 0.05 * logits_ref.abs().max()      # bf16 weights: skip near-ties
        assert torch.equal(nxt[clear], logits_ref.argmax(-1)[clear])
        # the step's K/V landed in place at the old length
        L = int(kv_len[0])
        for l in range(shape.num_layers):
            got = m.k_cache[l][:, :, L].float().cpu()
            assert float((got - k_ref[l][:, :, L]).norm() / k_ref[l][:, :, L].norm()) < 2e-2
        tokens, kv_len, positions = nxt, kv_len + 1, positions + 1
        assert torch.equal(m.kv_len.cpu(), kv_len)


def _routed_model(seed):
    from msa_b200.decoder import DecoderShape, SparseDecodeModel
    from msa_b200.memory import AttentionGeometry, Document, ModelConfig
    from msa_b200.service import MSAService
    from tests.util import make_bank
    n_docs, cpd, top_k, hkv, d = 40, 4, 4, 8, 128
    geo = AttentionGeometry(num_hidden_layers=4, num_attention_heads=32, num_key_value_heads=hkv, head_dim=d,
                            dtype=torch.bfloat16)
    svc = MSAService(0, None, ModelConfig(doc_top_k=top_k, router_layer_idx="2,3"), None, geo, world_size=1, rank=0)
    svc.uniform_seqlen = True
    docs = [Document(doc_id=i, num_chunks=cpd) for i in range(n_docs)]
    layers = {}
    for l in (2, 3):
        rk, _ = make_bank([cpd] * n_docs, hkv, d, torch.bfloat16, seed=l)
        g = torch.Generator().manual_seed(100 + l)
        k = torch.randn(n_docs * cpd, hkv, d, generator=g).to(torch.bfloat16)
        v = torch.randn(n_docs * cpd, hkv, d, generator=g).to(torch.bfloat16)
        layers[l] = (k.to(DEV), v.to(DEV), rk.to(DEV))
    svc.load_pooled(docs, layers)
    shape = DecoderShape(num_layers=4, hidden=256, n_q_heads=32, n_kv_heads=hkv, head_dim=d, ffn=512, vocab=1000)
    return SparseDecodeModel(shape, svc, [2, 3], batch=3, local_ctx=40, max_new=12, retrieved_entries=top_k * cpd,
                             device=DEV, seed=seed)


@pytest.mark.parametrize("beside", ["dense", "routing"])
def test_pipelined_loop_produces_the_same_tokens_and_caches(beside, monkeypatch):
    """step_pipelined is step rotated to start at the first router layer: same tokens, same caches (the
    retrieved segments included), eagerly and replayed from a CUDA graph; with a layer's host gather started right
    after its attention ("dense") or with the next router layer's scoring ("routing")."""
    assert _routed_model(9).fetch_beside == "dense"        # what the rule picks for a bank this small
    monkeypatch.setenv("MSA_B200_DECODE_FETCH_BESIDE", beside)
    a, b, c = _routed_model(9), _routed_model(9), _routed_model(9)
    assert a.fetch_beside == beside
    n = 5
    toks_a = [a.step().cpu() for _ in range(n)]
    b.prime()
    toks_b = [b.step_pipelined().cpu() for _ in range(n)]
    torch.cuda.synchronize()
    for x, y in zip(toks_a, toks_b):
        assert torch.equal(x, y)
    for l in range(4):
        # b has already run the lower layers of the next step: compare the positions both have written
        L = int(a.kv_len[0])
        assert torch.equal(a.k_cache[l][:, :, :L], b.k_cache[l][:, :, :L])
        assert torch.equal(a.v_cache[l][:, :, :L], b.v_cache[l][:, :, :L])
    # the retrieved segment really changed (the fetch ran)
    fresh = _routed_model(9)
    lo, hi = a.s.template_len, a.s.template_len + a.retrieved
    assert not torch.equal(fresh.k_cache[2][:, :, lo:hi], a.k_cache[2][:, :, lo:hi])
    # graph replay of the rotated loop
    c.prime()
    c.step_pipelined()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        c.step_pipelined()
    c.reset()
    c.tokens.copy_(_routed_model(9).tokens)
    fresh2 = _routed_model(9)
    for l in range(4):
        c.k_cache[l].copy_(fresh2.k_cache[l])
        c.v_cache[l].copy_(fresh2.v_cache[l])
    c.prime()
    toks_c = []
    for _ in range(n):
        graph.replay()
        toks_c.append(c.tokens.cpu().clone())
    for x, y in zip(toks_a, toks_c):
        assert torch.equal(x, y)
    a.svc.check_status()
    for m in (a, b, c):
        m.check_fetch_counts()     # every step fetched a full retrieved segment for every sequence


def test_dense_glue_kernels_match_torch():
    """q/k norm + RoPE, residual add + RMSNorm and SiLU*up against the torch ops they replace (bf16 inputs,
    fp32 restatement, one bf16 rounding step of tolerance)."""
    from msa_b200 import ops
    g = torch.Generator().manual_seed(4)
    b, nq, nkv, d, hidden, ffn, eps = 5, 8, 2, 128, 2560, 1024, 1e-6
    qkv = torch.randn(b, (nq + 2 * nkv + nq) * d, generator=g).to(torch.bfloat16).to(DEV)
    qw = (1 + 0.1 * torch.randn(d, generator=g)).to(torch.bfloat16).to(DEV)
    kw = (1 + 0.1 * torch.randn(d, generator=g)).to(torch.bfloat16).to(DEV)
    ang = torch.rand(b, d // 2, generator=g) * 6.28
    emb = torch.cat([ang, ang], -1)
    cos, sin = emb.cos().to(torch.bfloat16).to(DEV), emb.sin().to(torch.bfloat16).to(DEV)
    q, k = ops.qk_norm_rope(qkv, nq, nkv, qw, kw, eps, cos, sin)

    def ref_heads(x, w):
        x = x.float()
        x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w.float()
        return O.rope_rotate_half(x, cos.float().unsqueeze(1), sin.float().unsqueeze(1))
    q_ref = ref_heads(qkv[:, : nq * d].view(b, nq, d), qw)
    k_ref = ref_heads(qkv[:, nq * d:(nq + nkv) * d].view(b, nkv, d), kw)
    assert (q.float() - q_ref).abs().max().item() < 3e-2 and rel(q.float(), q_ref) < 8e-3
    assert (k.float() - k_ref).abs().max().item() < 3e-2 and rel(k.float(), k_ref) < 8e-3

    x = torch.randn(b, hidden, generator=g).to(torch.bfloat16).to(DEV)
    y = torch.randn(b, hidden, generator=g).to(torch.bfloat16).to(DEV)
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16).to(DEV)
    x_new, h = ops.add_rmsnorm(x, y, w, eps)
    assert torch.equal(x_new, x + y)
    xs = (x + y).float()
    h_ref = xs * torch.rsqrt(xs.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    assert rel(h.float(), h_ref) < 8e-3
    x_same, h2 = ops.add_rmsnorm(x, None, w, eps)
    assert x_same is x and rel(h2.float(), F.rms_norm(x.float(), (hidden,), w.float(), eps)) < 8e-3

    gu = torch.randn(b, 2 * ffn, generator=g).to(torch.bfloat16).to(DEV)
    out = ops.silu_mul(gu, ffn)
    assert rel(out.float(), F.silu(gu[:, :ffn].float()) * gu[:, ffn:].float()) < 8e-3


def rel(a, b):
    return float((a - b).norm() / b.norm())

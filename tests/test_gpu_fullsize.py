"""Properties at the benchmark configurations' full sizes, where the CPU oracle is too slow to run whole.

Each test uses a property that does not depend on the size: invariance of the document score table
under a split of the shard (max is exact, so the tables must agree bit for bit), spot checks of sampled
(query, document) pairs against the oracle, top-k order and threshold against the table itself, merge of
per-shard candidates = top-k of the whole, linearity and mass conservation of chunk-mean pooling, split
invariance of decode attention, and a permutation round trip of the host gather.
"""
import pytest
import torch

from oracle import msa_oracle as O
from tests.util import check_topk

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HKV, D, GRP = 8, 128, 4


@pytest.fixture(scope="module")
def ops():
    from msa_b200 import ops as _ops
    return _ops


def _bank(n_docs, chunks_per_doc, seed):
    """bf16 router keys [C, Hkv, D] with per-document means (benchmark config 3/4 distribution)."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    mu = torch.randn((n_docs, 1, HKV, D), generator=g, device=DEV) * 0.5
    rk = mu + torch.randn((n_docs, chunks_per_doc, HKV, D), generator=g, device=DEV) / 8.0
    rk = torch.nn.functional.normalize(rk, dim=-1).to(torch.bfloat16).view(n_docs * chunks_per_doc, HKV, D)
    chunk_doc = torch.arange(1, n_docs + 1, device=DEV, dtype=torch.int32).repeat_interleave(chunks_per_doc)
    return rk, chunk_doc


def _score(ops, qf, bias, b, s_pad, rk, chunk_doc, n_docs):
    keys, status = ops.route_scores(qf, bias, b, s_pad, rk, chunk_doc, n_docs, alpha=1.0 / (HKV * GRP),
                                    min_val=torch.finfo(torch.bfloat16).min)
    assert status.cpu().tolist()[0] == 0
    return keys


def test_routing_config4_shard_properties(ops):
    """One of eight shards of benchmark config 4: 24,415 documents x 8 chunks (400 MB of keys),
    128 queries x 256 tokens (32,768 query rows: the two-CTA kernel's case)."""
    n_docs, cpd, b, s, k = 24415, 8, 128, 256, 16
    rk, chunk_doc = _bank(n_docs, cpd, seed=1)
    g = torch.Generator(device=DEV).manual_seed(2)
    q = torch.nn.functional.normalize(torch.randn((b, HKV * GRP, s, D), generator=g, device=DEV), dim=-1).to(torch.bfloat16)
    mask = torch.ones((b, s), dtype=torch.bool, device=DEV)
    mask[3, 100:] = False
    mask[7, :31] = False
    qf, bias, s_pad = ops.fold_queries(q, mask, GRP)
    keys = _score(ops, qf, bias, b, s_pad, rk, chunk_doc, n_docs)
    table = ops.keys_to_scores(keys)

    # (1) split invariance: documents [0, h) and [h, n) scored separately give the same bits
    h = 12001
    lo = _score(ops, qf, bias, b, s_pad, rk[: h * cpd], chunk_doc[: h * cpd], h)
    hi = _score(ops, qf, bias, b, s_pad, rk[h * cpd:].contiguous(), (chunk_doc[h * cpd:] - h).contiguous(), n_docs - h)
    assert torch.equal(keys[:, 1: h + 1], lo[:, 1:])
    assert torch.equal(keys[:, h + 1:], hi[:, 1:])

    # (2) a subset of the queries scored alone (fewer rows: the one-CTA kernel) agrees within the routing tolerance
    sub = [3, 7, 64, 127]
    qs, ms = q[sub].contiguous(), mask[sub].contiguous()
    qf2, bias2, s_pad2 = ops.fold_queries(qs, ms, GRP)
    t2 = ops.keys_to_scores(_score(ops, qf2, bias2, len(sub), s_pad2, rk, chunk_doc, n_docs))
    assert torch.allclose(t2, table[sub], atol=1e-3, rtol=0)

    # (3) sampled (query, document) pairs against the oracle
    gs = torch.Generator().manual_seed(3)
    docs = torch.randint(0, n_docs, (48,), generator=gs)
    rows = torch.cat([torch.arange(d * cpd, (d + 1) * cpd) for d in docs.tolist()])
    pool_ids = torch.arange(1, 49).repeat_interleave(cpd)
    q5 = qs.view(len(sub), HKV, GRP, s, D).float().cpu()
    ref = O.route_doc_scores(q5, ms.cpu(), rk[rows.to(DEV)].float().cpu().transpose(0, 1), pool_ids, 48)
    got = table[sub][:, (docs + 1).to(DEV)].cpu()
    assert torch.allclose(got, ref[:, 1:], atol=1e-3, rtol=0)

    # (4) top-k against the table itself: sorted, distinct, nothing above the threshold left out
    sc, li, _ = ops.topk_select(keys, k)
    check_topk(table, sc, li, k, tol=0.0)

    # (5) per-shard candidates merged = top-k of the whole (two shards, 2k candidates each)
    s_lo, l_lo, _ = ops.topk_select(lo, 2 * k)
    s_hi, l_hi, _ = ops.topk_select(hi, 2 * k)
    cs = torch.stack([s_lo, s_hi], dim=0)                        # [W, B, k']
    cl = torch.stack([l_lo, l_hi], dim=0)
    cg = torch.stack([l_lo, l_hi + h], dim=0)
    ms_, _, mg, mr = ops.topk_merge(cs, cl, cg, k)
    assert torch.equal(ms_, sc)
    same = torch.equal(mg, li)
    if not same:    # equal scores may be ordered differently: the sets of (score, id) must still agree per row
        for i in range(b):
            assert sorted(zip(ms_[i].tolist(), mg[i].tolist())) == sorted(zip(sc[i].tolist(), li[i].tolist()))
    assert ((mr == 0) == (mg <= h)).all()


def test_pooling_config2_linearity_and_mass(ops):
    """Benchmark config 2: 2,048 documents x 512 tokens, 8 heads x 128, chunk 64 (1 M tokens)."""
    n_docs, doc_len, p = 2048, 512, 64
    t = n_docs * doc_len
    doc_ids = torch.arange(1, n_docs + 1, device=DEV).repeat_interleave(doc_len).view(1, t)
    tok, off, _ = ops.chunk_bookkeeping(doc_ids, None, p)
    assert off.numel() - 1 == t // p and int(off[-1]) == t
    g = torch.Generator(device=DEV).manual_seed(5)
    a = torch.randn((1, HKV, t, D), generator=g, device=DEV)
    c = torch.randn((1, HKV, t, D), generator=g, device=DEV)
    pa, pc, pac = ops.pool_chunks(a, off, tok), ops.pool_chunks(c, off, tok), ops.pool_chunks(a + c, off, tok)
    assert torch.allclose(pac, pa + pc, atol=1e-5, rtol=0)                     # linearity (fp32)
    # mass: sum over chunks of len * mean = sum over tokens, per (head, dim)
    lens = (off[1:] - off[:-1]).float().view(-1, 1, 1)
    assert torch.allclose((pa * lens).sum(0), a[0].sum(1), atol=2e-2, rtol=1e-4)
    # a constant signal pools to itself, in bf16 too
    const = torch.full((1, HKV, t, D), 0.3125, device=DEV, dtype=torch.bfloat16)
    assert (ops.pool_chunks(const, off, tok) == 0.3125).all()
    # normalised pooling has unit rows
    pn = ops.pool_chunks(a, off, tok, l2_normalize=True)
    assert torch.allclose(pn.norm(dim=-1), torch.ones_like(pn[..., 0]), atol=1e-5)


def test_decode_config5_split_invariance(ops):
    """Benchmark config 5 layer: batch 32, 3 + 128 + 2048 cached entries, 32 q / 8 kv heads."""
    b, L = 32, 3 + 128 + 2048
    g = torch.Generator(device=DEV).manual_seed(6)
    kc = torch.randn((b, HKV, L + 4, D), generator=g, device=DEV).to(torch.bfloat16)
    vc = torch.randn((b, HKV, L + 4, D), generator=g, device=DEV).to(torch.bfloat16)
    q = torch.randn((b, HKV * GRP, D), generator=g, device=DEV).to(torch.bfloat16)
    nk = torch.randn((b, HKV, D), generator=g, device=DEV).to(torch.bfloat16)
    nv = torch.randn((b, HKV, D), generator=g, device=DEV).to(torch.bfloat16)
    kv_len = torch.full((b,), L, dtype=torch.int32, device=DEV)
    kv_len[5] = 17
    outs = []
    for n_splits in (1, 4, 16):
        k2, v2 = kc.clone(), vc.clone()
        outs.append(ops.sparse_decode_attn(q, k2, v2, kv_len.clone(), nk, nv, n_splits=n_splits).float())
        assert torch.equal(k2[0, :, L], nk[0]) and torch.equal(v2[5, :, 17], nv[5])      # appended in place
    for o in outs[1:]:
        assert (o - outs[0]).norm() / outs[0].norm() < 1e-2
    # two sequences against the oracle
    for i in (0, 5):
        n = int(kv_len[i])
        ref = O.decode_attention(q[i:i + 1].float().cpu().unsqueeze(2), kc[i:i + 1, :, :n].float().cpu(),
                                 vc[i:i + 1, :, :n].float().cpu(), torch.tensor([n]),
                                 nk[i:i + 1].float().cpu().unsqueeze(2), nv[i:i + 1].float().cpu().unsqueeze(2))[:, 0]
        got = outs[0][i].cpu().view(1, -1)
        assert (got - ref.reshape(1, -1)).norm() / ref.norm() < 1e-2


def test_gather_permutation_round_trip(ops):
    """Every document of a 4,096-document host bank fetched exactly once, in a random order: the
    result is a permutation of the bank's bytes."""
    n_docs, cpd, k = 4096, 8, 16
    g = torch.Generator().manual_seed(8)
    bank = torch.randn((n_docs * cpd, 2, HKV, D), generator=g).to(torch.bfloat16).pin_memory()
    lens = torch.tensor([0] + [cpd] * n_docs, dtype=torch.int32, device=DEV)
    offs = torch.cumsum(torch.cat([torch.zeros(1, dtype=torch.long, device=DEV), lens[:-1].long()]), 0)
    perm = torch.randperm(n_docs, generator=g)
    sel = (perm + 1).view(n_docs // k, k).to(DEV)
    plan, n_sel, total = ops.gather_plan(sel, None, 1, torch.zeros(1, dtype=torch.long, device=DEV), offs, lens,
                                         torch.tensor([bank.data_ptr()], dtype=torch.int64, device=DEV), 2 * HKV * D * 2)
    assert int(total.item()) == n_docs * cpd and (n_sel == k * cpd).all()
    out_k, out_v = ops.gather_run(plan, torch.bfloat16, HKV, D, n_docs * cpd)
    # within a sample the winners are fetched in ascending document order
    order = torch.sort(sel.cpu() - 1, dim=1).values.flatten()
    rows = (order.view(-1, 1) * cpd + torch.arange(cpd).view(1, -1)).flatten()
    assert torch.equal(out_k.cpu(), bank[rows, 0].permute(1, 0, 2))
    assert torch.equal(out_v.cpu(), bank[rows, 1].permute(1, 0, 2))

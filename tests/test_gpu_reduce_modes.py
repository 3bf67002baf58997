"""Routing in every combination of head / query / chunk reduce mode of ``Memory.prefill_stage2``
(src/msa_service.py:740-812), through ``msa_b200.memory.Memory`` and the C ABI underneath.

Reference values: the golden cases ``max_max_max`` and ``mean_max_mean`` produced by the reference's own
code (tests/golden/route_cases.npz), and the oracle on seeded ragged banks for all twelve combinations.
Tolerance: routing scores 1e-3 absolute, top-k exact outside a 1e-3 score gap.
"""
import pytest
import torch

from oracle import msa_oracle as O
from tests.util import T, check_topk, make_bank, ragged_docs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _memory(chunks, rk_chd, head, query, chunk, top_k, global_ids=None, cosine=True):
    from msa_b200.memory import AttentionGeometry, Document, Memory, ModelConfig
    geo = AttentionGeometry(num_hidden_layers=1, head_reduce_method=head, query_reduce_method=query,
                            chunk_reduce_method=chunk, dtype=rk_chd.dtype,
                            aux_loss_method="INFONCE" if cosine else "none")
    mem = Memory(0, None, ModelConfig(doc_top_k=top_k, router_layer_idx="0"), None, geo)
    ids = global_ids if global_ids is not None else list(range(100, 100 + len(chunks)))
    docs = [Document(doc_id=int(i), num_chunks=int(n)) for i, n in zip(ids, chunks)]
    zeros = torch.zeros_like(rk_chd)
    mem.load_pooled(docs, {0: (zeros, zeros, rk_chd.to(DEV))})
    return mem


@pytest.mark.parametrize("name", ["max_max_max", "mean_max_mean", "mean_max_max"])
def test_reduce_modes_golden_fp32(golden, name):
    g = golden("route_cases")
    head, query, chunk = name.split("_")
    chunks = g["chunks_per_doc"].tolist()
    mem = _memory(chunks, T(g["rk"]).transpose(0, 1).contiguous(), head, query, chunk, int(g["top_k"]),
                  g["global_ids"].tolist())
    q = T(g["q"]).to(DEV)
    mask = T(g["mask"]).to(DEV)
    s, li, gi = mem.prefill_stage2(0, q, mask.view(mask.shape[0], 1, 1, -1, 1))
    mem.check_status()
    ref_s = T(g[name + "__scores"])
    valid = ref_s > -1e9
    assert torch.allclose(s.cpu()[valid], ref_s[valid], atol=1e-4)
    # sample 2 has no routing token: every document ties there and the reference's order among ties is unspecified
    assert torch.equal(li.cpu()[:2], T(g[name + "__local_ids"])[:2])
    assert torch.equal(gi.cpu()[:2], T(g[name + "__global_ids"])[:2])
    assert (s.cpu()[2] == torch.finfo(torch.float32).min).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("chunk", ["max", "mean"])
@pytest.mark.parametrize("query", ["max", "mean", "last"])
@pytest.mark.parametrize("head", ["mean", "max"])
def test_reduce_modes_vs_oracle(head, query, chunk, dtype):
    b, s, grp, n_docs, k = 3, 40, 4, 70, 8
    chunks = ragged_docs(n_docs, 1, 9, seed=11)
    rk, pool_ids = make_bank(chunks, dtype=dtype, seed=12)
    gen = torch.Generator().manual_seed(13)
    q = torch.nn.functional.normalize(torch.randn(b, 8, grp, s, 128, generator=gen), dim=-1).to(dtype)
    mask = torch.ones(b, s, dtype=torch.bool)
    mask[0, s // 2:] = False
    mask[b - 1, s - 5:] = False
    table_ref = O.route_doc_scores(q.float(), mask, rk.float().transpose(0, 1), pool_ids, n_docs, head_reduce=head,
                                   query_reduce=query, chunk_reduce=chunk)
    mem = _memory(chunks, rk, head, query, chunk, k)
    sc, li, gi = mem.prefill_stage2(0, q.to(DEV), mask.to(DEV).view(b, 1, 1, s, 1))
    mem.check_status()
    check_topk(table_ref.clamp_min(torch.finfo(dtype).min), sc, li, k, tol=1e-3)
    assert torch.equal(gi.cpu(), li.cpu() + 99)      # local id i (1-based) -> global id 100 + i - 1


def test_chunk_table_and_reduce_entry_points_directly():
    """msa_route_chunk_scores + msa_route_reduce_chunks against a brute-force per-head computation, and the
    bounds check of the reducer: chunk ids outside 1..n_docs are skipped and counted."""
    from msa_b200 import ops
    chunks = [3, 1, 5, 2]
    rk, pool_ids = make_bank(chunks, dtype=torch.float32, seed=21)
    gen = torch.Generator().manual_seed(22)
    q = torch.randn(2, 32, 9, 128, generator=gen)
    mask = torch.ones(2, 9, dtype=torch.bool)
    mask[1, 6:] = False
    ck = ops.route_chunk_scores(q.to(DEV), mask.to(DEV), 4, rk.to(DEV), "max", "mean", scale=0.5)
    got = ops.keys_to_scores(ck)[:, 1:].cpu()
    dots = torch.einsum("bhsd,chd->bhsc", q, rk.repeat_interleave(4, dim=1)).amax(dim=1)       # [B, S, C]
    ref = torch.stack([dots[i][mask[i]].mean(0) for i in range(2)]) * 0.5
    assert torch.allclose(got, ref, atol=1e-4)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    bad = pool_ids.clone().to(torch.int32)
    bad[-2:] = 9                                     # a document id beyond n_docs = 4
    keys = ops.route_reduce_chunks(ck, bad.to(DEV), 4, "max", torch.finfo(torch.float32).min, status=status)
    torch.cuda.synchronize()
    assert status.cpu().tolist()[2] == 1             # one (skipped) document, counted once
    table = ops.keys_to_scores(keys).cpu()
    assert (table[:, 4] == torch.finfo(torch.float32).min).all()          # document 4 received nothing
    assert torch.allclose(table[:, 1], ref[:, :3].amax(dim=1), atol=1e-4)

"""The Memory / MSAService mirrors against the reference's own outputs (golden) and the oracle.

`doc_query` across ranks is checked twice: here on ONE GPU with the ranks' shards held by
separate Memory objects and the collectives replaced by stacking (everything but NCCL), and in
tests/test_gpu_multirank.py on two GPUs with real NCCL all-gathers.
"""
import pytest
import torch

from oracle import msa_oracle as O
from tests.util import T, make_bank, ragged_docs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _service(chunks, gids, k, v, rk, top_k, dtype, hkv=8, grp=4, d=128, **geo):
    from msa_b200.memory import AttentionGeometry, Document, ModelConfig
    from msa_b200.service import MSAService
    g = AttentionGeometry(num_hidden_layers=1, num_attention_heads=hkv * grp, num_key_value_heads=hkv, head_dim=d,
                          dtype=dtype, **geo)
    svc = MSAService(0, None, ModelConfig(doc_top_k=top_k, router_layer_idx="0"), None, g, world_size=1, rank=0)
    docs = [Document(doc_id=gid, num_chunks=n) for gid, n in zip(gids, chunks)]
    svc.load_pooled(docs, {0: (k.to(DEV), v.to(DEV), rk.to(DEV))})
    return svc


def test_prefill_stage2_golden(golden):
    g = golden("route_cases")
    rk = T(g["rk"]).transpose(0, 1).contiguous()           # [C, Hkv, D]
    chunks, gids = g["chunks_per_doc"].tolist(), g["global_ids"].tolist()
    svc = _service(chunks, gids, rk, rk, rk, int(g["top_k"]), torch.float32)
    q = T(g["q"]).to(DEV)
    mask = T(g["mask"]).view(3, 1, 1, 6, 1).to(DEV)
    s, li, gi = svc.prefill_stage2(0, q, mask)
    svc.check_status()
    assert torch.allclose(s.cpu()[:2], T(g["mean_max_max__scores"])[:2], atol=1e-4)
    assert torch.equal(li.cpu()[:2], T(g["mean_max_max__local_ids"])[:2])
    assert torch.equal(gi.cpu()[:2], T(g["mean_max_max__global_ids"])[:2])
    # reference-shaped views of the bank
    blk = svc.blocks[0]
    assert blk.rk_head_major.shape == (1, 8, sum(chunks), 128) and blk.k.shape == (1, 8, sum(chunks), 128)
    assert svc.get_max_local_pool_doc_id() == len(chunks)


def test_unknown_reduce_modes_are_rejected():
    """Every reduce mode of the reference is implemented (tests/test_gpu_reduce_modes.py); a name that is none of
    them is refused when the bank is created, not when the first query arrives."""
    from msa_b200 import _cabi as A
    z = torch.zeros(1, 8, 128)
    for kw in ({"head_reduce_method": "median"}, {"chunk_reduce_method": "sum"}, {"query_reduce_method": "first"}):
        with pytest.raises(A.MsaError, match="unknown"):
            _service([1], [5], z, z, z, 1, torch.float32, **kw)


def test_doc_query_golden_two_shards_one_gpu(golden):
    """Reference `MSAService.doc_query` on 2 gloo ranks vs this package's kernels with the two
    shards on one GPU: per-shard scoring of every rank's queries, merge, fetch from both banks."""
    from msa_b200 import ops
    from msa_b200.service import build_directory
    g = golden("doc_query_w2")
    w, top_k, grp = int(g["world"]), int(g["top_k"]), int(g["groups"])
    svcs = []
    for r in range(w):
        tr = lambda n: T(g[f"r{r}_{n}"]).transpose(0, 1).contiguous()
        svcs.append(_service(g[f"r{r}_chunks"].tolist(), g[f"r{r}_gids"].tolist(), tr("k"), tr("v"), tr("rk"), top_k,
                             torch.float32))
    base, offs, ln = build_directory([s.block_desc.doc_lens_cpu.tolist() for s in svcs])
    kv_base = torch.tensor([s.blocks[0].kv_device_address for s in svcs], dtype=torch.int64, device=DEV)
    for target in range(w):
        q, mask = T(g[f"r{target}_q"]).to(DEV), T(g[f"r{target}_mask"]).to(DEV)
        b, hq, s_len, d = q.shape
        qf, bias, s_pad = ops.fold_queries(q, mask, grp)
        cands = [svc.score_folded(0, qf, bias, b, s_pad, hq, top_k) for svc in svcs]
        sc = torch.stack([c[0] for c in cands]); li = torch.stack([c[1] for c in cands]); gi = torch.stack([c[2] for c in cands])
        fs, wl, wg, wr = ops.topk_merge(sc, li, gi, top_k)
        plan, n_sel, total = ops.gather_plan(wl, wr, w, base.to(DEV), offs.to(DEV), ln.to(DEV), kv_base,
                                             2 * 8 * 128 * 4)
        fk, fv = ops.gather_run(plan, torch.float32, 8, 128, int(total.item()))
        assert torch.allclose(fs.cpu(), T(g[f"r{target}_final_scores"]), atol=1e-4)
        assert torch.equal(wg.cpu(), T(g[f"r{target}_winner_global_ids"]))
        assert torch.equal(n_sel.cpu(), T(g[f"r{target}_num_selected"]))
        assert torch.equal(fk.cpu(), T(g[f"r{target}_final_k"]))
        assert torch.equal(fv.cpu(), T(g[f"r{target}_final_v"]))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_doc_query_single_rank_vs_oracle(dtype):
    chunks = ragged_docs(300, 1, 12, seed=17)
    gids = [1000 + 3 * i for i in range(len(chunks))]
    rk, pool_ids = make_bank(chunks, dtype=dtype, seed=18)
    g = torch.Generator().manual_seed(19)
    c = rk.shape[0]
    k = torch.randn(c, 8, 128, generator=g).to(dtype)
    v = torch.randn(c, 8, 128, generator=g).to(dtype)
    svc = _service(chunks, gids, k, v, rk, 16, dtype)
    b, s = 4, 48
    q = torch.nn.functional.normalize(torch.randn(b, 32, s, 128, generator=g), dim=-1).to(dtype)
    mask = torch.ones(b, s, dtype=torch.bool)
    mask[1, 30:] = False
    fk, fv, fs, n_sel, wg = svc.doc_query(q.to(DEV), mask.to(DEV), 0)
    svc.check_status()
    shard = O.Shard(k.float().transpose(0, 1), v.float().transpose(0, 1), rk.float().transpose(0, 1), chunks, gids)
    (rk_, rv_, rs_, rn_, rg_), = O.doc_query_world([q.float()], [mask], [shard], 16, 4)
    assert torch.allclose(fs.cpu(), rs_, atol=1e-3)
    # with well separated scores the winners, their order and therefore the fetched rows are identical
    gap = (rs_[:, :-1] - rs_[:, 1:]).min()
    if gap > 2e-3:
        assert torch.equal(wg.cpu(), rg_)
        assert torch.equal(n_sel.cpu(), rn_)
        assert torch.equal(fk.float().cpu(), rk_) and torch.equal(fv.float().cpu(), rv_)
    else:
        assert set(wg.cpu()[0].tolist()) & set(rg_[0].tolist())


def test_empty_shard_and_all_masked_queries():
    """A shard without documents and a batch whose queries have no routing token."""
    svc = _service([], [], torch.zeros(0, 8, 128, dtype=torch.bfloat16), torch.zeros(0, 8, 128, dtype=torch.bfloat16),
                   torch.zeros(0, 8, 128, dtype=torch.bfloat16), 4, torch.bfloat16)
    q = torch.randn(2, 32, 16, 128).to(torch.bfloat16).to(DEV)
    mask = torch.zeros(2, 16, dtype=torch.bool, device=DEV)
    fk, fv, fs, n_sel, wg = svc.doc_query(q, mask, 0)
    assert fs.shape == (2, 1) and (fs.cpu() == torch.finfo(torch.bfloat16).min).all()
    assert fk.shape == (8, 0, 128) and n_sel.cpu().tolist() == [0, 0]
    chunks = [3, 2]
    rk, _ = make_bank(chunks, dtype=torch.bfloat16, seed=1)
    svc = _service(chunks, [7, 9], rk, rk, rk, 4, torch.bfloat16)
    fk, fv, fs, n_sel, wg = svc.doc_query(q, mask, 0)
    assert (fs.cpu() <= -1e9).all() and n_sel.cpu().tolist() == [0, 0] and fk.shape[1] == 0


def test_bounded_wait_gives_up_and_reports():
    """A barrier wait that can never complete runs into its limit: the kernel returns, the status
    words say so, and the context keeps working (no trap, no hang)."""
    import time
    from msa_b200 import _cabi as A, ops
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    t0 = time.perf_counter()
    A.check(A.lib().msa_selftest_bounded_wait(20_000_000, A.ptr(status), A.stream_ptr(status.device)), "selftest")
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert status.cpu().tolist()[:2] == [9, 1]
    assert 0.015 < dt < 1.0
    # the device is still usable afterwards
    keys = torch.zeros((2, 5), dtype=torch.int32, device=DEV)
    ops.route_table_reset(keys, 4, -1.0)
    assert (ops.keys_to_scores(keys).cpu() == -1.0).all()
    # and Memory.check_status turns a non-zero status word into an exception
    svc = _service([1], [5], torch.zeros(1, 8, 128), torch.zeros(1, 8, 128), torch.zeros(1, 8, 128), 1, torch.float32)
    svc._status.copy_(status)
    with pytest.raises(A.MsaError, match="gave up"):
        svc.check_status()


@pytest.mark.parametrize("map_host_bank", [True, False])
def test_bank_serialize_roundtrip(tmp_path, map_host_bank):
    import os, tempfile
    if map_host_bank and os.path.isdir("/dev/shm"):      # a file system whose pages can be pinned in place
        tmp_path = type(tmp_path)(tempfile.mkdtemp(dir="/dev/shm", prefix="msa_b200_test_"))
    """A shard written to disk and loaded back (K/V bank mapped and pinned in place, or read into
    pinned memory) answers doc_query exactly as the original."""
    chunks = ragged_docs(60, 1, 9, seed=41)
    gids = [500 + i for i in range(len(chunks))]
    rk, _ = make_bank(chunks, dtype=torch.bfloat16, seed=42)
    g = torch.Generator().manual_seed(43)
    k = torch.randn(rk.shape, generator=g).to(torch.bfloat16)
    v = torch.randn(rk.shape, generator=g).to(torch.bfloat16)
    svc = _service(chunks, gids, k, v, rk, 4, torch.bfloat16)
    svc.template_prefix_kvcache = {0: (torch.ones(1, 8, 3, 128, device=DEV), torch.zeros(1, 8, 3, 128, device=DEV))}
    q = torch.nn.functional.normalize(torch.randn(3, 32, 20, 128, generator=g), dim=-1).to(torch.bfloat16).to(DEV)
    mask = torch.ones(3, 20, dtype=torch.bool, device=DEV)
    ref = svc.doc_query(q, mask, 0)
    svc.serialize(str(tmp_path / "bank"))
    svc2 = _service([], [], torch.zeros(0, 8, 128, dtype=torch.bfloat16), torch.zeros(0, 8, 128, dtype=torch.bfloat16),
                    torch.zeros(0, 8, 128, dtype=torch.bfloat16), 4, torch.bfloat16)
    svc2._directory = None
    svc2.deserialize(str(tmp_path / "bank"), map_host_bank=map_host_bank)
    out = svc2.doc_query(q, mask, 0)
    for a, b in zip(ref, out):
        assert torch.equal(a, b)
    assert torch.equal(svc2.get_template_prefix_kvcaches(0)[0], svc.get_template_prefix_kvcaches(0)[0])
    assert [d.doc_id for d in svc2.block_desc.docs] == gids
    assert svc2.bank_placement == ("mapped in place" if map_host_bank and os.path.isdir("/dev/shm") else
                                   "copied to pinned memory")
    svc2.release_mapped_banks()
    if str(tmp_path).startswith("/dev/shm/"):
        import shutil
        shutil.rmtree(str(tmp_path), ignore_errors=True)

"""Memory Parallel on two GPUs with real NCCL all-gathers and shared pinned host banks, checked
against the outputs the REFERENCE's MSAService.doc_query produced on two gloo ranks
(tests/golden/doc_query_w2.npz).  Skipped on a box with a single GPU."""
import os

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "doc_query_w2.npz")


def _rank(rank, world, port, ret):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from msa_b200.memory import AttentionGeometry, Document, ModelConfig
    from msa_b200.service import MSAService
    g = dict(np.load(GOLDEN))
    T = lambda n: torch.from_numpy(g[f"r{rank}_{n}"])
    geo = AttentionGeometry(num_hidden_layers=1, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                            dtype=torch.float32)
    svc = MSAService(rank, None, ModelConfig(doc_top_k=int(g["top_k"]), router_layer_idx="0"), None, geo,
                     world_size=world, rank=rank)
    docs = [Document(doc_id=int(i), num_chunks=int(n)) for i, n in zip(g[f"r{rank}_gids"], g[f"r{rank}_chunks"])]
    tr = lambda n: T(n).transpose(0, 1).contiguous().to(dev)
    svc.load_pooled(docs, {0: (tr("k"), tr("v"), tr("rk"))})
    svc.share_host_banks(tag=f"t{port}")
    outs = []
    for _ in range(2):   # twice: the second call reuses every cached table
        fk, fv, fs, n_sel, wg = svc.doc_query(T("q").to(dev), T("mask").to(dev), 0)
        outs.append([x.cpu() for x in (fk, fv, fs, n_sel, wg)])
    # a decode-shaped call (one token per sequence, every mask all ones): the bias all-gather may be skipped
    q1 = T("q")[:, :, :1].contiguous().to(dev)
    m1 = torch.ones(q1.shape[0], 1, dtype=torch.bool, device=dev)
    a = svc.route(q1, m1, 0)
    b = svc.route(q1, m1, 0, all_valid=True)
    assert all(torch.equal(x, y) for x, y in zip(a, b))
    svc.check_status()
    svc.close_host_banks()
    ret[rank] = outs
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_doc_query_two_gpus_matches_reference_golden():
    world = 2
    ret = mp.Manager().dict()
    mp.spawn(_rank, args=(world, 29755, ret), nprocs=world, join=True)
    g = dict(np.load(GOLDEN))
    for rank in range(world):
        for fk, fv, fs, n_sel, wg in ret[rank]:
            R = lambda n: torch.from_numpy(g[f"r{rank}_{n}"])
            assert torch.allclose(fs, R("final_scores"), atol=1e-4)
            assert torch.equal(wg, R("winner_global_ids"))
            assert torch.equal(n_sel, R("num_selected"))
            assert torch.equal(fk, R("final_k")) and torch.equal(fv, R("final_v"))

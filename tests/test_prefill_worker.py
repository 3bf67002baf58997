"""The stage-1 worker process (msa_b200.prefill.PrefillStage1Worker): the reference's queue protocol
(src/prefill.py:31-35, 112-140; src/types.py:11-21), block splitting, block inputs, and the shared-memory transfer
of the pooled tensors.  The CPU tests run the worker in a spawned process with a stand-in model; the GPU test builds
a bank through the worker (real stage-1 kernels in the worker process) and compares it with a bank filled directly."""
import os

import pytest
import torch
import torch.multiprocessing as mp

TEMPLATE = {"prompt": "<|im_start|>user\n{prompt}<|im_end|>\n"}
FACTORY = "tests.fake_stage1:factory"


def _docs(pool):
    from msa_b200.memory import Document
    from msa_b200.tools import compose_input
    from tests.fake_stage1 import ByteTokenizer
    tok = ByteTokenizer()
    texts = ["alpha beta gamma", "x", "the quick brown fox jumps over the lazy dog", "memory sparse attention", "tail"]
    docs = []
    for i, t in enumerate(texts):
        n = len(compose_input(t, i, tok)[1]["input_ids"])
        docs.append(Document(doc=t, doc_id=i, num_chunks=(n + pool - 1) // pool))
    return docs


def test_split_docs_and_block_inputs():
    from msa_b200.memory import Document
    from msa_b200.prefill import PrefillStage1Worker
    docs = [Document(doc_id=i, num_chunks=n) for i, n in enumerate([3, 3, 5, 9, 1, 1])]
    blocks = PrefillStage1Worker.split_docs(docs, 6)
    assert [[d.doc_id for d in b] for b in blocks] == [[0, 1], [2], [3], [4, 5]]      # an oversized document stands alone
    os.environ["MSA_B200_MODEL_FACTORY"] = FACTORY
    try:
        w = PrefillStage1Worker(0, "unused", TEMPLATE, 4, {}) if not torch.cuda.is_available() else None
    finally:
        os.environ.pop("MSA_B200_MODEL_FACTORY", None)
    if w is None:
        pytest.skip("block inputs are checked on the CPU stand-in")
    docs = _docs(4)
    x = w._prepare_block_inputs(docs[:2])
    head = len(w.template_head_input_ids)
    assert x.doc_ids[0, :head].tolist() == [-2] * head and x.position_ids[0, :head].tolist() == list(range(head))
    n0 = docs[0].num_chunks
    ids = x.doc_ids[0, head:].tolist()
    assert set(ids) == {1, 2} and ids == sorted(ids)                      # 1-based index INSIDE the block
    first = ids.count(1)
    assert x.position_ids[0, head:head + first].tolist() == list(range(first))       # positions restart per document
    assert x.position_ids[0, head + first].item() == 0
    assert x.chunk_sizes == [n0, docs[1].num_chunks] and x.num_chunks == n0 + docs[1].num_chunks
    bad = [type(docs[0])(doc=docs[0].doc, doc_id=0, num_chunks=docs[0].num_chunks + 1)]
    with pytest.raises(AssertionError, match="pre calculated chunk"):
        w._prepare_block_inputs(bad)


def test_worker_process_protocol_and_shared_memory_payload(tmp_path):
    """READY -> MEMORY_DOCS -> one META per block -> CLOSE, in a spawned process; every META's pooled tensors come
    through a shared-memory file and equal what the same model gives in this process."""
    if torch.cuda.is_available():
        pytest.skip("host-only protocol test (the GPU variant is test_bank_built_through_the_worker)")
    from msa_b200.cache import SparseCacheOnCPU
    from msa_b200.prefill import PrefillStage1Worker
    from tests.fake_stage1 import CpuStandIn
    pool, block_size = 4, 12
    docs = _docs(pool)
    ctx = mp.get_context("spawn")
    req, rsp = ctx.Queue(), ctx.Queue()
    envs = {"MSA_B200_MODEL_FACTORY": FACTORY, "MSA_B200_SHM_DIR": str(tmp_path)}
    p = ctx.Process(target=PrefillStage1Worker.prefill_worker_main,
                    args=(0, req, rsp, "unused", TEMPLATE, pool, block_size, envs))
    p.start()
    PrefillStage1Worker.wait_for_ready(rsp)
    PrefillStage1Worker.send_documents(req, docs)
    blocks = PrefillStage1Worker.split_docs(docs, block_size)
    assert len(blocks) > 1
    os.environ["MSA_B200_MODEL_FACTORY"] = FACTORY
    local = PrefillStage1Worker(0, "unused", TEMPLATE, pool, {})
    os.environ.pop("MSA_B200_MODEL_FACTORY")
    model = CpuStandIn()
    for block in blocks:
        meta = PrefillStage1Worker.recv_meta(rsp)
        assert set(meta) == {"chunk_sizes", "past_key_values", "nr_docs", "doc_ids", "nr_chunks"}
        assert meta["nr_docs"] == len(block) and meta["doc_ids"] == [d.doc_id for d in block]
        assert meta["nr_chunks"] == [d.num_chunks for d in block] == meta["chunk_sizes"]
        x = local._prepare_block_inputs(block)
        ref = SparseCacheOnCPU()
        model.model(input_ids=x.doc_input_ids, attention_mask=x.doc_attention_mask, position_ids=x.position_ids,
                    past_key_values=ref, doc_ids=x.doc_ids)
        got = meta["past_key_values"]
        assert os.path.exists(got.path) and os.path.dirname(got.path) == str(tmp_path)
        k, v = got.get_kvcache(1)
        rk, rv = ref.get_kvcache(1)
        assert k.shape == rk.shape == (1, 2, sum(meta["nr_chunks"]), 128)
        assert torch.equal(k, rk) and torch.equal(v, rv) and torch.equal(got.get_router_kcache(1), ref.get_router_kcache(1))
        assert got.kv_chunk_major(1).shape == (sum(meta["nr_chunks"]), 2, 2, 128)       # the bank's own layout
        assert torch.equal(got.cache_kwargs[1]["pooled_doc_ids"], ref.cache_kwargs[1]["pooled_doc_ids"])
        assert torch.equal(got.cache_kwargs[0]["template_prefix_kcache"], ref.cache_kwargs[0]["template_prefix_kcache"])
        got.clear_kvcache()
        assert not os.path.exists(got.path)
    PrefillStage1Worker.close_worker(req)
    p.join(60)
    assert p.exitcode == 0


@pytest.mark.gpu
def test_bank_built_through_the_worker(tmp_path):
    """Memory.generate_blocks pulls the META payloads from its own worker process (real stage 1 on the GPU there);
    the bank must equal one filled from the same model's pooled tensors computed in this process."""
    from msa_b200.cache import SparseCacheOnCPU
    from msa_b200.memory import AttentionGeometry, MemoryConfig, ModelConfig
    from msa_b200.prefill import PrefillStage1Worker
    from msa_b200.service import MSAService
    from tests.fake_stage1 import ByteTokenizer, gpu_model
    from types import SimpleNamespace
    pool, block_size = 64, 3
    docs = _docs(pool)
    long_text = " ".join(f"word{i}" for i in range(60))
    from msa_b200.memory import Document
    from msa_b200.tools import compose_input
    n = len(compose_input(long_text, 5, ByteTokenizer())[1]["input_ids"])
    docs.append(Document(doc=long_text, doc_id=5, num_chunks=(n + pool - 1) // pool))
    geo = AttentionGeometry(num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=128)
    envs = {"MSA_B200_MODEL_FACTORY": FACTORY, "MSA_B200_SHM_DIR": str(tmp_path)}
    svc = MSAService(0, SimpleNamespace(template=TEMPLATE, world=1),
                     ModelConfig(model_path="unused", doc_top_k=2, pooling_kernel_size=pool, router_layer_idx="1", envs=envs),
                     MemoryConfig(block_size=block_size, pooling_kernel_size=pool), geo, world_size=1, rank=0)
    svc.generate_blocks(docs)
    assert not os.listdir(tmp_path)                       # every block file was consumed and removed
    # the same blocks through the same (seeded) model in this process
    os.environ["MSA_B200_MODEL_FACTORY"] = FACTORY
    local = PrefillStage1Worker(0, "unused", TEMPLATE, pool, {})
    os.environ.pop("MSA_B200_MODEL_FACTORY")
    ks, vs, rks, pooled = [], [], [], []
    for block in PrefillStage1Worker.split_docs(docs, block_size):
        x = local._prepare_block_inputs(block)
        cache = SparseCacheOnCPU()
        for layer in range(2):
            cache.record_kwargs(layer, {"stage": "prefill_stage1"})
        with torch.no_grad():
            local.model.model(input_ids=x.doc_input_ids.cuda(), attention_mask=x.doc_attention_mask.cuda(),
                              position_ids=x.position_ids.cuda(), past_key_values=cache, doc_ids=x.doc_ids.cuda())
        k, v = cache.get_kvcache(1)
        ks.append(k[0].permute(1, 0, 2)); vs.append(v[0].permute(1, 0, 2)); rks.append(cache.get_router_kcache(1)[0].permute(1, 0, 2))
    blk = svc.blocks[1]
    assert blk.kv.shape[0] == sum(d.num_chunks for d in docs)
    assert torch.equal(blk.kv[:, 0], torch.cat(ks)) and torch.equal(blk.kv[:, 1], torch.cat(vs))
    assert torch.equal(blk.rk.cpu(), torch.cat(rks))
    assert svc.block_desc.pool_ids.cpu().tolist() == [i + 1 for i, d in enumerate(docs) for _ in range(d.num_chunks)]
    assert set(svc.template_prefix_kvcache) == {0, 1}

"""Host-side logic that needs no GPU: ABI surface, partitioning, directory, candidate packing,
and the all-gather layouts of the Memory-Parallel exchange on 2 gloo ranks."""
import os
import re

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_loads_and_exports_every_declared_symbol():
    from msa_b200 import _cabi as A
    from msa_b200.build import build
    build()
    lib = A.lib()
    header = open(os.path.join(ROOT, "include", "msa_b200.h")).read()
    declared = set(re.findall(r"\b(msa_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(A.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.msa_abi_version() == 2
    assert lib.msa_route_s_pad(256, 0) == 256 and lib.msa_route_s_pad(100, 0) == 112
    assert lib.msa_route_s_pad(300, 0) == 320 and lib.msa_route_s_pad(1, 0) == 1 and lib.msa_route_s_pad(77, 1) == 1
    assert lib.msa_decode_workspace_bytes(2, 32, 128, 4) == 2 * 32 * 4 * 130 * 4


def test_argument_errors_are_reported_before_any_launch():
    from msa_b200 import _cabi as A
    lib = A.lib()
    assert lib.msa_pool_chunks(None, 1, 0, 0, None, None, None, 1, 8, 128, None, 0, 0, 0, None) == -1
    assert b"null pointer" in lib.msa_last_error()
    assert lib.msa_topk_select(1, 8, 1, 4, 5000, None, 1, 1, None, None, 0, None) == -1
    assert b"exceeds the supported maximum" in lib.msa_last_error()
    # msa_gather_plan: directory smaller than the shards' dummy rows, negative per-sample room
    assert lib.msa_gather_plan(1, None, 1, 4, 2, 1, 1, 1, 1, 1, 4096, 0, 1, 1, 1, None, None, None) == -1
    assert b"n_dir_rows" in lib.msa_last_error()
    assert lib.msa_gather_plan(1, None, 1, 4, 1, 1, 8, 1, 1, 1, 4096, -1, 1, 1, 1, None, None, None) == -1
    assert b"sample_stride" in lib.msa_last_error()
    assert lib.msa_gather_run(1, 4, 1, 8, 128, 1, 1, 1024, 4, -16, 0, None) == -1
    # the resident-set plan needs a table and slots of at least one entry
    assert lib.msa_gather_plan_resident(1, None, 1, 4, 1, 1, 8, 1, 1, 1, 4096, 2, None, 1, 1, 1, None, None) == -1
    assert b"null pointer" in lib.msa_last_error()
    assert lib.msa_gather_plan_resident(1, None, 1, 4, 1, 1, 8, 1, 1, 1, 4096, 0, 1, 1, 1, 1, None, None) == -1
    assert b"resident table needs" in lib.msa_last_error()
    # reduce modes
    assert lib.msa_route_chunk_scores(None, 1, 0, 0, 0, None, 0, 1, 32, 4, 8, 128, 7, 0, None, 1024, 4, 1.0, 0.0, None, 5,
                                      None) == -1
    assert b"head_reduce" in lib.msa_last_error()
    assert lib.msa_route_reduce_chunks(None, 5, 1, 4, None, 2, 3, 0.0, None, 3, None, None) == -1
    assert b"chunk_reduce" in lib.msa_last_error()
    # fused decode-time routing: shapes it does not take are refused with MSA_ERR_UNSUPPORTED before any launch
    one = 1       # any non-null pointer value: nothing is dereferenced on these paths
    unsupported = A.lib().msa_route_score_select(one, one, A.dtype_code(torch.float32), 4, one, 1024, 4096, 1024, one, 1.0, 8, -1e38,
                                                 16, None, one, one, None, one, 1 << 20, 0, one, None)
    assert unsupported not in (0, -1) and b"at most 128 sequences" in lib.msa_last_error()
    assert lib.msa_route_score_select(one, one, A.dtype_code(torch.bfloat16), 200, one, 1024, 4096, 1024, one, 1.0, 8, -1e38,
                                      16, None, one, one, None, one, 1 << 20, 0, one, None) == unsupported
    assert lib.msa_route_score_select(one, one, A.dtype_code(torch.bfloat16), 4, one, 1024, 4096, 1024, one, 0.0, 8, -1e38,
                                      16, None, one, one, None, one, 1 << 20, 0, one, None) == -1
    assert b"alpha must be positive" in lib.msa_last_error()
    assert lib.msa_router_keys_blocked_bytes(129, 1024) == 2 * 16 * 128 * 64 * 2
    # tcgen05 attention entry points: dtype / head size, store layout and bitmap size are checked before any tensor map
    bf16, f32 = A.dtype_code(torch.bfloat16), A.dtype_code(torch.float32)
    ctx = lambda dtype, d, stride_h: lib.msa_sparse_prefill_attn_tc(
        256, 64 * 8 * d, d, 8 * d, 256, 256, 2 * 100 * d, stride_h, 100, one, one, one, one, 2, 64, 8, 2, d, dtype, 1, 0.1,
        256, one, None)
    assert ctx(f32, 128, 100 * 128) == -1 and b"bf16 with head_dim 128 only" in lib.msa_last_error()
    assert ctx(bf16, 64, 100 * 64) == -1 and b"bf16 with head_dim 128 only" in lib.msa_last_error()
    assert ctx(bf16, 128, 101 * 128) == -1 and b"contiguous [B, Hkv, store_len, D]" in lib.msa_last_error()
    masked = lambda words: lib.msa_doc_attention_tc_masked(
        256, 0, 128, 8 * 128, 256, 256, 0, 128, 2 * 128, one, one, 1, 300, 1, 1000, 8, 2, 128, bf16, 0.1, 256, one, words,
        one, None)
    assert masked(1000 // 32) == -1 and b"bitmap must cover" in lib.msa_last_error()
    with pytest.raises(A.MsaError, match="CUDA tensors"):
        from msa_b200 import ops
        ops.pool_chunks(torch.zeros(4, 8, 128), torch.tensor([0, 4], dtype=torch.int32))


def test_balanced_bucket_partition_and_directory():
    from msa_b200.memory import Document
    from msa_b200.service import balanced_bucket_partition, build_directory
    docs = [Document(doc_id=i, num_chunks=n) for i, n in enumerate([9, 1, 1, 8, 3, 3, 7, 2])]
    buckets = balanced_bucket_partition(docs, 3)
    loads = [sum(d.num_chunks for d in b) for b in buckets]
    assert sorted(d.doc_id for b in buckets for d in b) == list(range(8))
    assert max(loads) - min(loads) <= 2
    base, offs, lens = build_directory([[0, 2, 3], [0, 5], [0]])
    assert base.tolist() == [0, 3, 5]
    assert lens.tolist() == [0, 2, 3, 0, 5, 0] and offs.tolist() == [0, 0, 2, 0, 0, 0]


def test_candidate_buffer_roundtrip():
    """Scores and ids written into the planes of one buffer come back bit for bit from a stack of such buffers."""
    from msa_b200 import ops
    s = torch.tensor([[0.5, -3.4e38, float("-inf")], [1e-9, -0.0, 7.0]])
    l = torch.tensor([[1, 2, 0], [9, 8, 7]])
    bufs = []
    for w in range(3):
        buf, sv, lv, gv = ops.candidate_buffer(2, 3, "cpu")
        sv.copy_(s + w); lv.copy_(l + w); gv.copy_(l + 100 + w)
        bufs.append(buf)
    s2, l2, g2 = ops.candidate_views(torch.stack(bufs))
    for w in range(3):
        assert torch.equal(s2[w].contiguous().view(torch.int32), (s + w).view(torch.int32))
        assert torch.equal(l2[w], l + w) and torch.equal(g2[w], l + 100 + w)
    assert s2.stride(2) == 1 and s2.stride(1) == 3 and l2.stride(1) == 3     # what the merge kernel requires


def _rank(rank, world, port, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from msa_b200 import ops
    from msa_b200.service import all_gather_cat, build_directory
    b, k = 3, 4
    # every rank scored ALL world*b queries against its shard; candidates are gathered to [W, B_all, k]
    scores = torch.arange(world * b * k, dtype=torch.float32).view(world * b, k) + 1000 * rank
    local = torch.full((world * b, k), rank + 1)
    buf, sv, lv, gv = ops.candidate_buffer(world * b, k, "cpu")
    sv.copy_(scores); lv.copy_(local); gv.copy_(local + 10)
    s, l, g = ops.candidate_views(all_gather_cat(buf, world))
    lens = [None] * world
    dist.all_gather_object(lens, [0] + [rank + 1] * (rank + 2))
    base, offs, ln = build_directory(lens)
    ret[rank] = (s.clone(), l.clone(), base.tolist(), ln.tolist())
    dist.barrier()
    dist.destroy_process_group()


def test_exchange_layout_two_gloo_ranks():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_rank, args=(world, 29733, ret), nprocs=world, join=True)
    for rank in range(world):
        s, l, base, ln = ret[rank]
        assert s.shape == (world, world * 3, 4)
        for owner in range(world):
            assert (l[owner] == owner + 1).all()
            assert s[owner, 0, 0] == 1000 * owner
        assert base == [0, 3] and ln == [0, 1, 1, 0, 2, 2, 2]
    assert torch.equal(ret[0][0], ret[1][0])


def test_tensor_layouts_the_tcgen05_attention_accepts():
    """ops._tc_view_ok: token-major views (what the layer's projections give) and contiguous head-major tensors."""
    import torch
    from msa_b200 import ops
    b, h, s, d = 2, 4, 24, 128
    token_major = torch.zeros(b, s, h, d, dtype=torch.bfloat16).transpose(1, 2)
    head_major = torch.zeros(b, h, s, d, dtype=torch.bfloat16)
    fused = torch.zeros(b, s, 3 * h * d, dtype=torch.bfloat16)[:, :, h * d: 2 * h * d].view(b, s, h, d).transpose(1, 2)
    assert ops._tc_view_ok(token_major) and ops._tc_view_ok(head_major) and ops._tc_view_ok(fused)
    assert ops._tc_view_ok(head_major[:, :, ::2])                        # every other token: still one stride per row
    assert not ops._tc_view_ok(head_major[:, :, :10])                    # a window of tokens: heads no longer evenly spaced
    assert not ops._tc_view_ok(torch.zeros(b, h, d, s, dtype=torch.bfloat16).transpose(2, 3))   # feature axis not contiguous
    assert not ops._tc_view_ok(head_major.permute(1, 0, 2, 3).contiguous().permute(1, 0, 2, 3))  # batch inside heads


def test_decode_loop_places_the_host_gather_by_shard_and_fetch_size():
    """SparseDecodeModel._fetch_placement on the benchmark's sizes: beside the scoring kernel on 1-2 GPUs, beside the
    dense GEMMs from 4 GPUs on, and beside the GEMMs whenever there is no bank to score."""
    from types import SimpleNamespace
    import torch
    from msa_b200.decoder import DecoderShape, SparseDecodeModel
    shape = DecoderShape()
    chunks = 1_562_560
    picks = {}
    for world in (1, 2, 4, 8):
        rk = torch.empty((chunks // world, shape.n_kv_heads, shape.head_dim), dtype=torch.bfloat16, device="meta")
        for stored in ("rows", "blocked"):
            blk = SimpleNamespace(rk=rk if stored == "rows" else None, rk_blocked=None if stored == "rows" else rk)
            me = SimpleNamespace(svc=SimpleNamespace(blocks={18: blk, 19: blk}, world_size=world), router_layers={18, 19}, s=shape,
                                 batch=32 // world, retrieved=128, dtype=torch.bfloat16)      # a rank decodes its share of the batch
            picks[world, stored] = SparseDecodeModel._fetch_placement(me)
    assert [picks[w, "rows"] for w in (1, 2, 4, 8)] == ["routing", "routing", "dense", "dense"]
    assert all(picks[w, "blocked"] == picks[w, "rows"] for w in (1, 2, 4, 8))
    empty = SimpleNamespace(svc=None, router_layers=set(), s=shape, batch=32, retrieved=128, dtype=torch.bfloat16)
    assert SparseDecodeModel._fetch_placement(empty) == "dense"


def test_span_tables_of_documents_with_masked_tokens():
    """ops.document_spans / ops.token_bitmap: what the tcgen05 kernel takes for documents with masked tokens inside."""
    import torch
    from msa_b200 import ops
    g = torch.Generator().manual_seed(3)
    mask = torch.rand(2, 75, generator=g) < 0.6
    bits = ops.token_bitmap(mask)
    flat = mask.reshape(-1)
    assert bits.dtype == torch.int32 and bits.numel() == (150 + 256 + 31) // 32 + 1
    for pos in range(150 + 64):
        want = bool(flat[pos]) if pos < 150 else False
        assert bool((int(bits[pos >> 5]) >> (pos & 31)) & 1) == want
    # three documents as token lists with holes: spans run from the first to the last listed token
    tok = torch.tensor([4, 5, 7, 20, 21, 22, 40, 44], dtype=torch.int32)
    off = torch.tensor([0, 3, 6, 8], dtype=torch.int32)
    index, span_off, longest = ops.document_spans(tok, off)
    assert index.tolist() == [4, 5, 6, 7, 20, 21, 22, 40, 41, 42, 43, 44]
    assert span_off.tolist() == [0, 4, 7, 12] and longest == 5 and index.dtype == span_off.dtype == torch.int32


def test_reference_format_bank_is_detected_and_converted(tmp_path):
    """A bank directory in the reference's on-disk format (src/msa_service.py:351-420) is recognised, and the
    one-time converter writes this package's chunk-major raw files with the same numbers."""
    import json
    import sys
    import types
    from dataclasses import dataclass

    import numpy as np
    from msa_b200.memory import convert_reference_bank, is_reference_bank

    @dataclass
    class RefDocument:           # pickles as src.types.Document, the class the reference's meta.pt refers to
        doc: str = ""
        doc_id: int = 0
        num_chunks: int = 0
    RefDocument.__module__, RefDocument.__qualname__, RefDocument.__name__ = "src.types", "Document", "Document"
    had = {n: sys.modules.get(n) for n in ("src", "src.types")}
    mod = types.ModuleType("src.types")
    mod.Document = RefDocument
    sys.modules["src"], sys.modules["src.types"] = types.ModuleType("src"), mod
    src, dst = tmp_path / "ref", tmp_path / "new"
    src.mkdir()
    try:
        docs = [RefDocument(doc_id=5, num_chunks=2), RefDocument(doc_id=9, num_chunks=3)]
        json.dump({"world": 1}, open(src / "stub.json", "w"))
        torch.save({"router_layer_ids": [1], "block_desc": {"docs": docs, "doc_ids": torch.tensor([0, 5, 9]),
                                                            "pool_ids": torch.tensor([1, 1, 2, 2, 2])}}, src / "meta.pt")
        g = torch.Generator().manual_seed(0)
        k, v, rk = (torch.randn(1, 2, 5, 4, generator=g) for _ in range(3))
        for n, t in (("k", k), ("v", v), ("rk", rk)):
            torch.save(t, src / f"layer_1_{n}.pt")
    finally:
        for n, m in had.items():
            if m is None:
                sys.modules.pop(n, None)
            else:
                sys.modules[n] = m
    assert is_reference_bank(str(src))
    meta = convert_reference_bank(str(src), str(dst))
    assert meta["doc_ids"] == [5, 9] and meta["doc_chunks"] == [2, 3] and meta["n_chunks"] == 5
    assert not is_reference_bank(str(dst))
    kv = torch.from_numpy(np.fromfile(dst / "kv_L1.bin", dtype=np.float32)).view(5, 2, 2, 4)
    rk2 = torch.from_numpy(np.fromfile(dst / "rk_L1.bin", dtype=np.float32)).view(5, 2, 4)
    assert torch.equal(kv[:, 0].permute(1, 0, 2), k[0]) and torch.equal(kv[:, 1].permute(1, 0, 2), v[0])
    assert torch.equal(rk2.permute(1, 0, 2), rk[0])


def test_reference_own_code_agrees_with_the_oracle_when_present():
    """oracle/_ref (the reference's files, copied by oracle/build_ref.py) runs Memory._generate_slice +
    Memory.prefill_stage2 unmodified; the oracle port must give the same scores and winners."""
    from oracle import msa_oracle as O
    from oracle import ref_runner as R
    if not R.available():
        pytest.skip("oracle/_ref has not been built on this machine")
    g = torch.Generator().manual_seed(0)
    chunks = torch.randint(1, 9, (600,), generator=g).tolist()      # ~2,700 chunks: two slices of >= 1024
    c = sum(chunks)
    rk = torch.nn.functional.normalize(torch.randn(1, 8, c, 128, generator=g), dim=-1)
    q = torch.nn.functional.normalize(torch.randn(2, 8, 4, 16, 128, generator=g), dim=-1)
    mask = torch.ones(2, 16, dtype=torch.bool)
    mask[1, 9:] = False
    mem = R.make_reference_memory(rk, chunks, range(500, 500 + len(chunks)), 16, slice_chunks=1024)
    s, li, gi = R.reference_prefill_stage2(mem, q, mask)
    pool = torch.repeat_interleave(torch.arange(1, len(chunks) + 1), torch.tensor(chunks))
    s2, l2, g2 = O.prefill_stage2(q, mask, rk[0], pool, torch.tensor([0] + list(range(500, 500 + len(chunks)))), 16)
    assert len(mem.slice_desc) > 1
    assert torch.allclose(s, s2, atol=1e-6) and torch.equal(li, l2) and torch.equal(gi, g2)

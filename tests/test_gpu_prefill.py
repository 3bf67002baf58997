"""Stage-1 and stage-2 attention kernels against the reference layer's own outputs at head_dim 128
(tests/golden/layer_attn128.npz) and, on more shapes, against the oracle's fp32 restatements of
src/msa/memory_sparse_attention.py:216-241 and :282-357 (which tests/test_oracle_golden.py pins to the same fixture).
Tolerance: 1e-2 norm-wise for bf16 attention outputs and pooled tensors."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, b, s, hq, hkv, d, t_len, n_sel, valid_frac, dtype, dev):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(b, hq, s, d, generator=g).to(dtype)
    k = torch.randn(b, hkv, s, d, generator=g).to(dtype)
    v = torch.randn(b, hkv, s, d, generator=g).to(dtype)
    tk = torch.randn(1, hkv, t_len, d, generator=g).to(dtype)
    tv = torch.randn(1, hkv, t_len, d, generator=g).to(dtype)
    tot = int(sum(n_sel))
    sk = torch.randn(hkv, tot, d, generator=g).to(dtype)
    sv = torch.randn(hkv, tot, d, generator=g).to(dtype)
    valid = torch.rand(b, s, generator=g) < valid_frac
    valid[:, -1] = True                      # every sequence keeps at least its last token
    if b > 1:
        valid[1, : s // 2] = False           # a left-padded sequence
    return [x.to(dev) for x in (q, k, v, tk, tv, sk, sv, valid)]


def _reference(q, k, v, tk, tv, sk, sv, valid, n_sel, scale):
    """The oracle's stage-2 restatement (pinned to the reference layer by tests/test_oracle_golden.py), fp32 on the
    CPU.  Returns (out [B,S,Hq*D], list of per-sequence (K, V) contexts)."""
    from oracle import msa_oracle as O
    c = lambda t: t.cpu()
    out, ck, cv, lens = O.stage2_context_attention(c(q), c(k), c(v), c(tk), c(tv), c(sk), c(sv), c(valid), n_sel, scale)
    max_l = ck.shape[2]
    ctx = [(ck[i, :, max_l - int(lens[i]):].to(q.device), cv[i, :, max_l - int(lens[i]):].to(q.device))
           for i in range(q.shape[0])]
    return out.to(q.device), ctx


@pytest.mark.parametrize("b,s,hq,hkv,t_len,n_sel,frac", [
    (3, 70, 8, 2, 3, [130, 0, 61], 0.8),
    (2, 256, 32, 8, 3, [1024, 517], 1.0),
    (1, 1, 4, 4, 0, [5], 1.0),
    (4, 33, 16, 8, 3, [0, 0, 0, 0], 0.5),
])
def test_assemble_and_prefill_match_restatement(b, s, hq, hkv, t_len, n_sel, frac):
    from msa_b200 import ops
    dev = torch.device("cuda:0")
    d = 128
    q, k, v, tk, tv, sk, sv, valid = _case(11 + b, b, s, hq, hkv, d, t_len, n_sel, frac, torch.bfloat16, dev)
    nsel = torch.tensor(n_sel, dtype=torch.int64, device=dev)
    lens = [t_len + n_sel[i] + int(valid[i].sum()) for i in range(b)]
    max_kv, reserve = max(lens), 7
    ks, vs, kv_start, kv_len, q_tok, num_q, err = ops.assemble_context(tk, tv, sk, sv, nsel, k, v, valid, max_kv, reserve)
    scale = 1.0 / math.sqrt(d)
    out = ops.sparse_prefill_attn(q, ks, vs, kv_start, kv_len, q_tok, num_q, scale)
    torch.cuda.synchronize()
    ref, ctx = _reference(q, k, v, tk, tv, sk, sv, valid, n_sel, scale)
    assert int(err.item()) == 0
    assert kv_len.tolist() == lens
    assert kv_start.tolist() == [max_kv - x for x in lens]
    assert num_q.tolist() == [int(valid[i].sum()) for i in range(b)]
    for i in range(b):   # the compact cache is a copy: bit exact, left padding untouched (zero)
        assert torch.equal(ks[i, :, max_kv - lens[i]:max_kv], ctx[i][0])
        assert torch.equal(vs[i, :, max_kv - lens[i]:max_kv], ctx[i][1])
        assert ks[i, :, :max_kv - lens[i]].abs().sum().item() == 0
        assert ks[i, :, max_kv:].abs().sum().item() == 0
        idx = valid[i].nonzero().flatten()
        assert q_tok[i, :idx.numel()].tolist() == idx.tolist()
    # bf16 probabilities and outputs: 1e-2 of the output's norm
    errn = (out.float() - ref).norm() / ref.norm().clamp_min(1e-6)
    assert errn.item() < 1e-2, errn.item()
    assert out[~valid].abs().sum().item() == 0


@pytest.mark.parametrize("b,s,hq,hkv,t_len,n_sel,pad", [
    (3, 70, 8, 2, 3, [130, 0, 61], "left"),            # one row block, ragged contexts, a sequence without retrieved entries
    (2, 300, 32, 8, 3, [1024, 517], "left"),           # three row blocks of queries
    (4, 128, 16, 8, 3, [64, 0, 200, 1], "right"),      # right padding, queries ending inside a row block
    (3, 33, 8, 8, 0, [0, 5, 0], "none"),               # no template, contexts shorter than one key tile
])
def test_context_attention_on_tcgen05_kernel_matches_restatement(b, s, hq, hkv, t_len, n_sel, pad):
    """Stage-2 attention through the tcgen05 kernel's context mode (every sequence's valid tokens are one run) against
    the oracle's restatement and against the mma.sync kernel on the same store, token-major queries as the layer
    passes them; one sequence has no valid token at all."""
    from msa_b200 import ops
    dev = torch.device("cuda:0")
    d = 128
    q, k, v, tk, tv, sk, sv, _ = _case(300 + b, b, s, hq, hkv, d, t_len, n_sel, 1.0, torch.bfloat16, dev)
    q = q.transpose(1, 2).contiguous().transpose(1, 2)        # [B, Hq, S, D] view of token-major storage
    g = torch.Generator().manual_seed(5 + s)
    valid = torch.ones(b, s, dtype=torch.bool)
    for i in range(b):
        n = int(torch.randint(1, s + 1, (1,), generator=g)) if (pad != "none" and i > 0) else s
        if pad == "left":
            valid[i, : s - n] = False
        elif pad == "right":
            valid[i, n:] = False
    if b > 2:
        valid[2] = False                                       # nothing to attend for: its rows must come back zero
    valid = valid.to(dev)
    nsel = torch.tensor(n_sel, dtype=torch.int64, device=dev)
    lens = [t_len + n_sel[i] + int(valid[i].sum()) for i in range(b)]
    max_kv, reserve = max(lens), 9
    ks, vs, kv_start, kv_len, q_tok, num_q, err = ops.assemble_context(tk, tv, sk, sv, nsel, k, v, valid, max_kv, reserve)
    scale = 1.0 / math.sqrt(d)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    out = torch.full((b, s, hq * d), float("nan"), dtype=torch.bfloat16, device=dev)     # the kernel writes every row
    ops.sparse_prefill_attn(q, ks, vs, kv_start, kv_len, q_tok, num_q, scale, out=out, q_runs=True, status=status)
    legacy = ops.sparse_prefill_attn(q, ks, vs, kv_start, kv_len, q_tok, num_q, scale)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0] and int(err.item()) == 0
    ref, _ = _reference(q, k, v, tk, tv, sk, sv, valid, n_sel, scale)
    assert out[~valid].abs().sum().item() == 0
    errn = (out.float()[valid] - ref[valid]).norm() / ref[valid].norm().clamp_min(1e-6)
    assert errn.item() < 1e-2, errn.item()
    assert ((out.float() - legacy.float()).norm() / legacy.float().norm().clamp_min(1e-6)).item() < 1e-2


def test_context_attention_on_tcgen05_kernel_without_causal_mask():
    """A multi-token decode segment (every valid token sees the whole grown context) through the context mode: contexts
    that end inside a key tile, a segment longer than one row block."""
    from msa_b200 import ops
    from oracle import msa_oracle as O
    dev = torch.device("cuda:0")
    b, hq, hkv, d, l0, q_len, cap = 3, 8, 2, 128, 150, 200, 400
    g = torch.Generator().manual_seed(43)
    lens = torch.tensor([150, 97, 3])
    ck, cv = [torch.randn(b, hkv, l0, d, generator=g).to(torch.bfloat16) for _ in range(2)]
    key_mask = torch.arange(l0).unsqueeze(0) >= (l0 - lens.unsqueeze(1))
    q = torch.randn(b, hq, q_len, d, generator=g).to(torch.bfloat16)
    nk, nv = [torch.randn(b, hkv, q_len, d, generator=g).to(torch.bfloat16) for _ in range(2)]
    new_mask = torch.ones(b, q_len, dtype=torch.bool)
    new_mask[1, :77] = False                 # left padded
    new_mask[2, 5:] = False                  # right padded
    ref, _, _, _ = O.decode_segment_attention(q.float(), ck.float(), cv.float(), key_mask, nk.float(), nv.float(), new_mask)
    k_store = torch.zeros(b, hkv, cap, d, dtype=torch.bfloat16, device=dev)
    v_store = torch.zeros_like(k_store)
    k_store[:, :, :l0], v_store[:, :, :l0] = ck.to(dev), cv.to(dev)
    kv_start, kv_len = (l0 - lens).to(torch.int32).to(dev), lens.to(torch.int32).to(dev)
    q_tok, num_q, err = ops.append_segment(nk.to(dev), nv.to(dev), new_mask.to(dev), k_store, v_store, kv_start, kv_len)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    out = ops.sparse_prefill_attn(q.to(dev), k_store, v_store, kv_start, kv_len, q_tok, num_q, causal=False, q_runs=True,
                                  status=status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0] and int(err.item()) == 0
    got = out.float().cpu()
    assert ((got[new_mask] - ref[new_mask]).norm() / ref[new_mask].norm()).item() < 1e-2
    assert got[~new_mask].abs().sum().item() == 0


def test_run_check_that_picks_the_stage2_kernel():
    """MemorySparseAttention._valid_runs: 1 when every row's valid tokens are one run (left / right padding, empty rows),
    0 when a row has a hole; the second word is the status of the earlier tensor-core attention launches."""
    from types import SimpleNamespace
    from msa_b200.attention import MemorySparseAttention
    dev = torch.device("cuda:0")
    cache = SimpleNamespace(meta={})
    runs = torch.zeros(4, 12, dtype=torch.bool, device=dev)
    runs[0] = True
    runs[1, 5:] = True
    runs[2, :3] = True                      # row 3 stays empty
    assert MemorySparseAttention._valid_runs(None, runs, cache).tolist() == [1, 0]
    hole = runs.clone()
    hole[1, 8] = False
    assert MemorySparseAttention._valid_runs(None, hole, cache).tolist() == [0, 0]
    cache.meta["_msa_b200_attn_status"][0] = 6          # what a kernel that gave up leaves behind
    assert MemorySparseAttention._valid_runs(None, runs, cache).tolist() == [1, 6]
    with pytest.raises(Exception, match="bounded barrier wait"):
        MemorySparseAttention._check_attn_status(6)


def test_assemble_fp32_and_overflow_flag():
    from msa_b200 import ops
    dev = torch.device("cuda:0")
    b, s, hkv, d, t_len, n_sel = 2, 20, 2, 64, 3, [9, 4]
    q, k, v, tk, tv, sk, sv, valid = _case(5, b, s, 4, hkv, d, t_len, n_sel, 0.7, torch.float32, dev)
    nsel = torch.tensor(n_sel, dtype=torch.int64, device=dev)
    lens = [t_len + n_sel[i] + int(valid[i].sum()) for i in range(b)]
    ks, vs, kv_start, kv_len, q_tok, num_q, err = ops.assemble_context(tk, tv, sk, sv, nsel, k, v, valid, max(lens))
    _, ctx = _reference(q, k, v, tk, tv, sk, sv, valid, n_sel, 1.0)
    assert int(err.item()) == 0
    for i in range(b):
        assert torch.equal(ks[i, :, max(lens) - lens[i]:], ctx[i][0])
        assert torch.equal(vs[i, :, max(lens) - lens[i]:], ctx[i][1])
    # a cache that is too short: flagged, and the sequence that does not fit is left unwritten
    ks2, _, start2, _, _, _, err2 = ops.assemble_context(tk, tv, sk, sv, nsel, k, v, valid, min(lens))
    assert int(err2.item()) == 1
    long_one = lens.index(max(lens))
    if max(lens) > min(lens):
        assert start2[long_one].item() < 0 and ks2[long_one].abs().sum().item() == 0


@pytest.mark.parametrize("dtype,d,tol", [(torch.float32, 16, 1e-5), (torch.float32, 128, 1e-5), (torch.bfloat16, 64, 1e-2),
                                         (torch.float32, 200, 1e-5)])
@pytest.mark.parametrize("causal", [True, False])
def test_general_attention_kernel_in_store(dtype, d, tol, causal):
    """fp32 and head sizes other than 128 (the reference's CPU-runnable configuration among them): stage-2 attention
    on the general kernel, with and without the causal mask, against the oracle."""
    from msa_b200 import ops
    from oracle import msa_oracle as O
    dev = torch.device("cuda:0")
    b, s, hq, hkv, t_len, n_sel = 3, 37, 8, 2, 3, [11, 0, 40]
    q, k, v, tk, tv, sk, sv, valid = _case(23, b, s, hq, hkv, d, t_len, n_sel, 0.8, dtype, dev)
    nsel = torch.tensor(n_sel, dtype=torch.int64, device=dev)
    lens = [t_len + n_sel[i] + int(valid[i].sum()) for i in range(b)]
    ks, vs, kv_start, kv_len, q_tok, num_q, err = ops.assemble_context(tk, tv, sk, sv, nsel, k, v, valid, max(lens), 2)
    out = ops.sparse_prefill_attn(q, ks, vs, kv_start, kv_len, q_tok, num_q, causal=causal)
    torch.cuda.synchronize()
    if causal:
        ref, _ = _reference(q, k, v, tk, tv, sk, sv, valid, n_sel, d ** -0.5)
    else:   # every valid token sees its whole context
        ref = torch.zeros(b, s, hq * d)
        for i in range(b):
            idx = valid[i].nonzero().flatten().cpu()
            kk, vv = ks[i, :, max(lens) - lens[i]:max(lens)].cpu(), vs[i, :, max(lens) - lens[i]:max(lens)].cpu()
            full = O._causal_segment(q[i][:, idx].cpu(), kk, vv, d ** -0.5, lens[i])       # offset >= nk: no masking
            ref[i, idx] = full
        ref = ref.to(dev)
    errn = (out.float() - ref.float()).norm() / ref.float().norm()
    assert errn.item() < tol, errn.item()
    assert out[~valid].abs().sum().item() == 0


@pytest.mark.parametrize("dtype,d,tol", [(torch.float32, 16, 1e-5), (torch.bfloat16, 64, 1e-2), (torch.float32, 128, 1e-5)])
def test_general_attention_kernel_by_index(dtype, d, tol):
    """Stage-1 attention inside documents on the general kernel (masked tokens inside documents, two block rows)."""
    from msa_b200 import ops
    from oracle import msa_oracle as O
    dev = torch.device("cuda:0")
    hq, hkv, s = 4, 2, 90
    g = torch.Generator().manual_seed(31)
    doc_ids = torch.zeros(2, s, dtype=torch.long)
    doc_ids[0, :3] = -2
    doc_ids[0, 3:40], doc_ids[0, 40:41], doc_ids[0, 41:90] = 1, 2, 3
    doc_ids[1, 5:70], doc_ids[1, 70:88] = 1, 2
    mask = torch.ones(2, s, dtype=torch.long)
    mask[0, 10:13] = 0
    mask[1, 69] = 0
    q, k, v = [torch.randn(2, h, s, d, generator=g).to(dtype) for h in (hq, hkv, hkv)]
    ref = O.stage1_doc_attention(q, k, v, doc_ids, mask)
    tok, off, _ = ops.chunk_bookkeeping(doc_ids.to(dev), mask.to(dev), 8)
    flat = (doc_ids > 0) & (mask == 1)
    counts = torch.unique_consecutive((torch.arange(2).view(2, 1) * 10 + doc_ids)[flat], return_counts=True)[1]
    seg = torch.cat([torch.zeros(1, dtype=torch.long), counts.cumsum(0)]).to(torch.int32).to(dev)
    out, _, _ = ops.doc_attention_pool(q.to(dev), k.to(dev), v.to(dev), tok, seg, int(counts.max()))
    t_tok = torch.arange(3, dtype=torch.int32, device=dev)
    ops.doc_attention_pool(q.to(dev), k.to(dev), v.to(dev), t_tok, torch.tensor([0, 3], dtype=torch.int32, device=dev), 3, out=out)
    torch.cuda.synchronize()
    assert ((out.float().cpu() - ref).norm() / ref.norm()).item() < tol
    untouched = ~(flat | ((doc_ids == -2) & (mask == 1)))
    assert out.cpu()[untouched].abs().sum().item() == 0


def test_append_segment_and_noncausal_attention_bf16():
    """Multi-token decode segment on the tensor-core kernel: the segment's unmasked tokens are appended in place and
    every valid token attends to the whole grown context (oracle.decode_segment_attention)."""
    from msa_b200 import ops
    from oracle import msa_oracle as O
    dev = torch.device("cuda:0")
    b, hq, hkv, d, l0, q_len, cap = 3, 8, 2, 128, 150, 40, 230
    g = torch.Generator().manual_seed(41)
    lens = torch.tensor([150, 97, 3])
    ck, cv = [torch.randn(b, hkv, l0, d, generator=g).to(torch.bfloat16) for _ in range(2)]
    key_mask = torch.arange(l0).unsqueeze(0) >= (l0 - lens.unsqueeze(1))
    q = torch.randn(b, hq, q_len, d, generator=g).to(torch.bfloat16)
    nk, nv = [torch.randn(b, hkv, q_len, d, generator=g).to(torch.bfloat16) for _ in range(2)]
    new_mask = torch.rand(b, q_len, generator=g) < 0.7
    new_mask[2] = False
    new_mask[2, -1] = True
    ref, _, _, _ = O.decode_segment_attention(q.float(), ck.float(), cv.float(), key_mask, nk.float(), nv.float(), new_mask)
    k_store = torch.zeros(b, hkv, cap, d, dtype=torch.bfloat16, device=dev)
    v_store = torch.zeros_like(k_store)
    k_store[:, :, :l0], v_store[:, :, :l0] = ck.to(dev), cv.to(dev)
    kv_start, kv_len = (l0 - lens).to(torch.int32).to(dev), lens.to(torch.int32).to(dev)
    q_tok, num_q, err = ops.append_segment(nk.to(dev), nv.to(dev), new_mask.to(dev), k_store, v_store, kv_start, kv_len)
    out = ops.sparse_prefill_attn(q.to(dev), k_store, v_store, kv_start, kv_len, q_tok, num_q, causal=False)
    torch.cuda.synchronize()
    assert int(err.item()) == 0 and num_q.cpu().tolist() == new_mask.sum(1).tolist()
    assert kv_len.cpu().tolist() == (lens + new_mask.sum(1)).tolist()
    for i in range(b):      # appended in order, right behind the old entries
        idx = new_mask[i].nonzero().flatten()
        assert torch.equal(k_store[i, :, l0:l0 + len(idx)].cpu(), nk[i][:, idx])
        assert q_tok[i, :len(idx)].cpu().tolist() == idx.tolist()
    got = out.float().cpu()
    assert ((got[new_mask] - ref[new_mask]).norm() / ref[new_mask].norm()).item() < 1e-2
    assert got[~new_mask].abs().sum().item() == 0
    # no room: flagged, sequence untouched
    small = torch.zeros(b, hkv, l0 + 5, d, dtype=torch.bfloat16, device=dev)
    kv_len2 = lens.to(torch.int32).to(dev)
    _, num_q2, err2 = ops.append_segment(nk.to(dev), nv.to(dev), new_mask.to(dev), small, small.clone(), kv_start, kv_len2)
    assert int(err2.item()) == 1 and kv_len2.cpu().tolist()[0] == 150 and num_q2.cpu().tolist()[0] == 0


# ----------------------------------------------------------------------------------------------
# stage 1: attention inside every document with the K / V chunk means from the same pass
# (src/msa/memory_sparse_attention.py:216-241, :166-176)
# ----------------------------------------------------------------------------------------------
def _stage1_case(seed, doc_lens, n_template, hq, hkv, pad, drop):
    """One block row: [template | documents | padding]; `drop` masks a few tokens inside documents."""
    g = torch.Generator().manual_seed(seed)
    ids = [-2] * n_template
    for i, n in enumerate(doc_lens):
        ids += [i + 1] * n
    ids += [0] * pad
    s = len(ids)
    doc_ids = torch.tensor(ids).view(1, s)
    mask = torch.ones(1, s, dtype=torch.long)
    if pad:
        mask[0, -pad:] = 0
    for t in drop:
        mask[0, t] = 0
    q = torch.randn(1, hq, s, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(1, hkv, s, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(1, hkv, s, 128, generator=g).to(torch.bfloat16)
    return doc_ids, mask, q, k, v


def _segment_reference(q, k, v, tokens, scale):
    """fp32 causal attention of one segment (the oracle's routine); q [Hq,S,D], k/v [Hkv,S,D]; returns [n, Hq*D]."""
    from oracle import msa_oracle as O
    return O._causal_segment(q[:, tokens], k[:, tokens], v[:, tokens], scale, 0)


@pytest.mark.parametrize("doc_lens,drop_frac,layout", [
    ([300, 129, 700], 0.1, "token_major"),
    ([128, 513, 40, 260], 0.3, "head_major"),       # a short document between long ones, many holes
    ([1000], 0.02, "token_major"),
])
def test_doc_attention_tc_masked_matches_restatement(doc_lens, drop_frac, layout):
    """Documents with masked tokens inside on the tcgen05 kernel: spans of memory + bitmap of the tokens that take
    part, against the oracle's causal attention over each document's compacted token list and against the mma.sync
    kernel; rows of masked tokens keep what the output held."""
    from msa_b200 import ops
    dev = torch.device("cuda:0")
    hq, hkv, n_t = 8, 2, 3
    g = torch.Generator().manual_seed(len(doc_lens) * 7 + 1)
    total = sum(doc_lens)
    drop = [n_t + int(t) for t in torch.nonzero(torch.rand(total, generator=g) < drop_frac).flatten()]
    # the first and the last token of every document stay (a span is delimited by participating tokens)
    edges, pos = set(), n_t
    for n in doc_lens:
        edges.update((pos, pos + n - 1))
        pos += n
    drop = [t for t in drop if t not in edges]
    doc_ids, mask, q, k, v = _stage1_case(5, doc_lens, n_t, hq, hkv, pad=9, drop=drop)
    s = doc_ids.shape[1]
    if layout == "token_major":
        q, k, v = [x.transpose(1, 2).contiguous().transpose(1, 2) for x in (q, k, v)]
    valid = (doc_ids[0] > 0) & (mask[0] == 1)
    segs = [[t for t in range(s) if valid[t] and doc_ids[0, t] == i + 1] for i in range(len(doc_lens))]
    tok = torch.tensor([t for x in segs for t in x], dtype=torch.int32, device=dev)
    seg_off = torch.tensor([0] + [len(x) for x in segs]).cumsum(0).to(torch.int32).to(dev)
    span_tok, span_off, max_span = ops.document_spans(tok, seg_off)
    assert span_off.tolist() == [0] + torch.tensor(doc_lens).cumsum(0).tolist() and max_span == max(doc_lens)
    bits = ops.token_bitmap(valid.view(1, s).to(dev))
    scale = 128 ** -0.5
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    out = torch.full((1, s, hq * 128), 7.0, dtype=torch.bfloat16, device=dev)
    _, status = ops.doc_attention_tc_masked(qd, kd, vd, span_tok, span_off, max_span, bits, out=out, scale=scale)
    legacy, _, _ = ops.doc_attention_pool(qd, kd, vd, tok, seg_off, max(len(x) for x in segs), scale=scale)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    ref = torch.zeros(s, hq * 128)
    for x in segs:
        ref[x] = _segment_reference(q[0], k[0], v[0], x, scale)
    got = out[0].float().cpu()
    listed = valid.clone()
    assert (got[listed] - ref[listed]).norm() / ref[listed].norm() < 1e-2
    assert (got[listed] - legacy[0].float().cpu()[listed]).norm() / ref[listed].norm() < 1e-2
    assert bool((got[~listed] == 7.0).all())             # masked, template and padding rows: untouched


@pytest.mark.parametrize("doc_lens,drop,p", [
    ([512, 64, 1, 65, 130], [], 64),
    ([100, 300, 31], [5, 6, 150, 151, 152], 64),      # masked tokens inside documents
    ([200, 40], [], 32),
])
def test_doc_attention_pool_matches_restatement(doc_lens, drop, p):
    from msa_b200 import ops
    from oracle import msa_oracle as O
    dev = torch.device("cuda:0")
    hq, hkv, n_t = 8, 2, 3
    drop = [n_t + t for t in drop]
    doc_ids, mask, q, k, v = _stage1_case(3, doc_lens, n_t, hq, hkv, pad=9, drop=drop)
    s = doc_ids.shape[1]
    tok, off, pooled_ids = ops.chunk_bookkeeping(doc_ids.to(dev), mask.to(dev), p)
    valid = (doc_ids[0] > 0) & (mask[0] == 1)
    segs = [[t for t in range(s) if valid[t] and doc_ids[0, t] == i + 1] for i in range(len(doc_lens))]
    seg_off = torch.tensor([0] + [len(x) for x in segs]).cumsum(0).to(torch.int32).to(dev)
    assert tok.cpu().tolist() == [t for x in segs for t in x]
    scale = 128 ** -0.5
    out, pk, pv = ops.doc_attention_pool(q.to(dev), k.to(dev), v.to(dev), tok, seg_off, max(len(x) for x in segs),
                                         chunk_offsets=off, pool_size=p, scale=scale)
    # template segment through the same kernel, no pooling
    t_tok = torch.arange(n_t, dtype=torch.int32, device=dev)
    ops.doc_attention_pool(q.to(dev), k.to(dev), v.to(dev), t_tok, torch.tensor([0, n_t], dtype=torch.int32, device=dev),
                           n_t, out=out, scale=scale)
    torch.cuda.synchronize()
    ref = torch.zeros(s, hq * 128)
    for x in segs + [list(range(n_t))]:
        ref[x] = _segment_reference(q[0], k[0], v[0], x, scale)
    got = out[0].float().cpu()
    assert (got - ref).norm() / ref.norm() < 1e-2
    untouched = [t for t in range(n_t, s) if not valid[t]]
    assert got[untouched].abs().sum() == 0
    # pooled K / V: the oracle's exact chunk means (bf16 rounding: 1e-2), and the pooling kernel bit for bit
    # up to one rounding step of the fp32 sum order
    lens = (off[1:] - off[:-1]).cpu().long()
    flat = torch.tensor([t for x in segs for t in x])
    for pooled, states in ((pk, k), (pv, v)):
        exact = O.pool_chunks_exact(states[0][:, flat].permute(1, 0, 2).float(), lens).float()
        assert (pooled.float().cpu() - exact).norm() / exact.norm() < 1e-2
        alone = ops.pool_chunks(states.to(dev), off, tok)
        assert (pooled.float() - alone.float()).abs().max().item() <= 2 ** -7 * alone.float().abs().max().item()
        assert (pooled == alone).float().mean().item() > 0.99


def test_layer_bf16_on_own_kernels_matches_fp32_layer_on_library_path():
    """The layer mirror with head_dim 128: in bf16 stage 1 and stage 2 run on this package's attention kernels
    (fused K/V pooling, one-launch assembly), in fp32 on the library path.  Same weights, same inputs."""
    from transformers.models.qwen3.modeling_qwen3 import Qwen3RotaryEmbedding
    from msa_b200.attention import MemorySparseAttention
    from msa_b200.cache import SparseCache, SparseCacheOnCPU
    from msa_b200.configuration import MSAConfig
    from msa_b200.memory import AttentionGeometry, Document, ModelConfig
    from msa_b200.service import MSAService
    dev = "cuda:0"
    hq, hkv, d, pool, top_k = 8, 2, 128, 64, 3
    cfg = MSAConfig(
        msa_config=dict(router_layer_idx="0", aux_loss=False, aux_loss_method="INFONCE", decouple_router=True,
                        top_k_docs=top_k, pooling_kernel_size=pool, head_reduce_method="mean",
                        query_reduce_method="max", chunk_reduce_method="max", decouple_pooling_mode="mean"),
        hidden_size=256, num_attention_heads=hq, num_key_value_heads=hkv, head_dim=d, num_hidden_layers=1,
        intermediate_size=64, vocab_size=32, max_position_embeddings=1024)
    cfg._attn_implementation = "eager"
    torch.manual_seed(3)
    layer32 = MemorySparseAttention(cfg, 0).eval().to(dev)
    layer16 = MemorySparseAttention(cfg, 0).eval().to(dev)
    layer16.load_state_dict(layer32.state_dict())
    layer16.to(torch.bfloat16)
    rope = Qwen3RotaryEmbedding(cfg).to(dev)

    doc_lens = [130, 64, 77]
    doc_ids, mask, _, _, _ = _stage1_case(4, doc_lens, 3, hq, hkv, pad=0, drop=[])
    s = doc_ids.shape[1]
    g = torch.Generator().manual_seed(12)
    hidden = torch.randn(1, s, 256, generator=g).to(dev)
    pos = torch.cat([torch.arange(3)] + [torch.arange(n) for n in doc_lens]).view(1, s).to(dev)
    b2, s2 = 2, 12
    hidden2 = torch.randn(b2, s2, 256, generator=g).to(dev)
    ids2 = torch.zeros(b2, s2, dtype=torch.long, device=dev)
    mask2 = torch.ones(b2, s2, dtype=torch.long, device=dev)
    mask2[1, :5] = 0
    pos2 = (torch.arange(s2).view(1, s2) + 3 + top_k).expand(b2, s2).contiguous().to(dev)

    results = []
    for layer, dt in ((layer32, torch.float32), (layer16, torch.bfloat16)):
        cache1 = SparseCacheOnCPU()
        cache1.record_kwargs(0, {"stage": "prefill_stage1"})
        h = hidden.to(dt)
        with torch.no_grad():
            out1, _ = layer(h, doc_ids.to(dev), mask.to(dev), rope(h, pos), cache1)
        kw = cache1.cache_kwargs[0]
        pk, pv = cache1.get_kvcache(0)
        prk = cache1.get_router_kcache(0)
        chunks = torch.unique_consecutive(kw["pooled_doc_ids"], return_counts=True)[1].tolist()
        docs = [Document(doc_id=10 + i, num_chunks=n) for i, n in enumerate(chunks)]
        geo = AttentionGeometry(num_hidden_layers=1, num_attention_heads=hq, num_key_value_heads=hkv, head_dim=d, dtype=dt)
        svc = MSAService(0, None, ModelConfig(doc_top_k=top_k, pooling_kernel_size=pool, router_layer_idx="0"), None,
                         geo, world_size=1, rank=0)
        svc.generate_blocks(docs, metas=[{"past_key_values": cache1, "nr_docs": len(docs), "chunk_sizes": chunks,
                                          "doc_ids": [dd.doc_id for dd in docs], "nr_chunks": chunks}])
        svc.setup_memory_client(layer)
        cache2 = SparseCache()
        cache2.meta["max_generate_tokens"] = 4
        cache2.record_kwargs(0, {"stage": "prefill_stage2"})
        h2 = hidden2.to(dt)
        with torch.no_grad():
            out2, _ = layer(h2, ids2, mask2, rope(h2, pos2), cache2)
        svc.check_status()
        kw2 = cache2.cache_kwargs[0]
        results.append(dict(out1=out1.float().cpu(), pk=pk.float().cpu(), pv=pv.float().cpu(), prk=prk.float().cpu(),
                            out2=out2.float().cpu(), kv_lengths=kw2["kv_lengths"].cpu(),
                            ck=kw2["compacked_key_cache"].float().cpu(), cv=kw2["compacked_value_cache"].float().cpu(),
                            pad=kw2["attention_mask"].cpu()))
    a, b_ = results

    def rel(x, y):
        return float((x - y).norm() / y.norm().clamp_min(1e-9))
    assert rel(b_["out1"], a["out1"]) < 3e-2
    assert rel(b_["pk"], a["pk"]) < 2e-2 and rel(b_["pv"], a["pv"]) < 2e-2 and rel(b_["prk"], a["prk"]) < 2e-2
    assert torch.equal(a["kv_lengths"], b_["kv_lengths"]) and torch.equal(a["pad"], b_["pad"])   # every document selected
    assert rel(b_["ck"], a["ck"]) < 2e-2 and rel(b_["cv"], a["cv"]) < 2e-2
    valid = mask2.bool().cpu()
    assert rel(b_["out2"][valid], a["out2"][valid]) < 3e-2


@pytest.mark.parametrize("layout", ["token_major", "head_major"])
@pytest.mark.parametrize("doc_lens", [[100], [128, 64, 1, 65, 130, 512, 300], [700, 257]])
def test_doc_attention_tc_matches_restatement(doc_lens, layout):
    """The tcgen05 document attention kernel: single-tile and multi-tile documents, partial row blocks, neighbours
    whose rows fall into the same TMA boxes, both tensor layouts."""
    from msa_b200 import ops
    dev = torch.device("cuda:0")
    hq, hkv, n_t = 8, 2, 3
    doc_ids, mask, q, k, v = _stage1_case(7, doc_lens, n_t, hq, hkv, pad=5, drop=[])
    s = doc_ids.shape[1]
    if layout == "token_major":      # [B, S, H, D] storage viewed as [B, H, S, D], as the layer produces it
        q, k, v = [x.transpose(1, 2).contiguous().transpose(1, 2) for x in (q, k, v)]
    q, k, v = q.to(dev), k.to(dev), v.to(dev)
    tok, off, _ = ops.chunk_bookkeeping(doc_ids.to(dev), mask.to(dev), 64)
    bounds = [n_t]
    for n in doc_lens:
        bounds.append(bounds[-1] + n)
    seg_off = (torch.tensor(bounds) - n_t).to(torch.int32).to(dev)
    scale = 128 ** -0.5
    out, status = ops.doc_attention_tc(q, k, v, tok, seg_off, max(doc_lens), scale=scale)
    torch.cuda.synchronize()
    assert status.cpu().tolist()[0] == 0
    ref = torch.zeros(s, hq * 128)
    for i in range(len(doc_lens)):
        x = list(range(bounds[i], bounds[i + 1]))
        ref[x] = _segment_reference(q[0].cpu(), k[0].cpu(), v[0].cpu(), x, scale)
    got = out[0].float().cpu()
    assert (got - ref).norm() / ref.norm() < 1e-2
    worst = ((got - ref).norm(dim=1) / ref.norm(dim=1).clamp_min(1e-3)).max().item()
    assert worst < 3e-2, worst
    outside = [t for t in range(s) if t < n_t or t >= bounds[-1]]
    assert got[outside].abs().sum() == 0
    # and against the mma.sync kernel
    alt, _, _ = ops.doc_attention_pool(q, k, v, tok, seg_off, max(doc_lens), scale=scale)
    assert (got - alt[0].float().cpu()).norm() / ref.norm() < 1e-2


def test_doc_attention_kernels_with_several_block_rows():
    """Two block rows with different document layouts: the flat token positions carry the row, and both kernels
    must address q / k / v of the second row correctly (token-major tensors, as the layer produces them)."""
    from msa_b200 import ops
    dev = torch.device("cuda:0")
    hq, hkv, s = 8, 2, 400
    g = torch.Generator().manual_seed(21)
    doc_ids = torch.zeros(2, s, dtype=torch.long)
    rows = [[(0, 140), (140, 300), (300, 400)], [(10, 200), (200, 330)]]      # (start, end) of every document
    for r, docs in enumerate(rows):
        for i, (a, b) in enumerate(docs):
            doc_ids[r, a:b] = i + 1
    mask = torch.ones(2, s, dtype=torch.long)
    q, k, v = [torch.randn(2, s, h, 128, generator=g).to(torch.bfloat16).to(dev).transpose(1, 2) for h in (hq, hkv, hkv)]
    tok, off, _ = ops.chunk_bookkeeping(doc_ids.to(dev), mask.to(dev), 64)
    lens = [b - a for docs in rows for (a, b) in docs]
    seg_off = torch.tensor([0] + lens).cumsum(0).to(torch.int32).to(dev)
    scale = 128 ** -0.5
    out_tc, status = ops.doc_attention_tc(q, k, v, tok, seg_off, max(lens), scale=scale)
    out_mma, pk, pv = ops.doc_attention_pool(q, k, v, tok, seg_off, max(lens), chunk_offsets=off, pool_size=64, scale=scale)
    torch.cuda.synchronize()
    assert status.cpu().tolist()[0] == 0
    ref = torch.zeros(2, s, hq * 128)
    for r, docs in enumerate(rows):
        for (a, b) in docs:
            ref[r, a:b] = _segment_reference(q[r].cpu(), k[r].cpu(), v[r].cpu(), list(range(a, b)), scale)
    for out in (out_tc, out_mma):
        got = out.float().cpu()
        assert (got - ref).norm() / ref.norm() < 1e-2
        assert got[1, :10].abs().sum() == 0 and got[1, 330:].abs().sum() == 0
    # the fused K / V chunk means across both rows against the oracle's exact means
    from oracle import msa_oracle as O
    flat = tok.cpu().long()
    clen = (off[1:] - off[:-1]).cpu().long()
    for pooled, states in ((pk, k), (pv, v)):
        rows_ = states.cpu()[flat // s, :, flat % s]                       # [Td, Hkv, D]
        exact = O.pool_chunks_exact(rows_.float(), clen).float()
        assert (pooled.float().cpu() - exact).norm() / exact.norm() < 1e-2


# ----------------------------------------------------------------------------------------------
# the kernels against the REFERENCE layer's outputs (fixture made by tests/golden/make_golden.py)
# ----------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def attn128(golden):
    """The layer mirror in bf16 with the fixture's weights; a hook keeps what enters o_proj, and the kernel
    wrappers are counted so that every test can say which kernel produced its numbers."""
    from transformers.models.qwen3.modeling_qwen3 import Qwen3RotaryEmbedding
    from msa_b200 import ops
    from msa_b200.attention import MemorySparseAttention
    from msa_b200.configuration import MSAConfig
    from tests.util import attn128_case
    g = golden("layer_attn128")
    weights, geo = attn128_case(g)
    cfg = MSAConfig(
        msa_config=dict(router_layer_idx="0", aux_loss=False, aux_loss_method="INFONCE", decouple_router=True,
                        top_k_docs=geo["top_k"], pooling_kernel_size=geo["pool"], head_reduce_method="mean",
                        query_reduce_method="max", chunk_reduce_method="max", decouple_pooling_mode="mean"),
        hidden_size=geo["hidden"], num_attention_heads=geo["hq"], num_key_value_heads=geo["hkv"], head_dim=geo["d"],
        num_hidden_layers=1, intermediate_size=64, vocab_size=32, max_position_embeddings=1024)
    cfg._attn_implementation = "eager"
    layer = MemorySparseAttention(cfg, 0).eval()
    layer.load_state_dict(weights)
    layer.to(torch.bfloat16).to("cuda:0")
    rope = Qwen3RotaryEmbedding(cfg).to("cuda:0")
    pre, calls = {}, {}
    layer.o_proj.register_forward_pre_hook(lambda mod, args: pre.__setitem__("x", args[0].detach().float().cpu()))
    originals = {}
    for name in ("doc_attention_tc", "doc_attention_tc_masked", "doc_attention_pool", "sparse_prefill_attn", "assemble_context",
                 "pool_chunks"):
        originals[name] = getattr(ops, name)

        def counted(*a, _n=name, **kw):
            calls[_n] = calls.get(_n, 0) + 1
            calls[_n + ":kwargs"] = kw
            return originals[_n](*a, **kw)
        setattr(ops, name, counted)
    yield g, geo, layer, rope, pre, calls
    for name, fn in originals.items():
        setattr(ops, name, fn)


def _run_stage1(attn128, block):
    from msa_b200.cache import SparseCacheOnCPU
    from tests.util import T, from_bf16_bits
    g, geo, layer, rope, pre, calls = attn128
    calls.clear()
    hidden = from_bf16_bits(g[block + "_hidden_bits"]).to(torch.bfloat16).to("cuda:0")
    cache = SparseCacheOnCPU()
    cache.record_kwargs(0, {"stage": "prefill_stage1"})
    with torch.no_grad():
        layer(hidden, T(g[block + "_doc_ids"]).to("cuda:0"), T(g[block + "_attention_mask"]).to("cuda:0"),
              rope(hidden, T(g[block + "_position_ids"]).to("cuda:0")), cache)
    torch.cuda.synchronize()
    return cache, pre["x"]


def _rel(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm())


def test_stage1_unmasked_documents_on_tcgen05_kernel_match_reference_layer(attn128):
    from tests.util import T
    g, geo, layer, rope, pre, calls = attn128
    cache, attn = _run_stage1(attn128, "a")
    assert calls.get("doc_attention_tc") == 1            # documents: the tcgen05 kernel (the template: mma.sync)
    ref = T(g["a_attn"])
    assert _rel(attn, ref) < 1e-2
    pk, pv = cache.get_kvcache(0)
    assert _rel(pk.float().cpu(), T(g["a_pooled_k"])) < 1e-2 and _rel(pv.float().cpu(), T(g["a_pooled_v"])) < 1e-2
    assert _rel(cache.get_router_kcache(0).float().cpu(), T(g["a_pooled_rk"])) < 1e-2
    assert torch.equal(cache.cache_kwargs[0]["pooled_doc_ids"].cpu(), T(g["a_pooled_doc_ids"]))


def test_stage1_masked_documents_on_tcgen05_kernel_match_reference_layer(attn128):
    from tests.util import T
    g, geo, layer, rope, pre, calls = attn128
    cache, attn = _run_stage1(attn128, "b")
    # documents: the tcgen05 kernel over spans + bitmap; the template: mma.sync
    assert "doc_attention_tc" not in calls and calls.get("doc_attention_tc_masked") == 1 and calls.get("doc_attention_pool") == 1
    ref = T(g["b_attn"])
    assert _rel(attn, ref) < 1e-2
    masked = T(g["b_attention_mask"])[0] == 0
    assert float(attn[0][masked].abs().sum()) == 0
    pk, pv = cache.get_kvcache(0)
    assert _rel(pk.float().cpu(), T(g["b_pooled_k"])) < 1e-2 and _rel(pv.float().cpu(), T(g["b_pooled_v"])) < 1e-2
    assert _rel(cache.get_router_kcache(0).float().cpu(), T(g["b_pooled_rk"])) < 1e-2
    assert torch.equal(cache.cache_kwargs[0]["pooled_doc_ids"].cpu(), T(g["b_pooled_doc_ids"]))


def test_stage2_on_prefill_kernel_matches_reference_layer(attn128):
    from msa_b200.cache import SparseCache
    from msa_b200.memory import AttentionGeometry, Document, ModelConfig
    from msa_b200.service import MSAService
    from tests.util import T, from_bf16_bits
    g, geo, layer, rope, pre, calls = attn128
    cache1, _ = _run_stage1(attn128, "a")
    kw = cache1.cache_kwargs[0]
    chunks = torch.unique_consecutive(kw["pooled_doc_ids"], return_counts=True)[1].tolist()
    docs = [Document(doc_id=int(i), num_chunks=n) for i, n in zip(g["doc_global_ids"], chunks)]
    svc = MSAService(0, None, ModelConfig(doc_top_k=geo["top_k"], pooling_kernel_size=geo["pool"], router_layer_idx="0"),
                     None, AttentionGeometry(num_hidden_layers=1, num_attention_heads=geo["hq"],
                                             num_key_value_heads=geo["hkv"], head_dim=geo["d"], dtype=torch.bfloat16),
                     world_size=1, rank=0)
    svc.generate_blocks(docs, metas=[{"past_key_values": cache1, "nr_docs": len(docs), "chunk_sizes": chunks,
                                      "doc_ids": [d.doc_id for d in docs], "nr_chunks": chunks}])
    svc.setup_memory_client(layer)
    layer.template_prefix_kcache = layer.template_prefix_vcache = None
    calls.clear()
    cache2 = SparseCache()
    cache2.meta["require_recall_topk"] = True
    cache2.meta["max_generate_tokens"] = 4
    cache2.record_kwargs(0, {"stage": "prefill_stage2"})
    hidden2 = from_bf16_bits(g["s2_hidden_bits"]).to(torch.bfloat16).to("cuda:0")
    with torch.no_grad():
        layer(hidden2, T(g["s2_doc_ids"]).to("cuda:0"), T(g["s2_attention_mask"]).to("cuda:0"),
              rope(hidden2, T(g["s2_position_ids"]).to("cuda:0")), cache2)
    svc.check_status()
    assert calls.get("sparse_prefill_attn") == 1 and calls.get("assemble_context") == 1
    assert calls["sparse_prefill_attn:kwargs"].get("q_runs") is True       # left-padded questions: the tcgen05 kernel
    kw2 = cache2.cache_kwargs[0]
    assert [r["topk_doc_ids"] for r in kw2["recall_topk"]] == g["s2_recall_ids"].tolist()
    got_scores = torch.tensor([r["score"] for r in kw2["recall_topk"]])
    assert torch.allclose(got_scores, T(g["s2_recall_scores"]).float(), atol=1e-3)
    assert torch.equal(kw2["kv_lengths"].cpu(), T(g["s2_kv_lengths"]))
    assert torch.equal(kw2["attention_mask"].cpu(), T(g["s2_mask"]))
    assert _rel(kw2["compacked_key_cache"].float().cpu(), T(g["s2_cache_k"])) < 1e-2
    assert _rel(kw2["compacked_value_cache"].float().cpu(), T(g["s2_cache_v"])) < 1e-2
    valid = T(g["s2_attention_mask"]).bool()
    ref = T(g["s2_attn"])
    assert _rel(pre["x"][valid], ref[valid]) < 1e-2
    layer.set_memory_client(None)

"""Stage-2 context assembly and sparse prefill attention kernels against a torch fp32 restatement of
src/msa/memory_sparse_attention.py:282-357 ([template | retrieved | valid query tokens] per sequence,
bottom-right aligned causal attention, left-padded compact cache)."""
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
    """fp32, one sequence at a time.  Returns (out [B,S,Hq*D], list of per-sequence (K, V) contexts)."""
    b, hq, s, d = q.shape
    hkv = k.shape[1]
    grp = hq // hkv
    out = torch.zeros(b, s, hq * d, dtype=torch.float32, device=q.device)
    ctx = []
    off = 0
    for i in range(b):
        idx = valid[i].nonzero().flatten()
        kk = torch.cat([tk[0], sk[:, off:off + n_sel[i]], k[i][:, idx]], dim=1)
        vv = torch.cat([tv[0], sv[:, off:off + n_sel[i]], v[i][:, idx]], dim=1)
        off += n_sel[i]
        ctx.append((kk, vv))
        nq, nk = idx.numel(), kk.shape[1]
        qq = q[i][:, idx].float()                                        # [Hq, nq, D]
        kf = kk.float().repeat_interleave(grp, dim=0)
        vf = vv.float().repeat_interleave(grp, dim=0)
        att = torch.einsum("hqd,hkd->hqk", qq, kf) * scale
        pos_q = torch.arange(nq, device=q.device)[:, None] + (nk - nq)
        att = att.masked_fill(torch.arange(nk, device=q.device)[None, :] > pos_q, float("-inf"))
        o = torch.einsum("hqk,hkd->hqd", att.softmax(-1), vf)            # [Hq, nq, D]
        out[i, idx] = o.permute(1, 0, 2).reshape(nq, hq * d)
    return out, ctx


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


def test_prefill_rejects_other_shapes():
    from msa_b200 import ops
    from msa_b200._cabi import MsaError
    dev = torch.device("cuda:0")
    q = torch.zeros(1, 4, 8, 64, dtype=torch.bfloat16, device=dev)
    ks = torch.zeros(1, 2, 16, 64, dtype=torch.bfloat16, device=dev)
    z = torch.zeros(1, dtype=torch.int32, device=dev)
    qt = torch.zeros(1, 8, dtype=torch.int32, device=dev)
    with pytest.raises(MsaError):
        ops.sparse_prefill_attn(q, ks, ks, z, z, qt, z)

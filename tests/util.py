"""Helpers shared by the tests: seeded synthetic banks and tolerance-aware comparisons."""
import numpy as np
import torch


def T(x):
    return torch.from_numpy(np.asarray(x))


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """Norm-wise relative error ||a - b|| / ||b|| in fp64."""
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def ragged_docs(n_docs, lo, hi, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi + 1, (n_docs,), generator=g).tolist()


def make_bank(chunks_per_doc, hkv=8, d=128, dtype=torch.float32, seed=0, doc_mean_std=0.5, normalize=True):
    """Pooled router keys [C, Hkv, D] drawn per document as mean + noise (the distribution of
    benchmark config 3), plus the 1-based chunk->doc table."""
    g = torch.Generator().manual_seed(seed)
    n_docs = len(chunks_per_doc)
    lens = torch.tensor(chunks_per_doc)
    mu = torch.randn(n_docs, hkv, d, generator=g) * doc_mean_std
    c = int(lens.sum())
    rk = torch.repeat_interleave(mu, lens, dim=0) + torch.randn(c, hkv, d, generator=g) / 8.0
    if normalize:
        rk = torch.nn.functional.normalize(rk, dim=-1)
    pool_ids = torch.repeat_interleave(torch.arange(1, n_docs + 1), lens)
    return rk.to(dtype), pool_ids


def check_topk(table: torch.Tensor, scores: torch.Tensor, ids: torch.Tensor, k: int, tol: float):
    """Tie-aware top-k check of (scores, ids) against an oracle score table [B, N+1].

    * returned scores are sorted descending and equal table[b, id] within tol;
    * ids are distinct;
    * every column whose oracle score beats the oracle's k-th score by more than tol is present;
    * every returned column's oracle score is within tol of the oracle's k-th score or above it.
    """
    table = table.float().cpu()
    scores, ids = scores.float().cpu(), ids.cpu()
    b, n = table.shape
    k_eff = min(k, n)
    assert scores.shape == (b, k_eff) and ids.shape == (b, k_eff)
    ref_sorted = table.sort(dim=1, descending=True).values
    kth = ref_sorted[:, k_eff - 1]
    for i in range(b):
        s, d = scores[i], ids[i]
        finite = torch.isfinite(s) & (s > -1e30)
        assert (s[:-1] >= s[1:]).all(), "scores not sorted"
        assert len(set(d.tolist())) == k_eff, "duplicate ids"
        got = table[i, d]
        assert torch.allclose(got[finite], s[finite], atol=tol, rtol=0), (got, s)
        must = set(torch.nonzero(table[i] > kth[i] + tol).flatten().tolist())
        assert must <= set(d.tolist()), f"row {i}: missing clear winners {must - set(d.tolist())}"
        assert (got >= kth[i] - tol).all() or not finite.all(), f"row {i}: selected a clear loser"
        assert torch.allclose(s[finite], ref_sorted[i, :k_eff][finite], atol=tol, rtol=0)


def from_bf16_bits(x) -> torch.Tensor:
    """fp32 tensor from bf16 bit patterns stored as uint16 (how the fixtures keep bf16-representable values)."""
    return torch.from_numpy(np.asarray(x).view(np.int16).copy()).view(torch.bfloat16).to(torch.float32)


def attn128_case(g):
    """Weights (fp32, bf16-representable) and geometry of tests/golden/layer_attn128.npz."""
    weights = {k[len("wbits__"):]: from_bf16_bits(v) for k, v in g.items() if k.startswith("wbits__")}
    geo = dict(hq=int(g["hq"]), hkv=int(g["hkv"]), d=int(g["d"]), top_k=int(g["top_k"]), pool=int(g["pooling_kernel_size"]),
               hidden=int(g["hidden_size"]), theta=float(g["rope_theta"]))
    return weights, geo

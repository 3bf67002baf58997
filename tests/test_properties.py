"""Property tests (hypothesis) of the host-side logic and of the oracle's bookkeeping.  CPU only."""
import torch
from hypothesis import given, settings, strategies as st

from msa_b200.memory import Document
from msa_b200 import ops
from msa_b200.service import balanced_bucket_partition, build_directory
from oracle import msa_oracle as O

doc_lens = st.lists(st.integers(min_value=1, max_value=40), min_size=1, max_size=30)


@settings(max_examples=60, deadline=None)
@given(doc_lens, st.integers(min_value=1, max_value=8))
def test_partition_assigns_every_document_once_and_balances(lens, n_buckets):
    docs = [Document(doc_id=i, num_chunks=n) for i, n in enumerate(lens)]
    buckets = balanced_bucket_partition(docs, n_buckets)
    assert sorted(d.doc_id for b in buckets for d in b) == list(range(len(lens)))
    loads = [sum(d.num_chunks for d in b) for b in buckets]
    assert max(loads) - min(loads) <= max(lens)          # greedy least-loaded bound


@settings(max_examples=60, deadline=None)
@given(st.lists(doc_lens, min_size=1, max_size=4))
def test_directory_offsets_are_prefix_sums_per_shard(per_rank):
    base, offs, lens = build_directory([[0] + l for l in per_rank])
    for r, l in enumerate(per_rank):
        b = int(base[r])
        assert lens[b:b + len(l) + 1].tolist() == [0] + l
        run = 0
        for i, n in enumerate([0] + l):
            assert int(offs[b + i]) == run
            run += n


@settings(max_examples=40, deadline=None)
@given(doc_lens, st.integers(min_value=1, max_value=16))
def test_oracle_bookkeeping_matches_a_plain_loop(lens, p):
    ids = [-2, -2, -2]
    for i, n in enumerate(lens):
        ids += [i + 1] * n
    doc_ids = torch.tensor([ids])
    _, _, pooled, chunk_lengths = O.chunk_bookkeeping(doc_ids, torch.ones_like(doc_ids), p)
    want_len, want_doc = [], []
    for i, n in enumerate(lens):
        full, rest = divmod(n, p)
        want_len += [p] * full + ([rest] if rest else [])
        want_doc += [i + 1] * (full + (1 if rest else 0))
    assert chunk_lengths.tolist() == want_len and pooled.tolist() == want_doc


@settings(max_examples=40, deadline=None)
@given(st.lists(st.floats(width=32, allow_nan=False), min_size=1, max_size=12))
def test_candidate_buffer_is_lossless(vals):
    s = torch.tensor([vals], dtype=torch.float32)
    l = torch.arange(len(vals)).view(1, -1)
    buf, sv, lv, gv = ops.candidate_buffer(1, len(vals), "cpu")
    sv.copy_(s); lv.copy_(l); gv.copy_(l + 7)
    s2, l2, g2 = ops.candidate_views(torch.stack([buf, buf.clone()]))
    for w in range(2):
        assert torch.equal(s2[w].contiguous().view(torch.int32), s.view(torch.int32))
        assert torch.equal(l2[w], l) and torch.equal(g2[w], l + 7)

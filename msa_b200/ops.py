"""Functional wrappers: torch tensors in, torch tensors out, one C-ABI call each.

These are what ``memory.py``, ``service.py`` and ``attention.py`` (the mirrors of the
reference's ``Memory``, ``MSAService`` and ``MemorySparseAttention``) are built from.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from . import _cabi as A


# ---------------------------------------------------------------------------------------
# Stage 1
# ---------------------------------------------------------------------------------------

def chunk_bookkeeping(doc_ids: torch.Tensor, attention_mask: Optional[torch.Tensor], pooling_kernel_size: int,
                      max_chunks: Optional[int] = None):
    """Device version of src/msa/memory_sparse_attention.py:138-163.

    doc_ids ``[B, T]`` int64 (CUDA).  Returns ``(token_index[Td] int32, chunk_offsets[C+1] int32,
    pooled_doc_ids[C] int64)``.  Reads two integers back from the device to size the results
    (the reference synchronises at the same spot through ``.item()``).
    """
    A.need_cuda(doc_ids, attention_mask)
    doc_ids = doc_ids.contiguous()
    if doc_ids.dtype != torch.int64:
        raise A.MsaError("doc_ids must be int64")
    if attention_mask is not None:
        attention_mask = attention_mask.to(torch.int64).contiguous()
    rows, row_len = doc_ids.shape
    n = rows * row_len
    if max_chunks is None:
        # every document adds at most one partial chunk; a document has at least one token
        max_chunks = n // pooling_kernel_size + min(n, int(doc_ids.max().item()) * rows if n else 0) + 1
    dev = doc_ids.device
    token_index = torch.empty(max(n, 1), dtype=torch.int32, device=dev)
    chunk_offsets = torch.empty(max_chunks + 1, dtype=torch.int32, device=dev)
    pooled = torch.empty(max(max_chunks, 1), dtype=torch.int64, device=dev)
    counts = torch.zeros(4, dtype=torch.int32, device=dev)
    ws_bytes = int(A.lib().msa_bookkeeping_workspace_bytes(rows, row_len))
    workspace = torch.empty((ws_bytes + 7) // 8, dtype=torch.int64, device=dev)
    A.check(A.lib().msa_chunk_bookkeeping(A.ptr(doc_ids), A.ptr(attention_mask), rows, row_len, pooling_kernel_size,
                                          A.ptr(token_index), A.ptr(chunk_offsets), A.ptr(pooled), max_chunks,
                                          A.ptr(counts), A.ptr(workspace), workspace.numel() * 8, A.stream_ptr(dev)),
            "msa_chunk_bookkeeping")
    n_tok, n_chunks, overflow, _ = counts.tolist()
    if overflow:
        raise A.MsaError(f"chunk_bookkeeping: more than max_chunks={max_chunks} chunks")
    return token_index[:n_tok], chunk_offsets[: n_chunks + 1], pooled[:n_chunks]


def pool_chunks(states: torch.Tensor, chunk_offsets: torch.Tensor, token_index: Optional[torch.Tensor] = None,
                l2_normalize: bool = False, head_major_out: bool = False) -> torch.Tensor:
    """Chunk mean of ``states``.

    ``states`` is ``[1, H, T, D]`` (the layer's key/value states, head major) or ``[T, H, D]``.
    Returns ``[C, H, D]`` (chunk major, the bank's layout) or, with ``head_major_out``,
    ``[1, H, C, D]`` as the reference stores it (src/msa/memory_sparse_attention.py:173-174).
    """
    A.need_cuda(states, chunk_offsets, token_index)
    if states.dim() == 4:
        if states.shape[0] != 1:
            raise A.MsaError("pool_chunks: a [B, H, T, D] input needs B == 1 (call it per row)")
        _, h, t, d = states.shape
        vec = 16 // states.element_size()
        # any [1, H, T, D] view with a contiguous feature axis and 16-byte aligned rows is read in place (the layer's
        # projections are token major: heads side by side in a token's row); only other layouts are copied
        if not (states.stride(3) == 1 and states.stride(1) % vec == 0 and states.stride(2) % vec == 0
                and states.data_ptr() % 16 == 0):
            states = states.contiguous()
        tok_stride, head_stride = states.stride(2), states.stride(1)
    elif states.dim() == 3:
        t, h, d = states.shape
        states = states.contiguous()
        tok_stride, head_stride = h * d, d
    else:
        raise A.MsaError("pool_chunks: states must be [1, H, T, D] or [T, H, D]")
    c = chunk_offsets.numel() - 1
    dev = states.device
    if head_major_out:
        out = torch.empty((1, h, c, d), dtype=states.dtype, device=dev)
        oc, oh = d, c * d
    else:
        out = torch.empty((c, h, d), dtype=states.dtype, device=dev)
        oc, oh = h * d, d
    if c > 0:
        A.check(A.lib().msa_pool_chunks(A.ptr(states), A.dtype_code(states.dtype), tok_stride, head_stride,
                                        A.ptr(token_index), A.ptr(chunk_offsets.contiguous()), None, c, h, d,
                                        A.ptr(out), oc, oh, int(l2_normalize), A.stream_ptr(dev)), "msa_pool_chunks")
    return out


# ---------------------------------------------------------------------------------------
# Routing
# ---------------------------------------------------------------------------------------

def route_s_pad(seq_len: int, query_reduce: str = "max") -> int:
    return int(A.lib().msa_route_s_pad(seq_len, A.QREDUCE[query_reduce]))


def fold_queries(q: torch.Tensor, query_mask: torch.Tensor, num_kv_groups: int, l2_normalize: bool = False,
                 query_reduce: str = "max", s_pad: Optional[int] = None):
    """q ``[B, Hq, S, D]`` (any strides with D contiguous), query_mask ``[B, S]`` bool.
    Returns ``(q_folded[B*s_pad, Hkv*D], row_bias[B*s_pad] f32, s_pad)``."""
    A.need_cuda(q, query_mask)
    b, hq, s, d = q.shape
    if q.stride(3) != 1:
        q = q.contiguous()
    mask = query_mask.reshape(b, s).to(torch.uint8).contiguous()
    if s_pad is None:
        s_pad = route_s_pad(s, query_reduce)
    hkv = hq // num_kv_groups
    dev = q.device
    qf = torch.empty((b * s_pad, hkv * d), dtype=q.dtype, device=dev)
    bias = torch.empty((b * s_pad,), dtype=torch.float32, device=dev)
    A.check(A.lib().msa_fold_queries(A.ptr(q), A.dtype_code(q.dtype), q.stride(0), q.stride(1), q.stride(2),
                                     A.ptr(mask), s, b, hq, num_kv_groups, s, d, int(l2_normalize),
                                     A.QREDUCE[query_reduce], s_pad, A.ptr(qf), A.ptr(bias), A.stream_ptr(dev)),
            "msa_fold_queries")
    return qf, bias, s_pad


def block_router_keys(rk: torch.Tensor, blocked: Optional[torch.Tensor] = None, first_chunk: int = 0,
                      n_chunks_total: Optional[int] = None) -> torch.Tensor:
    """Row-major router keys ``[n, Hkv*D]`` / ``[n, Hkv, D]`` (bf16) into the tile-blocked layout
    ``[tiles, kdim/64, 128, 64]`` that the bandwidth-bound routing reads ~19 % faster (see ``msa_router_keys_block``).
    With ``blocked`` given, the rows are written as chunks ``first_chunk ..`` of that storage (bank ingestion block by
    block); otherwise storage for ``n_chunks_total`` (default: ``first_chunk + n``) chunks is allocated, zeroed."""
    A.need_cuda(rk, blocked)
    if rk.dtype != torch.bfloat16:
        raise A.MsaError("block_router_keys: bf16 keys only (fp32 banks stay row major)")
    n = rk.shape[0]
    rk2 = rk.reshape(n, -1) if rk.is_contiguous() else rk.flatten(1)
    if n > 0 and rk2.stride(1) != 1:
        rk2 = rk2.contiguous()
    kdim = rk2.shape[1]
    if kdim % 64 != 0:
        raise A.MsaError("block_router_keys: the key width must be a multiple of 64")
    if blocked is None:
        total = first_chunk + n if n_chunks_total is None else n_chunks_total
        blocked = torch.zeros(((total + 127) // 128, kdim // 64, 128, 64), dtype=rk.dtype, device=rk.device)
    elif blocked.dtype != rk.dtype or not blocked.is_contiguous() or tuple(blocked.shape[1:]) != (kdim // 64, 128, 64) or \
            first_chunk + n > blocked.shape[0] * 128:
        raise A.MsaError("block_router_keys: blocked storage must be contiguous [tiles, kdim/64, 128, 64] with room for the rows")
    A.check(A.lib().msa_router_keys_block(A.ptr(rk2), rk2.stride(0) if n > 0 else kdim, first_chunk, n, kdim, A.ptr(blocked),
                                          A.stream_ptr(rk.device)), "msa_router_keys_block")
    return blocked


def unblock_router_keys(blocked: torch.Tensor, n_chunks: int) -> torch.Tensor:
    """The row-major ``[n_chunks, kdim]`` copy of tile-blocked keys (for inspection and tests)."""
    t, kb, r, c = blocked.shape
    return blocked.permute(0, 2, 1, 3).reshape(t * r, kb * c)[:n_chunks].contiguous()


def route_scores(q_folded: torch.Tensor, row_bias: torch.Tensor, n_seq: int, s_pad: int, rk: torch.Tensor,
                 chunk_doc: torch.Tensor, n_docs: int, alpha: float, min_val: Optional[float] = None,
                 keys: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None, flags: int = 0,
                 blocked: bool = False):
    """Score table as order-preserving keys: int32 storage ``[n_seq, n_docs + 1]``.
    rk ``[C, Hkv*D]`` or ``[C, Hkv, D]`` (chunk major; the chunk stride may exceed the row), or, with ``blocked``,
    the tile-blocked storage of ``block_router_keys`` (the chunk count is then ``chunk_doc.numel()``)."""
    A.need_cuda(q_folded, row_bias, rk, chunk_doc)
    dev = rk.device
    if blocked:
        if rk.dim() != 4 or not rk.is_contiguous() or tuple(rk.shape[2:]) != (128, 64):
            raise A.MsaError("route_scores: blocked keys must be contiguous [tiles, kdim/64, 128, 64]")
        c, kdim = chunk_doc.numel(), rk.shape[1] * 64
        if c > rk.shape[0] * 128:
            raise A.MsaError("route_scores: chunk_doc lists more chunks than the blocked storage holds")
        rk2 = rk.view(-1, kdim)
        flags |= A.ROUTE_KEYS_BLOCKED
    else:
        c = rk.shape[0]
        kdim = 1
        for n in rk.shape[1:]:
            kdim *= n
        rk2 = rk.reshape(c, kdim) if rk.is_contiguous() else rk.flatten(1)
    if c > 0 and rk2.stride(1) != 1:
        raise A.MsaError("route_scores: router keys must have a contiguous feature axis")
    if chunk_doc.dtype != torch.int32:
        raise A.MsaError("route_scores: chunk_doc must be int32")
    if min_val is None:
        min_val = torch.finfo(rk.dtype).min
    if keys is None:
        keys = torch.empty((n_seq, n_docs + 1), dtype=torch.int32, device=dev)
    if status is None:
        status = torch.zeros(4, dtype=torch.int32, device=dev)
    A.check(A.lib().msa_route_scores(A.ptr(q_folded), A.ptr(row_bias), A.dtype_code(rk.dtype), n_seq, s_pad,
                                     A.ptr(rk2), rk2.stride(0) if c > 0 else kdim, c, kdim, A.ptr(chunk_doc),
                                     float(alpha), A.ptr(keys), keys.stride(0), n_docs, float(min_val), flags,
                                     A.ptr(status), A.stream_ptr(dev)), "msa_route_scores")
    return keys, status


def route_chunk_scores(q: torch.Tensor, query_mask: torch.Tensor, num_kv_groups: int, rk: torch.Tensor,
                       head_reduce: str = "max", query_reduce: str = "max", scale: float = 1.0,
                       min_val: Optional[float] = None, chunk_keys: Optional[torch.Tensor] = None):
    """Per-(sequence, chunk) scores for the reduce modes that cannot fold the heads (head_reduce "max";
    src/msa_service.py:740-780).  q ``[B, Hq, S, D]`` UNFOLDED, query_mask ``[B, S]``, rk ``[C, Hkv, D]`` chunk major.
    Returns keys ``[B, C + 1]`` (int32 storage), chunk c in column c + 1."""
    A.need_cuda(q, query_mask, rk, chunk_keys)
    b, hq, s, d = q.shape
    if q.stride(3) != 1:
        q = q.contiguous()
    c = rk.shape[0]
    rk2 = rk.reshape(c, -1) if rk.is_contiguous() else rk.flatten(1)
    if rk2.dtype != q.dtype:
        raise A.MsaError("route_chunk_scores: queries and router keys must share a dtype")
    mask = query_mask.reshape(b, s).to(torch.uint8).contiguous()
    if min_val is None:
        min_val = torch.finfo(rk.dtype).min
    if chunk_keys is None:
        chunk_keys = torch.empty((b, c + 1), dtype=torch.int32, device=q.device)
    A.check(A.lib().msa_route_chunk_scores(A.ptr(q), A.dtype_code(q.dtype), q.stride(0), q.stride(1), q.stride(2),
                                           A.ptr(mask), s, b, hq, num_kv_groups, s, d, A.HREDUCE[head_reduce],
                                           A.QREDUCE[query_reduce], A.ptr(rk2), rk2.stride(0) if c > 0 else hq * d, c,
                                           float(scale), float(min_val), A.ptr(chunk_keys), chunk_keys.stride(0),
                                           A.stream_ptr(q.device)), "msa_route_chunk_scores")
    return chunk_keys


def route_reduce_chunks(chunk_keys: torch.Tensor, chunk_doc: torch.Tensor, n_docs: int, chunk_reduce: str,
                        min_val: float, keys: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None):
    """Chunk -> document reduction ("max" or "mean", src/msa_service.py:787-812) of a chunk key table
    ``[B, C + 1]`` into a document key table ``[B, n_docs + 1]`` (allocated and reset here when not given)."""
    A.need_cuda(chunk_keys, chunk_doc, keys, status)
    if chunk_doc.dtype != torch.int32:
        raise A.MsaError("route_reduce_chunks: chunk_doc must be int32")
    n_seq, c = chunk_keys.shape[0], chunk_doc.numel()
    if keys is None:
        keys = torch.empty((n_seq, n_docs + 1), dtype=torch.int32, device=chunk_keys.device)
        route_table_reset(keys, n_docs, min_val)
    A.check(A.lib().msa_route_reduce_chunks(A.ptr(chunk_keys), chunk_keys.stride(0), n_seq, c, A.ptr(chunk_doc), n_docs,
                                            A.CREDUCE[chunk_reduce], float(min_val), A.ptr(keys), keys.stride(0),
                                            A.ptr(status), A.stream_ptr(chunk_keys.device)), "msa_route_reduce_chunks")
    return keys


ROUTE_SELECT_MAX_SEQ, ROUTE_SELECT_MAX_K = 128, 32


def route_score_select_supported(rk: torch.Tensor, n_seq: int, s_pad: int, top_k: int, blocked: bool = False) -> bool:
    """Whether ``route_score_select`` takes this shape (bf16 keys, one row per sequence, small batch and k)."""
    kdim = (rk.shape[1] * 64 if blocked else rk[0].numel()) if rk.shape[0] else 0
    return (rk.dtype == torch.bfloat16 and s_pad == 1 and 1 <= n_seq <= ROUTE_SELECT_MAX_SEQ and top_k <= ROUTE_SELECT_MAX_K
            and rk.shape[0] > 0 and kdim > 0 and kdim % 64 == 0)


def route_score_select(q_folded: torch.Tensor, row_bias: torch.Tensor, n_seq: int, rk: torch.Tensor,
                       chunk_doc: torch.Tensor, n_docs: int, alpha: float, top_k: int,
                       doc_ids_table: Optional[torch.Tensor] = None, min_val: Optional[float] = None,
                       status: Optional[torch.Tensor] = None, workspace: Optional[torch.Tensor] = None, out=None,
                       blocked: bool = False):
    """Decode-time routing in one call: scores ``n_seq`` single-row queries against the shard and selects the best
    ``top_k`` documents of each, without a score table (see ``msa_route_score_select``).  Same results, ties included,
    as ``route_scores`` + ``topk_select``.  ``rk`` as in ``route_scores`` (row major, or tile-blocked with ``blocked``).
    Returns ``(scores f32, local_ids i64, global_ids i64)``, ``[n_seq, k_eff]``."""
    A.need_cuda(q_folded, row_bias, rk, chunk_doc, doc_ids_table, status, workspace)
    dev = rk.device
    if chunk_doc.dtype != torch.int32:
        raise A.MsaError("route_score_select: chunk_doc must be int32")
    if blocked:
        if rk.dim() != 4 or not rk.is_contiguous() or tuple(rk.shape[2:]) != (128, 64):
            raise A.MsaError("route_score_select: blocked keys must be contiguous [tiles, kdim/64, 128, 64]")
        c, kdim, stride, rk2 = chunk_doc.numel(), rk.shape[1] * 64, rk.shape[1] * 64, rk
        if c > rk.shape[0] * 128:
            raise A.MsaError("route_score_select: chunk_doc lists more chunks than the blocked storage holds")
    else:
        c = rk.shape[0]
        rk2 = rk.reshape(c, -1) if rk.is_contiguous() else rk.flatten(1)
        kdim, stride = rk2.shape[1], rk2.stride(0)
        if chunk_doc.numel() != c:
            raise A.MsaError("route_score_select: one chunk_doc entry per key row")
    k_eff = min(top_k, n_docs + 1)
    if out is not None:
        scores, local, glob = out
    else:
        scores = torch.empty((n_seq, k_eff), dtype=torch.float32, device=dev)
        local = torch.empty((n_seq, k_eff), dtype=torch.int64, device=dev)
        glob = torch.empty((n_seq, k_eff), dtype=torch.int64, device=dev)
    if min_val is None:
        min_val = torch.finfo(rk.dtype).min
    if status is None:
        status = torch.zeros(4, dtype=torch.int32, device=dev)
    need = int(A.lib().msa_route_score_select_workspace_bytes(n_seq, top_k))
    if need < 0:
        raise A.MsaError("route_score_select: no CUDA device is current")
    if workspace is None or workspace.numel() * workspace.element_size() < need:
        workspace = torch.empty((need + 7) // 8, dtype=torch.int64, device=dev)
    A.check(A.lib().msa_route_score_select(A.ptr(q_folded), A.ptr(row_bias), A.dtype_code(rk.dtype), n_seq, A.ptr(rk2),
                                           stride, c, kdim, A.ptr(chunk_doc), float(alpha), n_docs,
                                           float(min_val), top_k, A.ptr(doc_ids_table), A.ptr(scores), A.ptr(local),
                                           A.ptr(glob), A.ptr(workspace), workspace.numel() * workspace.element_size(),
                                           A.ROUTE_KEYS_BLOCKED if blocked else 0, A.ptr(status), A.stream_ptr(dev)),
            "msa_route_score_select")
    return scores, local, glob


def route_table_reset(keys: torch.Tensor, n_docs: int, min_val: float, status: Optional[torch.Tensor] = None):
    A.need_cuda(keys, status)
    A.check(A.lib().msa_route_table_reset(A.ptr(keys), keys.stride(0), n_docs, keys.shape[0], float(min_val),
                                          A.ptr(status), A.stream_ptr(keys.device)), "msa_route_table_reset")


def topk_workspace_bytes(n_seq: int, n_cols: int, k: int) -> int:
    return int(A.lib().msa_topk_workspace_bytes(n_seq, n_cols, k))


def topk_select(keys: torch.Tensor, k: int, doc_ids_table: Optional[torch.Tensor] = None, n_cols: Optional[int] = None,
                workspace: Optional[torch.Tensor] = None, out=None):
    """Exact top-k of every row of a key table.  Returns ``(scores f32, local_ids i64, global_ids i64)``,
    each ``[n_seq, min(k, n_cols)]``, sorted by descending score (ties: ascending column).
    ``out``: three contiguous tensors of those shapes to write into (e.g. the planes of ``candidate_buffer``)."""
    A.need_cuda(keys, doc_ids_table)
    n_seq = keys.shape[0]
    n_cols = keys.shape[1] if n_cols is None else n_cols
    k_eff = min(k, n_cols)
    dev = keys.device
    if out is not None:
        scores, local, glob = out
        if not (scores.is_contiguous() and local.is_contiguous() and glob.is_contiguous()) or \
                tuple(scores.shape) != (n_seq, k_eff) or scores.dtype != torch.float32 or local.dtype != torch.int64:
            raise A.MsaError("topk_select: out must be contiguous (float32, int64, int64) tensors of shape [n_seq, k_eff]")
    else:
        scores = torch.empty((n_seq, k_eff), dtype=torch.float32, device=dev)
        local = torch.empty((n_seq, k_eff), dtype=torch.int64, device=dev)
        glob = torch.empty((n_seq, k_eff), dtype=torch.int64, device=dev)
    need = int(A.lib().msa_topk_workspace_bytes(n_seq, n_cols, k))
    if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
        workspace = torch.empty((need + 7) // 8, dtype=torch.int64, device=dev)
    A.check(A.lib().msa_topk_select(A.ptr(keys), keys.stride(0), n_seq, n_cols, k, A.ptr(doc_ids_table),
                                    A.ptr(scores), A.ptr(local), A.ptr(glob), A.ptr(workspace),
                                    workspace.numel() * workspace.element_size() if workspace is not None else 0,
                                    A.stream_ptr(dev)), "msa_topk_select")
    return scores, local, glob


def candidate_buffer(n_seq: int, k: int, device):
    """One int64 buffer ``[3, n_seq, k]`` that one collective can move: plane 0 holds the float32 scores in its
    first half, planes 1 and 2 the local and global ids.  Returns ``(buffer, scores, local, global)`` (views)."""
    buf = torch.empty((3, n_seq, k), dtype=torch.int64, device=device)
    scores = buf[0].view(torch.float32).view(-1)[: n_seq * k].view(n_seq, k)
    return buf, scores, buf[1], buf[2]


def candidate_views(gathered: torch.Tensor):
    """Views ``(scores, local, global)``, each ``[W, n_seq, k]``, of all-gathered candidate buffers ``[W, 3, n_seq, k]``."""
    w, _, n_seq, k = gathered.shape
    scores = gathered[:, 0].reshape(w, -1).view(torch.float32)[:, : n_seq * k].view(w, n_seq, k)
    return scores, gathered[:, 1], gathered[:, 2]


def topk_merge(cand_scores: torch.Tensor, cand_local: torch.Tensor, cand_global: torch.Tensor, k: int,
               seq_offset: int = 0, n_seq: Optional[int] = None, invalid_below: float = -1e9):
    """cand_* ``[W, B_all, kc]``, each rank's ``[B_all, kc]`` block contiguous (the rank stride is free, so the
    three may be planes of one all-gathered buffer); merges sequences ``seq_offset .. seq_offset+n_seq``.
    Returns ``(scores[n_seq,k] f32, local[n_seq,k] i64 (-1 = invalid), global[n_seq,k] i64, rank[n_seq,k] i32)``."""
    A.need_cuda(cand_scores, cand_local, cand_global)
    w, b_all, kc = cand_scores.shape
    n_seq = b_all - seq_offset if n_seq is None else n_seq
    dev = cand_scores.device
    k = min(k, w * kc)

    def blocks_ok(t):
        return t.stride(2) == 1 and t.stride(1) == kc
    cs = cand_scores if blocks_ok(cand_scores) else cand_scores.contiguous()
    cl = cand_local if blocks_ok(cand_local) else cand_local.contiguous()
    cg = cand_global if blocks_ok(cand_global) else cand_global.contiguous()
    if w > 1 and cl.stride(0) != cg.stride(0):
        cl, cg = cl.contiguous(), cg.contiguous()
    out_s = torch.empty((n_seq, k), dtype=torch.float32, device=dev)
    out_l = torch.empty((n_seq, k), dtype=torch.int64, device=dev)
    out_g = torch.empty((n_seq, k), dtype=torch.int64, device=dev)
    out_r = torch.empty((n_seq, k), dtype=torch.int32, device=dev)
    off = seq_offset * kc
    A.check(A.lib().msa_topk_merge(A.ptr(cs) + off * 4, A.ptr(cl) + off * 8, A.ptr(cg) + off * 8,
                                   cs.stride(0) if w > 1 else b_all * kc, cl.stride(0) if w > 1 else b_all * kc, w,
                                   n_seq, kc, k, invalid_below, A.ptr(out_s), A.ptr(out_l), A.ptr(out_g),
                                   A.ptr(out_r), A.stream_ptr(dev)), "msa_topk_merge")
    return out_s, out_l, out_g, out_r


# ---------------------------------------------------------------------------------------
# Fetch
# ---------------------------------------------------------------------------------------

def gather_plan(sel_local: torch.Tensor, sel_rank: Optional[torch.Tensor], world: int, shard_doc_base: torch.Tensor,
                doc_chunk_offset: torch.Tensor, doc_chunk_len: torch.Tensor, shard_kv_base: torch.Tensor,
                chunk_bytes: int, total_host: Optional[torch.Tensor] = None, sample_stride: int = 0,
                status: Optional[torch.Tensor] = None, resident: Optional[torch.Tensor] = None):
    """Plan the fetch of the winners ``sel_local[B, k]`` (owner ranks ``sel_rank``).  ``sample_stride`` 0 packs
    the samples one after another; > 0 gives every sample that many entries of room (see ``gather_run``).
    Winners outside the directory are dropped and counted in ``status[2]``.  ``resident`` ``[B, k]`` int64 (-1 =
    empty, updated in place; needs ``sample_stride`` = k slots of equal length): winners whose entries the sample's
    segment already holds are not planned again, the others go into the slots that became free.
    Returns ``(plan[B*k, 4], n_sel[B], total[1])``."""
    A.need_cuda(sel_local, sel_rank, shard_doc_base, doc_chunk_offset, doc_chunk_len, shard_kv_base, status)
    n_seq, k = sel_local.shape
    dev = sel_local.device
    if shard_doc_base.numel() != world or shard_kv_base.numel() != world:
        raise A.MsaError("gather_plan: shard_doc_base / shard_kv_base must have one entry per rank")
    if doc_chunk_offset.numel() != doc_chunk_len.numel():
        raise A.MsaError("gather_plan: doc_chunk_offset and doc_chunk_len differ in length")
    plan = torch.empty((n_seq * k, 4), dtype=torch.int64, device=dev)
    n_sel = torch.empty((n_seq,), dtype=torch.int64, device=dev)
    total = torch.empty((1,), dtype=torch.int64, device=dev)
    if resident is not None:
        A.need_cuda(resident)
        if resident.dtype != torch.int64 or tuple(resident.shape) != (n_seq, k) or not resident.is_contiguous():
            raise A.MsaError("gather_plan: resident must be a contiguous int64 [B, k] tensor")
        if sample_stride <= 0 or sample_stride % k != 0:
            raise A.MsaError("gather_plan: a resident table needs sample_stride = k slots of equal length")
        A.check(A.lib().msa_gather_plan_resident(
            A.ptr(sel_local.contiguous()), A.ptr(sel_rank.contiguous() if sel_rank is not None else None), n_seq, k, world,
            A.ptr(shard_doc_base), doc_chunk_len.numel(), A.ptr(doc_chunk_offset), A.ptr(doc_chunk_len), A.ptr(shard_kv_base),
            chunk_bytes, int(sample_stride) // k, A.ptr(resident), A.ptr(plan), A.ptr(n_sel), A.ptr(total), A.ptr(status),
            A.stream_ptr(dev)), "msa_gather_plan_resident")
        return plan, n_sel, total
    A.check(A.lib().msa_gather_plan(A.ptr(sel_local.contiguous()), A.ptr(sel_rank.contiguous() if sel_rank is not None else None),
                                    n_seq, k, world, A.ptr(shard_doc_base), doc_chunk_len.numel(), A.ptr(doc_chunk_offset),
                                    A.ptr(doc_chunk_len), A.ptr(shard_kv_base), chunk_bytes, int(sample_stride),
                                    A.ptr(plan), A.ptr(n_sel), A.ptr(total), A.ptr(total_host), A.ptr(status),
                                    A.stream_ptr(dev)), "msa_gather_plan")
    return plan, n_sel, total


def gather_run(plan: torch.Tensor, dtype: torch.dtype, n_kv_heads: int, head_dim: int, out_entries: int,
               max_ctas: int = 0, out=None):
    """Run a gather plan.  ``max_ctas``: 0 = one CTA per document; a small cap (24) when the fetch runs
    beside HBM-bound kernels, e.g. inside a decode step.  By default the result is packed
    ``[Hkv, out_entries, D]``.  ``out = (k_cache, v_cache, first_position)`` writes a plan made with
    ``sample_stride = out_entries`` straight into positions ``first_position ..`` of ``[B, Hkv, L, D]`` caches."""
    dev = plan.device
    if out is None:
        out_k = torch.empty((n_kv_heads, out_entries, head_dim), dtype=dtype, device=dev)
        out_v = torch.empty((n_kv_heads, out_entries, head_dim), dtype=dtype, device=dev)
        pk, pv, head_stride, sample_stride = A.ptr(out_k), A.ptr(out_v), out_entries * head_dim, 0
    else:
        out_k, out_v, first = out
        if out_k.stride() != out_v.stride() or out_k.stride(3) != 1 or out_k.stride(2) != head_dim or \
                first + out_entries > out_k.shape[2] or out_k.dtype != dtype:
            raise A.MsaError("gather_run: caches must be [B, Hkv, L, D] with contiguous (L, D) and room for the entries")
        off = first * head_dim * out_k.element_size()
        pk, pv, head_stride, sample_stride = A.ptr(out_k) + off, A.ptr(out_v) + off, out_k.stride(1), out_k.stride(0)
    A.check(A.lib().msa_gather_run(A.ptr(plan), plan.shape[0], A.dtype_code(dtype), n_kv_heads, head_dim,
                                   pk, pv, head_stride, out_entries, sample_stride, int(max_ctas),
                                   A.stream_ptr(dev)), "msa_gather_run")
    return out_k, out_v


# ---------------------------------------------------------------------------------------
# Decode attention
# ---------------------------------------------------------------------------------------

def decode_splits(n_seq: int, n_kv_heads: int, max_len: int, n_sm: int = 148) -> int:
    """KV splits for the decode kernel: about one CTA per SM in all, each keeping at least 256 keys.  Measured on
    B200 at 2,179 cached entries and 8 kv heads (us per layer, splits 1 / 2 / 4 / 8): 4 sequences 28.7 / 19.2 /
    14.3 / 16.4, 8 sequences 29.7 / 21.2 / 20.0 / 24.0, 16 sequences 30.6 / 32.1 / 32.2 / 40.0, 32 sequences
    52.6 / 54.7 / 57.7 / 62.6: more CTAs than SMs only add partial results to combine."""
    ctas = max(1, n_seq * n_kv_heads)
    return max(1, min(n_sm // ctas, max(1, max_len // 256)))


def sparse_decode_attn(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, kv_len: torch.Tensor,
                       new_k: Optional[torch.Tensor] = None, new_v: Optional[torch.Tensor] = None,
                       kv_start: Optional[torch.Tensor] = None, scale: Optional[float] = None,
                       n_splits: Optional[int] = None, workspace: Optional[torch.Tensor] = None,
                       out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q ``[B, Hq, D]``; caches ``[B, Hkv, Lcap, D]`` (position axis contiguous per head);
    kv_len / kv_start ``[B]`` int32; new_k / new_v ``[B, Hkv, D]``.  Returns ``[B, Hq*D]``."""
    A.need_cuda(q, k_cache, v_cache, kv_len, new_k, new_v, kv_start)
    b, hq, d = q.shape
    hkv, cap = k_cache.shape[1], k_cache.shape[2]
    if k_cache.stride(3) != 1 or k_cache.stride(2) != d or v_cache.stride() != k_cache.stride():
        raise A.MsaError("sparse_decode_attn: caches must be [B, Hkv, L, D] with contiguous (L, D)")
    if kv_len.dtype != torch.int32 or (kv_start is not None and kv_start.dtype != torch.int32):
        raise A.MsaError("sparse_decode_attn: kv_len / kv_start must be int32")
    dev = q.device
    q = q.contiguous()
    if new_k is not None:
        new_k, new_v = new_k.contiguous(), new_v.contiguous()
    if n_splits is None:
        n_splits = decode_splits(b, hkv, cap)
    need = int(A.lib().msa_decode_workspace_bytes(b, hq, d, n_splits))
    if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
        workspace = torch.empty(need // 4, dtype=torch.float32, device=dev)
    if out is None:
        out = torch.empty((b, hq * d), dtype=q.dtype, device=dev)
    scale = (1.0 / math.sqrt(d)) if scale is None else scale
    A.check(A.lib().msa_sparse_decode_attn(A.ptr(q), A.dtype_code(q.dtype), A.ptr(k_cache), A.ptr(v_cache),
                                           k_cache.stride(0), k_cache.stride(1), A.ptr(kv_start), A.ptr(kv_len),
                                           A.ptr(new_k), A.ptr(new_v), b, hq, hkv, d, float(scale), A.ptr(out),
                                           A.ptr(workspace), workspace.numel() * 4 if workspace is not None else 0,
                                           n_splits, A.stream_ptr(dev)), "msa_sparse_decode_attn")
    return out


def assemble_context(template_k, template_v, sel_k, sel_v, n_sel, key_states, value_states, valid, max_kv: int,
                     reserve: int = 0):
    """Build the compact stage-2 cache.  template_* ``[1, Hkv, t, D]``; sel_* ``[Hkv, sumN, D]`` (or None);
    n_sel ``[B]`` int64; key_states / value_states ``[B, Hkv, S, D]``; valid ``[B, S]`` bool.
    Returns ``(k_store, v_store [B, Hkv, max_kv + reserve, D], kv_start, kv_len, q_tok, num_q, error_flag)``;
    ``error_flag`` is 1 when some sequence is longer than ``max_kv`` (that sequence's storage is zeroed).
    ``q_tok[b]`` lists the valid tokens in order, then the others."""
    A.need_cuda(template_k, sel_k, n_sel, key_states, valid)
    b, hkv, s, d = key_states.shape
    dev, dt = key_states.device, key_states.dtype
    if key_states.stride(3) != 1 or value_states.stride() != key_states.stride():
        key_states, value_states = key_states.contiguous(), value_states.contiguous()
    t_len = template_k.shape[2]
    tk, tv = template_k.reshape(hkv, t_len, d), template_v.reshape(hkv, t_len, d)
    if not tk.is_contiguous() or not tv.is_contiguous():
        tk, tv = tk.contiguous(), tv.contiguous()
    if sel_k is not None and sel_k.shape[1] > 0:
        if sel_k.stride(2) != 1 or sel_k.stride(1) != d or sel_v.stride() != sel_k.stride():
            sel_k, sel_v = sel_k.contiguous(), sel_v.contiguous()
        sel_stride = sel_k.stride(0)
    else:
        sel_k = sel_v = None
        sel_stride = 0
    cap = max_kv + reserve
    store = torch.empty((2, b, hkv, cap, d), dtype=dt, device=dev)     # the kernel writes every position
    k_store, v_store = store[0], store[1]
    meta = torch.empty(3 * b + 1, dtype=torch.int32, device=dev)
    kv_start, kv_len, num_q, err = meta[:b], meta[b:2 * b], meta[2 * b:3 * b], meta[3 * b:]
    q_tok = torch.empty((b, max(s, 1)), dtype=torch.int32, device=dev)
    vmask = valid.reshape(b, s)
    vmask = vmask.contiguous().view(torch.uint8) if vmask.dtype == torch.bool else vmask.to(torch.uint8).contiguous()
    if n_sel.dtype != torch.int64 or not n_sel.is_contiguous():
        n_sel = n_sel.to(torch.int64).contiguous()
    A.check(A.lib().msa_assemble_context(
        A.ptr(tk), A.ptr(tv), t_len, A.ptr(sel_k), A.ptr(sel_v), sel_stride, A.ptr(n_sel),
        A.ptr(key_states), A.ptr(value_states), key_states.stride(0), key_states.stride(1), key_states.stride(2),
        A.ptr(vmask), b, s, hkv, d, A.dtype_code(dt), max_kv, cap, A.ptr(k_store), A.ptr(v_store), k_store.stride(0),
        k_store.stride(1), A.ptr(kv_start), A.ptr(kv_len), A.ptr(q_tok), A.ptr(num_q), A.ptr(err), A.stream_ptr(dev)),
        "msa_assemble_context")
    return k_store, v_store, kv_start, kv_len, q_tok, num_q, err


def append_segment(key_states: torch.Tensor, value_states: torch.Tensor, valid: torch.Tensor, k_store: torch.Tensor,
                   v_store: torch.Tensor, kv_start: Optional[torch.Tensor], kv_len: torch.Tensor):
    """Append the valid tokens of a segment ``[B, Hkv, S, D]`` to every sequence's store ``[B, Hkv, L, D]`` in place;
    ``kv_len`` (int32) grows by the number of valid tokens.  Returns ``(q_tok[B, S], num_q[B], error_flag[1])``;
    ``error_flag`` is 1 when some sequence's store had no room (that sequence is unchanged, ``num_q`` 0)."""
    A.need_cuda(key_states, value_states, valid, k_store, v_store, kv_start, kv_len)
    b, hkv, s, d = key_states.shape
    if key_states.stride(3) != 1 or value_states.stride() != key_states.stride():
        key_states, value_states = key_states.contiguous(), value_states.contiguous()
    if k_store.stride(3) != 1 or k_store.stride(2) != d or v_store.stride() != k_store.stride():
        raise A.MsaError("append_segment: stores must be [B, Hkv, L, D] with contiguous (L, D)")
    if kv_len.dtype != torch.int32 or (kv_start is not None and kv_start.dtype != torch.int32):
        raise A.MsaError("append_segment: kv_start / kv_len must be int32")
    vmask = valid.reshape(b, s)
    vmask = vmask.contiguous().view(torch.uint8) if vmask.dtype == torch.bool else vmask.to(torch.uint8).contiguous()
    dev = key_states.device
    q_tok = torch.empty((b, s), dtype=torch.int32, device=dev)
    meta = torch.zeros(b + 1, dtype=torch.int32, device=dev)
    A.check(A.lib().msa_append_segment(
        A.ptr(key_states), A.ptr(value_states), key_states.stride(0), key_states.stride(1), key_states.stride(2),
        A.ptr(vmask), b, s, hkv, d, A.dtype_code(key_states.dtype), A.ptr(k_store), A.ptr(v_store), k_store.stride(0),
        k_store.stride(1), k_store.shape[2], A.ptr(kv_start), A.ptr(kv_len), A.ptr(q_tok), A.ptr(meta), A.ptr(meta[b:]),
        A.stream_ptr(dev)), "msa_append_segment")
    return q_tok, meta[:b], meta[b:]


def sparse_prefill_attn(q: torch.Tensor, k_store, v_store, kv_start, kv_len, q_tok, num_q, scale: Optional[float] = None,
                        out: Optional[torch.Tensor] = None, causal: bool = True, q_runs: bool = False,
                        status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q ``[B, Hq, S, D]``.  Returns ``[B, S, Hq*D]``; rows of invalid tokens are zero (written by the kernel:
    ``out`` may be uninitialised).  ``causal``: bottom-right aligned causal mask (stage 2); False = every valid
    token sees the whole context (multi-token decode segments).  bf16 / D = 128 on tensor cores, anything else on
    the general kernel.  ``q_runs``: the caller has checked that every sequence's valid tokens are one run of
    consecutive tokens; bf16 / D = 128 then runs on the tcgen05 kernel (``status[0] != 0`` after a sync = it gave up)."""
    A.need_cuda(q, k_store, v_store)
    b, hq, s, d = q.shape
    if q.stride(3) != 1:
        q = q.contiguous()
    if out is None:
        out = torch.empty((b, s, hq * d), dtype=q.dtype, device=q.device)
    scale = (1.0 / math.sqrt(d)) if scale is None else scale
    if (q_runs and q.dtype == torch.bfloat16 and d == 128 and _tc_view_ok(q)
            and k_store.stride(3) == 1 and k_store.stride(2) == d and v_store.stride() == k_store.stride()
            and k_store.stride(1) == k_store.shape[2] * d and (b == 1 or k_store.stride(0) == k_store.shape[1] * k_store.stride(1))
            and k_store.data_ptr() % 16 == 0 and v_store.data_ptr() % 16 == 0
            and b * s * hq < 2 ** 31 and b * k_store.shape[1] * k_store.shape[2] < 2 ** 31):
        if status is None:
            status = torch.zeros(4, dtype=torch.int32, device=q.device)
        A.check(A.lib().msa_sparse_prefill_attn_tc(
            A.ptr(q), q.stride(0), q.stride(1), q.stride(2), A.ptr(k_store), A.ptr(v_store), k_store.stride(0),
            k_store.stride(1), k_store.shape[2], A.ptr(kv_start), A.ptr(kv_len), A.ptr(q_tok), A.ptr(num_q), b, s, hq,
            k_store.shape[1], d, A.dtype_code(q.dtype), int(causal), float(scale), A.ptr(out), A.ptr(status),
            A.stream_ptr(q.device)), "msa_sparse_prefill_attn_tc")
        return out
    A.check(A.lib().msa_sparse_prefill_attn(
        A.ptr(q), q.stride(0), q.stride(1), q.stride(2), A.ptr(k_store), A.ptr(v_store), k_store.stride(0),
        k_store.stride(1), A.ptr(kv_start), A.ptr(kv_len), A.ptr(q_tok), A.ptr(num_q), b, s, hq, k_store.shape[1], d,
        A.dtype_code(q.dtype), int(causal), float(scale), A.ptr(out), A.stream_ptr(q.device)), "msa_sparse_prefill_attn")
    return out


def doc_attention_pool(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, token_index: torch.Tensor,
                       seg_offsets: torch.Tensor, max_segment_len: int, out: Optional[torch.Tensor] = None,
                       chunk_offsets: Optional[torch.Tensor] = None, pool_size: int = 64, head_major_out: bool = False,
                       scale: Optional[float] = None):
    """Causal attention inside every segment of ``token_index`` and, when ``chunk_offsets`` is given (bf16, D = 128
    only), the chunk means of K and V from the same pass.  q ``[B, Hq, S, D]``; k, v ``[B, Hkv, S, D]``;
    token_index ``[Td]`` int32 flat positions; seg_offsets ``[n+1]`` int32.  ``out`` ``[B, S, Hq*D]`` keeps its
    content on rows that no segment lists (zeros when allocated here).
    Returns ``(out, pooled_k, pooled_v)``; pooled ``[C, Hkv, D]`` or, head major, ``[1, Hkv, C, D]`` (None without pooling)."""
    A.need_cuda(q, k, v, token_index, seg_offsets, chunk_offsets)
    b, hq, s, d = q.shape
    hkv = k.shape[1]
    if q.stride(3) != 1:
        q = q.contiguous()
    if k.stride(3) != 1 or v.stride() != k.stride():
        k, v = k.contiguous(), v.contiguous()
    if token_index.dtype != torch.int32 or seg_offsets.dtype != torch.int32:
        raise A.MsaError("doc_attention_pool: token_index and seg_offsets must be int32")
    if out is None:
        out = torch.zeros((b, s, hq * d), dtype=q.dtype, device=q.device)
    n_seg = seg_offsets.numel() - 1
    pooled_k = pooled_v = None
    cs = hs = n_chunks = 0
    if chunk_offsets is not None:
        n_chunks = chunk_offsets.numel() - 1
        shape = (1, hkv, n_chunks, d) if head_major_out else (n_chunks, hkv, d)
        pooled_k = torch.empty(shape, dtype=q.dtype, device=q.device)
        pooled_v = torch.empty(shape, dtype=q.dtype, device=q.device)
        cs, hs = (d, n_chunks * d) if head_major_out else (hkv * d, d)
    scale = (1.0 / math.sqrt(d)) if scale is None else scale
    for lo in range(0, max(n_seg, 1), 65535):      # grid.z limit
        n = min(65535, n_seg - lo)
        if n <= 0:
            break
        A.check(A.lib().msa_doc_attention_pool(
            A.ptr(q), q.stride(0), q.stride(1), q.stride(2), A.ptr(k), A.ptr(v), k.stride(0), k.stride(1), k.stride(2),
            A.ptr(token_index), A.ptr(seg_offsets) + 4 * lo, n, int(max_segment_len), s, hq, hkv, d,
            A.dtype_code(q.dtype), float(scale), A.ptr(out), A.ptr(chunk_offsets), n_chunks, int(pool_size),
            A.ptr(pooled_k), A.ptr(pooled_v), cs, hs, A.stream_ptr(q.device)), "msa_doc_attention_pool")
    return out, pooled_k, pooled_v


def _tc_view_ok(t: torch.Tensor) -> bool:
    """Token-major ([B, S, H, D] storage viewed as [B, H, S, D]) or contiguous head-major, rows 16-byte aligned."""
    b, h, s, d = t.shape
    sb, sh, ss, sd = t.stride()
    if sd != 1 or ss % 8 != 0 or t.data_ptr() % 16 != 0:
        return False
    token_major = sh == d and ss >= h * d and (b == 1 or sb == s * ss)
    head_major = ss >= d and sh == s * ss and (b == 1 or sb == h * sh)
    return token_major or head_major


def doc_attention_tc_supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> bool:
    """Whether ``doc_attention_tc`` takes these tensors as they are (dtype, head size, layouts)."""
    return (q.dtype == torch.bfloat16 and q.shape[-1] == 128 and k.stride() == v.stride() and _tc_view_ok(q)
            and _tc_view_ok(k) and v.data_ptr() % 16 == 0 and q.shape[0] * q.shape[1] * q.shape[2] < 2 ** 31)


def doc_attention_tc(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, token_index: torch.Tensor,
                     seg_offsets: torch.Tensor, max_segment_len: int, out: Optional[torch.Tensor] = None,
                     scale: Optional[float] = None, status: Optional[torch.Tensor] = None):
    """``doc_attention_pool`` without pooling on the tcgen05 kernel: every segment must be a run of consecutive
    tokens of one row, and q / k / v token-major or contiguous head-major (no copies are made here; other
    layouts raise).  Positions up to 127 tokens past a document's end must hold finite k / v values (they meet zero
    probabilities).  Returns ``(out, status)``; ``status[0] != 0`` after a sync means the kernel gave up."""
    A.need_cuda(q, k, v, token_index, seg_offsets)
    b, hq, s, d = q.shape
    hkv = k.shape[1]
    if v.stride() != k.stride() or q.stride(3) != 1 or k.stride(3) != 1:
        raise A.MsaError("doc_attention_tc: k and v must share strides and the feature axis must be contiguous")
    if token_index.dtype != torch.int32 or seg_offsets.dtype != torch.int32:
        raise A.MsaError("doc_attention_tc: token_index and seg_offsets must be int32")
    if out is None:
        out = torch.zeros((b, s, hq * d), dtype=q.dtype, device=q.device)
    if status is None:
        status = torch.zeros(4, dtype=torch.int32, device=q.device)
    scale = (1.0 / math.sqrt(d)) if scale is None else scale
    A.check(A.lib().msa_doc_attention_tc(
        A.ptr(q), q.stride(0), q.stride(1), q.stride(2), A.ptr(k), A.ptr(v), k.stride(0), k.stride(1), k.stride(2),
        A.ptr(token_index), A.ptr(seg_offsets), seg_offsets.numel() - 1, int(max_segment_len), b, s, hq, hkv, d,
        A.dtype_code(q.dtype), float(scale), A.ptr(out), A.ptr(status), A.stream_ptr(q.device)),
        "msa_doc_attention_tc")
    return out, status


def token_bitmap(mask: torch.Tensor) -> torch.Tensor:
    """``mask`` (bool, any shape) as a bitmap of 32-bit words over its flattened positions, padded by the 256
    positions and the extra word that ``doc_attention_tc_masked`` reads past the end."""
    flat = mask.reshape(-1)
    n = flat.numel()
    words = (n + 256 + 31) // 32 + 1
    padded = torch.zeros(words * 32, dtype=torch.int64, device=flat.device)
    padded[:n] = flat
    weights = torch.ones(32, dtype=torch.int64, device=flat.device) << torch.arange(32, device=flat.device)
    return (padded.view(words, 32) * weights).sum(dim=1).to(torch.int32)


def document_spans(token_index: torch.Tensor, seg_offsets: torch.Tensor):
    """From segments given as token lists (``token_index`` int32 ascending, ``seg_offsets``) the spans that
    ``doc_attention_tc_masked`` takes: every position from a segment's first to its last token.
    Returns ``(span_index int32, span_offsets int32, max_span_len)`` (one read-back for the sizes)."""
    first = token_index[seg_offsets[:-1].long()].long()
    last = token_index[(seg_offsets[1:] - 1).long()].long()
    length = last - first + 1
    off = torch.nn.functional.pad(length.cumsum(0), (1, 0))
    total, longest = torch.stack([off[-1], length.max()]).tolist()
    index = torch.repeat_interleave(first - off[:-1], length, output_size=total) + torch.arange(total, device=first.device)
    return index.to(torch.int32), off.to(torch.int32), int(longest)


def doc_attention_tc_masked(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, span_index: torch.Tensor,
                            span_offsets: torch.Tensor, max_span_len: int, valid_bits: torch.Tensor, out: torch.Tensor,
                            scale: Optional[float] = None, status: Optional[torch.Tensor] = None):
    """``doc_attention_tc`` for documents with masked tokens inside: segments are spans of memory
    (``document_spans``), ``valid_bits`` (``token_bitmap``) says which positions are tokens of their document; the
    rows of the others keep what ``out`` holds.  Returns ``(out, status)``."""
    A.need_cuda(q, k, v, span_index, span_offsets, valid_bits, out)
    b, hq, s, d = q.shape
    if v.stride() != k.stride() or q.stride(3) != 1 or k.stride(3) != 1:
        raise A.MsaError("doc_attention_tc_masked: k and v must share strides and the feature axis must be contiguous")
    if span_index.dtype != torch.int32 or span_offsets.dtype != torch.int32 or valid_bits.dtype != torch.int32:
        raise A.MsaError("doc_attention_tc_masked: span_index, span_offsets and valid_bits must be int32")
    if status is None:
        status = torch.zeros(4, dtype=torch.int32, device=q.device)
    scale = (1.0 / math.sqrt(d)) if scale is None else scale
    A.check(A.lib().msa_doc_attention_tc_masked(
        A.ptr(q), q.stride(0), q.stride(1), q.stride(2), A.ptr(k), A.ptr(v), k.stride(0), k.stride(1), k.stride(2),
        A.ptr(span_index), A.ptr(span_offsets), span_offsets.numel() - 1, int(max_span_len), b, s, hq, k.shape[1], d,
        A.dtype_code(q.dtype), float(scale), A.ptr(out), A.ptr(valid_bits.contiguous()), valid_bits.numel(), A.ptr(status),
        A.stream_ptr(q.device)), "msa_doc_attention_tc_masked")
    return out, status


def qk_norm_rope(qkv: torch.Tensor, n_q_heads: int, n_kv_heads: int, q_weight: torch.Tensor, k_weight: torch.Tensor,
                 eps: float, cos: torch.Tensor, sin: torch.Tensor, q_out: Optional[torch.Tensor] = None,
                 k_out: Optional[torch.Tensor] = None):
    """Per-head RMSNorm + rotary embedding of the q and k heads of a fused projection output ``[B, >= (Hq+Hkv)*128]``
    (bf16).  cos / sin ``[B, 128]``.  Returns ``(q[B, Hq, 128], k[B, Hkv, 128])``."""
    A.need_cuda(qkv, q_weight, k_weight, cos, sin)
    b = qkv.shape[0]
    if qkv.dtype != torch.bfloat16 or qkv.stride(1) != 1:
        raise A.MsaError("qk_norm_rope: qkv must be bf16 with a contiguous feature axis")
    cos, sin = cos.reshape(b, 128), sin.reshape(b, 128)
    if not cos.is_contiguous() or not sin.is_contiguous():
        cos, sin = cos.contiguous(), sin.contiguous()
    if q_out is None:
        q_out = torch.empty((b, n_q_heads, 128), dtype=qkv.dtype, device=qkv.device)
    if k_out is None:
        k_out = torch.empty((b, n_kv_heads, 128), dtype=qkv.dtype, device=qkv.device)
    A.check(A.lib().msa_qk_norm_rope(A.ptr(qkv), qkv.stride(0), b, n_q_heads, n_kv_heads, 128, A.ptr(q_weight),
                                     A.ptr(k_weight), float(eps), A.ptr(cos), A.ptr(sin), A.ptr(q_out), A.ptr(k_out),
                                     A.stream_ptr(qkv.device)), "msa_qk_norm_rope")
    return q_out, k_out


def add_rmsnorm(x: torch.Tensor, y: Optional[torch.Tensor], weight: torch.Tensor, eps: float):
    """``x_new = x + y`` (``y`` None: ``x``), ``h = rmsnorm(x_new) * weight``; rows ``[n, hidden]`` bf16 contiguous.
    Returns ``(x_new, h)``."""
    A.need_cuda(x, y, weight)
    if x.dtype != torch.bfloat16 or not x.is_contiguous() or (y is not None and not y.is_contiguous()):
        raise A.MsaError("add_rmsnorm: bf16 contiguous rows expected")
    n, hidden = x.shape
    x_new = torch.empty_like(x) if y is not None else x
    h = torch.empty_like(x)
    A.check(A.lib().msa_add_rmsnorm(A.ptr(x), A.ptr(y), A.ptr(weight), float(eps), n, hidden,
                                    A.ptr(x_new) if y is not None else 0, A.ptr(h), A.stream_ptr(x.device)),
            "msa_add_rmsnorm")
    return x_new, h


def silu_mul(gate_up: torch.Tensor, ffn: int) -> torch.Tensor:
    """``silu(gate_up[:, :ffn]) * gate_up[:, ffn:]`` (bf16)."""
    A.need_cuda(gate_up)
    if gate_up.dtype != torch.bfloat16 or gate_up.stride(1) != 1:
        raise A.MsaError("silu_mul: bf16 rows with a contiguous feature axis expected")
    n = gate_up.shape[0]
    out = torch.empty((n, ffn), dtype=gate_up.dtype, device=gate_up.device)
    A.check(A.lib().msa_silu_mul(A.ptr(gate_up), gate_up.stride(0), n, ffn, A.ptr(out), A.stream_ptr(gate_up.device)),
            "msa_silu_mul")
    return out


def keys_to_scores(keys: torch.Tensor) -> torch.Tensor:
    """Decode a table of order-preserving keys (int32 storage) back to float32 scores."""
    u = keys.to(torch.int64) & 0xFFFFFFFF
    bits = torch.where((u & 0x80000000) != 0, u & 0x7FFFFFFF, (~u) & 0xFFFFFFFF)
    bits = torch.where(bits >= 2 ** 31, bits - 2 ** 32, bits).to(torch.int32)
    return bits.view(torch.float32)

"""ctypes binding of ``libmsa_b200.so`` (declared in ``include/msa_b200.h``).

There is no fallback: if the library is missing or a call fails, an exception is raised.
Every wrapper takes torch tensors, checks device / dtype / contiguity, and passes raw
pointers, sizes and the current CUDA stream to the C ABI.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmsa_b200.so")

MSA_F32, MSA_BF16 = 0, 1
QREDUCE = {"max": 0, "mean": 1, "last": 2}
HREDUCE = {"mean": 0, "max": 1}
CREDUCE = {"max": 0, "mean": 1}
ROUTE_FORCE_SIMT, ROUTE_NO_INIT, ROUTE_KEYS_BLOCKED = 1, 2, 4

EXPORTS = [
    "msa_abi_version", "msa_last_error", "msa_bookkeeping_workspace_bytes", "msa_chunk_bookkeeping", "msa_pool_chunks", "msa_fold_queries",
    "msa_route_s_pad", "msa_router_keys_blocked_bytes", "msa_router_keys_block", "msa_selftest_bounded_wait", "msa_route_table_reset", "msa_route_scores", "msa_route_chunk_scores", "msa_route_reduce_chunks", "msa_route_score_select_workspace_bytes", "msa_route_score_select", "msa_topk_workspace_bytes", "msa_topk_select", "msa_topk_merge", "msa_gather_plan", "msa_gather_plan_resident",
    "msa_gather_run", "msa_bank_register_host", "msa_bank_unregister_host", "msa_assemble_context", "msa_sparse_prefill_attn", "msa_append_segment", "msa_doc_attention_pool", "msa_doc_attention_tc", "msa_doc_attention_tc_masked", "msa_sparse_prefill_attn_tc", "msa_qk_norm_rope", "msa_add_rmsnorm", "msa_silu_mul", "msa_decode_workspace_bytes", "msa_sparse_decode_attn",
    "msa_decode_static_scratch_bytes", "msa_sparse_decode_attn_static",
]


class MsaError(RuntimeError):
    pass


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m msa_b200.build` "
                "(nvcc, sm_100a).  msa_b200 has no CPU or PyTorch fallback.")
        l = C.CDLL(LIB_PATH)
        vp, i32, i64, f32, u32 = C.c_void_p, C.c_int32, C.c_int64, C.c_float, C.c_uint32
        l.msa_last_error.restype = C.c_char_p
        l.msa_abi_version.restype = C.c_int
        l.msa_bookkeeping_workspace_bytes.argtypes = [i32, i32]
        l.msa_bookkeeping_workspace_bytes.restype = i64
        l.msa_chunk_bookkeeping.argtypes = [vp, vp, i32, i32, i32, vp, vp, vp, i32, vp, vp, i64, vp]
        l.msa_pool_chunks.argtypes = [vp, i32, i64, i64, vp, vp, vp, i32, i32, i32, vp, i64, i64, i32, vp]
        l.msa_fold_queries.argtypes = [vp, i32, i64, i64, i64, vp, i64, i32, i32, i32, i32, i32, i32, i32, i32, vp, vp, vp]
        l.msa_route_s_pad.argtypes = [i32, i32]
        l.msa_route_s_pad.restype = i32
        l.msa_route_scores.argtypes = [vp, vp, i32, i32, i32, vp, i64, i32, i32, vp, f32, vp, i64, i32, f32, u32, vp, vp]
        l.msa_route_chunk_scores.argtypes = [vp, i32, i64, i64, i64, vp, i64, i32, i32, i32, i32, i32, i32, i32, vp, i64, i32,
                                             f32, f32, vp, i64, vp]
        l.msa_route_reduce_chunks.argtypes = [vp, i64, i32, i32, vp, i32, i32, f32, vp, i64, vp, vp]
        l.msa_route_score_select_workspace_bytes.argtypes = [i32, i32]
        l.msa_route_score_select_workspace_bytes.restype = i64
        l.msa_route_score_select.argtypes = [vp, vp, i32, i32, vp, i64, i32, i32, vp, f32, i32, f32, i32, vp, vp, vp, vp, vp,
                                             i64, u32, vp, vp]
        l.msa_router_keys_blocked_bytes.argtypes = [i32, i32]
        l.msa_router_keys_blocked_bytes.restype = i64
        l.msa_router_keys_block.argtypes = [vp, i64, i32, i32, i32, vp, vp]
        l.msa_selftest_bounded_wait.argtypes = [i64, vp, vp]
        l.msa_route_table_reset.argtypes = [vp, i64, i32, i32, f32, vp, vp]
        l.msa_topk_workspace_bytes.argtypes = [i32, i32, i32]
        l.msa_topk_workspace_bytes.restype = i64
        l.msa_topk_select.argtypes = [vp, i64, i32, i32, i32, vp, vp, vp, vp, vp, i64, vp]
        l.msa_topk_merge.argtypes = [vp, vp, vp, i64, i64, i32, i32, i32, i32, f32, vp, vp, vp, vp, vp]
        l.msa_gather_plan.argtypes = [vp, vp, i32, i32, i32, vp, i64, vp, vp, vp, i64, i64, vp, vp, vp, vp, vp, vp]
        l.msa_gather_plan_resident.argtypes = [vp, vp, i32, i32, i32, vp, i64, vp, vp, vp, i64, i32, vp, vp, vp, vp, vp, vp]
        l.msa_gather_run.argtypes = [vp, i32, i32, i32, i32, vp, vp, i64, i64, i64, i32, vp]
        l.msa_bank_register_host.argtypes = [vp, i64, vp]
        l.msa_bank_unregister_host.argtypes = [vp]
        l.msa_decode_workspace_bytes.argtypes = [i32, i32, i32, i32]
        l.msa_decode_workspace_bytes.restype = i64
        l.msa_sparse_decode_attn.argtypes = [vp, i32, vp, vp, i64, i64, vp, vp, vp, vp, i32, i32, i32, i32, f32, vp,
                                             vp, i64, i32, vp]
        l.msa_assemble_context.argtypes = [vp, vp, i32, vp, vp, i64, vp, vp, vp, i64, i64, i64, vp, i32, i32, i32, i32, i32,
                                           i32, i32, vp, vp, i64, i64, vp, vp, vp, vp, vp, vp]
        l.msa_sparse_prefill_attn.argtypes = [vp, i64, i64, i64, vp, vp, i64, i64, vp, vp, vp, vp, i32, i32, i32, i32, i32,
                                              i32, i32, f32, vp, vp]
        l.msa_append_segment.argtypes = [vp, vp, i64, i64, i64, vp, i32, i32, i32, i32, i32, vp, vp, i64, i64, i32, vp, vp,
                                         vp, vp, vp, vp]
        l.msa_doc_attention_pool.argtypes = [vp, i64, i64, i64, vp, vp, i64, i64, i64, vp, vp, i32, i32, i32, i32, i32, i32,
                                             i32, f32, vp, vp, i32, i32, vp, vp, i64, i64, vp]
        l.msa_doc_attention_tc.argtypes = [vp, i64, i64, i64, vp, vp, i64, i64, i64, vp, vp, i32, i32, i32, i32, i32, i32,
                                           i32, i32, f32, vp, vp, vp]
        l.msa_doc_attention_tc_masked.argtypes = [vp, i64, i64, i64, vp, vp, i64, i64, i64, vp, vp, i32, i32, i32, i32, i32, i32,
                                                  i32, i32, f32, vp, vp, i64, vp, vp]
        l.msa_sparse_prefill_attn_tc.argtypes = [vp, i64, i64, i64, vp, vp, i64, i64, i32, vp, vp, vp, vp, i32, i32, i32, i32,
                                                 i32, i32, i32, f32, vp, vp, vp]
        l.msa_qk_norm_rope.argtypes = [vp, i64, i32, i32, i32, i32, vp, vp, f32, vp, vp, vp, vp, vp]
        l.msa_add_rmsnorm.argtypes = [vp, vp, vp, f32, i32, i32, vp, vp, vp]
        l.msa_silu_mul.argtypes = [vp, i64, i32, i32, vp, vp]
        l.msa_decode_static_scratch_bytes.restype = i64
        l.msa_sparse_decode_attn_static.argtypes = [vp, i32, vp, vp, i64, i64, vp, vp, vp, vp, i32, i32, i32, i32, f32, vp,
                                                    i32, vp]
        for name in EXPORTS:
            fn = getattr(l, name)
            if fn.restype is C.c_int and name not in ("msa_abi_version",):
                fn.restype = C.c_int
        _lib = l
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise MsaError(f"{what} failed ({rc}): {lib().msa_last_error().decode()}")


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return MSA_F32
    if dt == torch.bfloat16:
        return MSA_BF16
    raise MsaError(f"unsupported dtype {dt}: the kernels take float32 or bfloat16")


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def stream_ptr(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise MsaError("msa_b200 kernels take CUDA tensors; there is no CPU path")

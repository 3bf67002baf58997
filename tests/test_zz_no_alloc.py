"""The allocation-free decode entry point (msa_sparse_decode_attn_static) against the regular
one (msa_sparse_decode_attn), both called through the C ABI.

The static variant is for hosts that cannot allocate device memory when a decode step runs (a
serving loop whose pool owns the whole GPU, a plugin that only gets its inputs and outputs);
its split-KV partials live in an array built into the library.  That array is shared by all
calls and keeps the previous call's contents, so the test makes two calls in a row with
different inputs and a different split count, and checks each against the regular entry
point, plus the rejection of a problem too large for the built-in array.

This file is collected last on purpose: a run that stops at the first failure has then
already run every other test.
"""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _call(fn, extra, q, kc, vc, kv_len, nk, nv, out, n_splits):
    from msa_b200 import _cabi as A
    b, hq, d = q.shape
    hkv = kc.shape[1]
    args = [A.ptr(q), A.dtype_code(q.dtype), A.ptr(kc), A.ptr(vc), kc.stride(0), kc.stride(1), None, A.ptr(kv_len),
            A.ptr(nk), A.ptr(nv), b, hq, hkv, d, 1.0 / math.sqrt(d), A.ptr(out)] + extra + [n_splits,
            A.stream_ptr(q.device)]
    return fn(*args)


def _inputs(seed, b, lens, dtype):
    g = torch.Generator().manual_seed(seed)
    hq, hkv, d = 32, 8, 128
    cap = max(lens) + 1
    mk = lambda *s: torch.randn(*s, generator=g).to(dtype).to(DEV)
    return (mk(b, hq, d), mk(b, hkv, cap, d), mk(b, hkv, cap, d),
            torch.tensor(lens, dtype=torch.int32, device=DEV), mk(b, hkv, d), mk(b, hkv, d))


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 1e-2), (torch.float32, 1e-5)])
def test_static_scratch_decode_matches_regular_entry_point(dtype, tol):
    from msa_b200 import _cabi as A
    lib = A.lib()
    assert lib.msa_decode_static_scratch_bytes() == 8 * 1024 * 1024
    for seed, lens, n_splits in [(1, [2179, 700, 64, 1], 6), (2, [300, 1500, 33, 2048], 3)]:
        q, kc, vc, kv_len, nk, nv = _inputs(seed, len(lens), lens, dtype)
        kc2, vc2 = kc.clone(), vc.clone()
        out_ref = torch.empty((len(lens), q.shape[1] * q.shape[2]), dtype=dtype, device=DEV)
        out_new = torch.full_like(out_ref, float("nan"))
        need = lib.msa_decode_workspace_bytes(len(lens), q.shape[1], q.shape[2], n_splits)
        ws = torch.empty(need // 4, dtype=torch.float32, device=DEV)
        A.check(_call(lib.msa_sparse_decode_attn, [A.ptr(ws), need], q, kc, vc, kv_len, nk, nv, out_ref, n_splits),
                "msa_sparse_decode_attn")
        A.check(_call(lib.msa_sparse_decode_attn_static, [], q, kc2, vc2, kv_len, nk, nv, out_new, n_splits),
                "msa_sparse_decode_attn_static")
        torch.cuda.synchronize()
        err = float((out_new.double() - out_ref.double()).norm() / out_ref.double().norm())
        assert err < tol, err
        assert torch.equal(kc, kc2) and torch.equal(vc, vc2)      # same in-place append
        # the point of the entry point: a call leaves the device's free memory and torch's pool untouched
        # (the first call on a device may load the module that holds the array, so this is a repeat call)
        torch.cuda.synchronize()
        free_before, pool_before = torch.cuda.mem_get_info(DEV)[0], torch.cuda.memory_reserved(DEV)
        A.check(_call(lib.msa_sparse_decode_attn_static, [], q, kc2, vc2, kv_len, nk, nv, out_new, n_splits),
                "msa_sparse_decode_attn_static")
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info(DEV)[0] == free_before and torch.cuda.memory_reserved(DEV) == pool_before


def test_static_scratch_rejects_oversized_problem():
    from msa_b200 import _cabi as A
    lib = A.lib()
    q, kc, vc, kv_len, nk, nv = _inputs(3, 2, [100, 100], torch.bfloat16)
    out = torch.empty((2, 32 * 128), dtype=torch.bfloat16, device=DEV)
    # 2 * 32 * n_splits * 130 * 4 bytes > 8 MiB  <=>  n_splits > 252
    rc = _call(lib.msa_sparse_decode_attn_static, [], q, kc, vc, kv_len, nk, nv, out, 300)
    assert rc == -1 and b"exceeds the built-in" in lib.msa_last_error()

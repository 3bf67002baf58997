"""Runs the reference's OWN routing code (``oracle/_ref``, built by ``oracle/build_ref.py``) on given tensors.
TEST INFRASTRUCTURE ONLY: imported by ``tests/`` and by ``bench.py``'s reference / baseline legs, never by the
product package.

The reference's ``Memory`` needs CUDA and a checkpoint in its constructor (src/msa_service.py:280-286), so the
object is made with ``object.__new__`` and only the attributes that ``_generate_slice`` (:644-695) and
``prefill_stage2`` (:703-828) read are set.  Those two methods then run unmodified, on the CPU or on a GPU.
"""
import os
import sys
from types import SimpleNamespace

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def available() -> bool:
    return os.path.exists(os.path.join(REF, "src", "msa_service.py"))


_svc = None


def reference_service_module():
    """``src.msa_service`` of the reference.  Two names that transformers 5 removed are given placeholders first:
    only the reference's unused quantized cache refers to them (src/utils/cache.py:11)."""
    global _svc
    if _svc is None:
        if not available():
            raise ImportError("oracle/_ref is missing: run `python oracle/build_ref.py --reference <MSA checkout>`")
        if REF not in sys.path:
            sys.path.insert(0, REF)
        import transformers.cache_utils as cu
        for n in ("QuantoQuantizedCache", "QuantizedCacheConfig"):
            if not hasattr(cu, n):
                setattr(cu, n, type(n, (), {}))
        import src.msa_service as svc
        _svc = svc
    return _svc


def make_reference_memory(rk_head_major: torch.Tensor, chunks_per_doc, global_ids, top_k: int,
                          reduce=("mean", "max", "max"), slice_chunks: int = 16 * 1024):
    """A reference ``Memory`` over one layer's router keys ``[1, Hkv, C, D]`` (the reference's layout), sliced by
    its own ``_generate_slice``."""
    svc = reference_service_module()
    dev = rk_head_major.device
    docs = [svc.Document(doc="", doc_id=int(g), num_chunks=int(n)) for g, n in zip(global_ids, chunks_per_doc)]
    m = object.__new__(svc.Memory)
    m.device = dev
    m.gpu_id = 0
    m.router_layer_ids = [0]
    m.head_reduce_method, m.query_reduce_method, m.chunk_reduce_method = reduce
    m.model_config = SimpleNamespace(doc_top_k=top_k)
    m.block_desc = svc.BlockDesc()
    m.block_desc.init_docs(docs, dev)
    m.block_desc.pool_ids = torch.repeat_interleave(torch.arange(1, len(docs) + 1),
                                                    torch.as_tensor(list(chunks_per_doc))).to(dev)
    m.blocks = {0: svc.BlockData(k=None, v=None, rk=rk_head_major)}
    m._generate_slice(slice_chunks)
    return m


def reference_prefill_stage2(memory, q5: torch.Tensor, mask: torch.Tensor):
    """``Memory.prefill_stage2(0, q[B, Hkv, G, S, D], mask[B, S])`` of the reference, unmodified."""
    b, s = mask.shape
    return memory.prefill_stage2(0, q5, mask.view(b, 1, 1, s, 1))

"""Per-GPU memory bank: the B200 counterpart of the reference's ``Memory`` worker.

Mirrors ``src/msa_service.py``: ``Document`` (src/types.py:5-9), ``BlockDesc`` (:191-231),
``BlockData`` (:234-242), ``Memory`` (:269-828).  Same method names and argument meaning;
the bodies call the CUDA kernels of this package.

Bank layout (differs from the reference's head-major ``[1, Hkv, C, D]`` on purpose):
  * routing keys ``rk``: ``[C, Hkv, D]`` on the GPU, chunk major, so one chunk is one
    contiguous 2 KiB row for TMA;
  * content ``kv``: ``[C, 2, Hkv, D]`` in pinned host memory (K then V per chunk), so one
    document is one contiguous run for the gather kernel.
``BlockData.k / .v / .rk_head_major`` give reference-shaped views.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from . import _cabi as A
from . import ops


@dataclass
class Document:
    doc: str = ""
    doc_id: int = 0
    num_chunks: int = 0


@dataclass
class ModelConfig:
    """The fields of the reference's ModelConfig (src/config/memory_config.py:28-46) this path reads."""
    model_path: str = ""
    doc_top_k: int = 16
    pooling_kernel_size: int = 64
    router_layer_idx: str = "all"
    template_token_id: int = -2
    template_id_num: int = 3
    envs: Optional[dict] = None     # environment of the stage-1 worker process (get_model_envs in the reference)


@dataclass
class MemoryConfig:
    """src/config/memory_config.py:48-56.  ``slice_chunk_size`` is accepted and unused: the
    fused kernel never materialises a score slice."""
    block_size: int = 16000
    slice_chunk_size: int = 16 * 1024
    pooling_kernel_size: int = 64
    memory_file_path: str = ""


@dataclass
class AttentionGeometry:
    """What the reference reads from the checkpoint's MSAConfig (src/msa_service.py:286-321)."""
    num_hidden_layers: int = 36
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    head_reduce_method: str = "mean"
    query_reduce_method: str = "max"
    chunk_reduce_method: str = "max"
    aux_loss_method: str = "INFONCE"
    decouple_router: bool = True
    dtype: torch.dtype = torch.bfloat16


class BlockDesc:
    """Tables of one GPU's shard (src/msa_service.py:191-231)."""

    def __init__(self):
        self.docs: List[Document] = []
        self.tmp_doc_ids: List[torch.Tensor] = []
        self.pool_ids: Optional[torch.Tensor] = None        # [C] int64, 1-based local doc per chunk
        self.chunk_doc: Optional[torch.Tensor] = None       # same, int32, what the kernels read
        self.doc_ids: Optional[torch.Tensor] = None         # [N+1] local -> global, slot 0 dummy
        self.doc_ids_cpu: Optional[torch.Tensor] = None
        self.doc_offsets_cpu: Optional[torch.Tensor] = None
        self.doc_lens_cpu: Optional[torch.Tensor] = None
        self.doc_offsets: Optional[torch.Tensor] = None     # device copies for the gather plan
        self.doc_lens: Optional[torch.Tensor] = None

    def init_docs(self, docs: List[Document], device):
        self.docs = docs
        self.doc_ids_cpu = torch.tensor([0] + [d.doc_id for d in docs], dtype=torch.long)
        self.doc_ids = self.doc_ids_cpu.to(device)
        self.tmp_doc_ids = []
        lens = [0] + [d.num_chunks for d in docs]
        self.doc_lens_cpu = torch.tensor(lens, dtype=torch.long)
        self.doc_offsets_cpu = torch.cumsum(torch.tensor([0] + lens[:-1], dtype=torch.long), dim=0)
        self.doc_offsets = self.doc_offsets_cpu.to(device)
        self.doc_lens = self.doc_lens_cpu.to(torch.int32).to(device)

    def create_global_doc_ids(self, local_doc_ids):
        return self.doc_ids[local_doc_ids]

    def set_pool_ids(self, pool_ids: torch.Tensor, device):
        self.pool_ids_cpu = pool_ids.cpu()
        self.pool_ids = pool_ids.to(device)
        self.chunk_doc = self.pool_ids.to(torch.int32)

    def merge_poolig_doc_id(self, device):
        """Concatenate the per-block ``pooled_doc_ids`` (each numbered from 1) into shard-wide
        ids, as ``cumulative_concat`` does (src/utils/tools.py:34-55, src/msa_service.py:221-224)."""
        out, base = [], 0
        for t in self.tmp_doc_ids:
            t = t.cpu().long()
            out.append(t + base)
            base += int(t[-1])
        self.set_pool_ids(torch.cat(out) if out else torch.empty(0, dtype=torch.long), device)
        self.tmp_doc_ids.clear()

    def pool_ids_from_docs(self, device):
        """pool_ids straight from the documents' chunk counts (equal to what ingestion yields)."""
        ids = torch.repeat_interleave(torch.arange(1, len(self.docs) + 1), self.doc_lens_cpu[1:])
        self.set_pool_ids(ids, device)

    def chunks(self) -> int:
        return sum(d.num_chunks for d in self.docs)

    @property
    def nr_docs(self) -> int:
        return len(self.docs)


@dataclass
class BlockData:
    rk: Optional[torch.Tensor] = None   # [C, Hkv, D] device (None once only the blocked copy is kept)
    rk_blocked: Optional[torch.Tensor] = None   # [tiles, Hkv*D/64, 128, 64] device: tile-blocked copy of rk
    n_chunks: int = 0                   # chunks held (rk_blocked is padded to whole tiles)
    kv: Optional[torch.Tensor] = None   # [C, 2, Hkv, D] pinned host
    kv_device_address: int = 0          # address the GPU uses for ``kv``

    @property
    def k(self):   # reference shape [1, Hkv, C, D] (a view of the pinned bank)
        return self.kv[:, 0].permute(1, 0, 2).unsqueeze(0)

    @property
    def v(self):
        return self.kv[:, 1].permute(1, 0, 2).unsqueeze(0)

    @property
    def rk_head_major(self):
        return self.get_router_k().permute(1, 0, 2).unsqueeze(0)

    def get_router_k(self):
        """Row-major router keys ``[C, Hkv, D]`` (materialised from the blocked copy when only that is kept)."""
        if self.rk is not None:
            return self.rk
        h, d = self.kv.shape[2], self.kv.shape[3]
        return ops.unblock_router_keys(self.rk_blocked, self.n_chunks).view(self.n_chunks, h, d)


def is_reference_bank(path: str) -> bool:
    """True when ``path`` holds a bank written by the reference's ``Memory.serialize``
    (src/msa_service.py:351-420: ``stub.json``, ``meta.pt``, ``layer_<l>_{k,v,rk}.pt``) and not one of this
    package's (``meta.json``)."""
    return (not os.path.exists(os.path.join(path, "meta.json"))
            and (os.path.exists(os.path.join(path, "stub.json")) or os.path.exists(os.path.join(path, "meta.pt"))))


def convert_reference_bank(src_dir: str, dst_dir: str) -> dict:
    """One-time conversion of a bank directory written by the reference (head-major ``[1, Hkv, C, D]`` tensors in
    ``layer_<l>_k.pt`` / ``_v.pt`` / ``_rk.pt``, documents in ``meta.pt``) into this package's format
    (``serialize``): chunk-major ``rk_L<l>.bin`` ``[C, Hkv, D]`` and ``kv_L<l>.bin`` ``[C, 2, Hkv, D]``.
    Runs on the CPU, one layer in memory at a time.  A bank without separate router keys (``decouple_router``
    off) routes on K, as in the reference (``BlockData.get_router_k``, :241-243).  Returns the written meta."""
    import sys
    import types
    if not is_reference_bank(src_dir):
        raise A.MsaError(f"{src_dir}: no reference-format bank found (meta.pt)")
    # meta.pt pickles the reference's src.types.Document; give the unpickler a class of that name and fields
    injected = []
    if "src.types" not in sys.modules:
        pkg = sys.modules.get("src") or types.ModuleType("src")
        mod = types.ModuleType("src.types")
        mod.Document = Document
        for name, m in (("src", pkg), ("src.types", mod)):
            if name not in sys.modules:
                sys.modules[name] = m
                injected.append(name)
    try:
        meta = torch.load(os.path.join(src_dir, "meta.pt"), map_location="cpu", weights_only=False)
    finally:
        for name in injected:
            sys.modules.pop(name, None)
    docs = meta["block_desc"]["docs"]
    layers = [int(l) for l in meta["router_layer_ids"]]
    os.makedirs(dst_dir, exist_ok=True)
    out = None
    for layer in layers:
        load = lambda kind: torch.load(os.path.join(src_dir, f"layer_{layer}_{kind}.pt"), map_location="cpu",
                                       weights_only=False)
        k, v = load("k"), load("v")
        rk = load("rk") if os.path.exists(os.path.join(src_dir, f"layer_{layer}_rk.pt")) else k
        _, h, c, d = k.shape
        if c != sum(int(x.num_chunks) for x in docs):
            raise A.MsaError(f"{src_dir}: layer {layer} holds {c} chunks, the documents list {sum(x.num_chunks for x in docs)}")
        kv = torch.stack([k[0].permute(1, 0, 2), v[0].to(k.dtype).permute(1, 0, 2)], dim=1).contiguous()   # [C, 2, Hkv, D]
        rk.to(k.dtype)[0].permute(1, 0, 2).contiguous().view(torch.uint8).numpy().tofile(os.path.join(dst_dir, f"rk_L{layer}.bin"))
        kv.view(torch.uint8).numpy().tofile(os.path.join(dst_dir, f"kv_L{layer}.bin"))
        out = {"format": "msa_b200-bank-1", "dtype": str(k.dtype).replace("torch.", ""), "n_chunks": int(c),
               "n_kv_heads": int(h), "head_dim": int(d), "router_layer_ids": layers,
               "doc_ids": [int(x.doc_id) for x in docs], "doc_chunks": [int(x.num_chunks) for x in docs]}
    prefix = os.path.join(src_dir, "prefix_cache.pt")
    pc = torch.load(prefix, map_location="cpu", weights_only=False) if os.path.exists(prefix) else {}
    torch.save({int(l): (k_, v_) for l, (k_, v_) in pc.items()}, os.path.join(dst_dir, "prefix_cache.pt"))
    with open(os.path.join(dst_dir, "meta.json"), "w") as f:
        json.dump(out, f)
    return out


class Memory:
    """One GPU's bank plus local scoring and selection (src/msa_service.py:269-828)."""

    def __init__(self, gpu_id: int, generate_config=None, model_config: Optional[ModelConfig] = None,
                 memory_config: Optional[MemoryConfig] = None, geometry: Optional[AttentionGeometry] = None):
        if not torch.cuda.is_available():
            raise A.MsaError("msa_b200.Memory needs a CUDA device; there is no CPU path")
        A.lib()  # fail now, loudly, if the kernels are not built
        self.gpu_id = gpu_id
        self.device = torch.device("cuda", gpu_id)
        self.generate_config = generate_config
        self.model_config = model_config or ModelConfig()
        self.memory_config = memory_config or MemoryConfig()
        self.geometry = geometry or AttentionGeometry()
        g = self.geometry
        ridx = self.model_config.router_layer_idx
        self.router_layer_ids = sorted(range(g.num_hidden_layers) if ridx == "all" else map(int, ridx.split(",")))
        self.num_key_value_groups = g.num_attention_heads // g.num_key_value_heads
        self.head_reduce_method = g.head_reduce_method
        self.query_reduce_method = g.query_reduce_method
        self.chunk_reduce_method = g.chunk_reduce_method
        self.aux_loss_method = g.aux_loss_method
        self.decouple_router = g.decouple_router
        if self.head_reduce_method not in A.HREDUCE:
            raise A.MsaError(f"unknown head_reduce_method {self.head_reduce_method!r}")
        if self.chunk_reduce_method not in A.CREDUCE:
            raise A.MsaError(f"unknown chunk_reduce_method {self.chunk_reduce_method!r}")
        if self.query_reduce_method not in A.QREDUCE:
            raise A.MsaError(f"unknown query_reduce_method {self.query_reduce_method!r}")
        # src/msa_service.py:318-321: -1 means "cosine mode, do not scale"
        self.scaling = -1.0 if (self.aux_loss_method == "INFONCE" and self.decouple_router) else g.head_dim ** -0.5
        self.blocks: Dict[int, BlockData] = {layer: BlockData() for layer in self.router_layer_ids}
        self.block_desc = BlockDesc()
        self.template_prefix_kvcache: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        self._kv_offset = 0
        self._status = torch.zeros(4, dtype=torch.int32, device=self.device)
        #: decode-time routing (one query row per sequence) on the fused score + select kernel
        self.fused_decode_routing = os.environ.get("MSA_B200_NO_FUSED_DECODE_ROUTING") is None

    # ------------------------------------------------------------------ bank build
    def _init_block_data(self, dtype: torch.dtype):
        """Allocate the shard for every router layer (src/msa_service.py:481-492)."""
        g = self.geometry
        c = self.block_desc.chunks()
        for layer in self.router_layer_ids:
            blk = self.blocks[layer]
            if blk.rk is None:
                blk.rk = torch.empty((c, g.num_key_value_heads, g.head_dim), dtype=dtype, device=self.device)
                blk.kv = torch.empty((c, 2, g.num_key_value_heads, g.head_dim), dtype=dtype, pin_memory=True)
                blk.kv_device_address = blk.kv.data_ptr()  # pinned by the CUDA allocator: same address under UVA

    def begin_blocks(self, docs: List[Document], dtype: Optional[torch.dtype] = None):
        self.block_desc.init_docs(docs, self.device)
        self._kv_offset = 0
        self._init_block_data(dtype or self.geometry.dtype)

    def ingest_meta(self, meta: dict):
        """Store one stage-1 block.  ``meta`` is the PREFILL_WORKER_META payload
        (src/prefill.py:152-157, 300-303); its cache answers ``get_kvcache`` /
        ``get_router_kcache`` with ``[1, Hkv, c, D]`` tensors.  Body of the receive loop at
        src/msa_service.py:519-571."""
        cache = meta["past_key_values"]
        if not self.template_prefix_kvcache:
            kw = cache.cache_kwargs
            self.template_prefix_kvcache = {
                layer: (kw[layer]["template_prefix_kcache"].to(self.device),
                        kw[layer]["template_prefix_vcache"].to(self.device))
                for layer in kw if "template_prefix_kcache" in kw[layer]}
        n = None
        chunk_major = hasattr(cache, "kv_chunk_major")     # a SharedPooledCache: already in the bank's layouts
        for layer in self.router_layer_ids:
            blk = self.blocks[layer]
            if chunk_major:
                kv, rk = cache.kv_chunk_major(layer), cache.rk_chunk_major(layer)
                n = kv.shape[0] if n is None else n
                assert n == kv.shape[0] and self._kv_offset + n <= self.block_desc.chunks()
                sl = slice(self._kv_offset, self._kv_offset + n)
                blk.kv[sl].copy_(kv)
                blk.rk[sl].copy_(rk if rk is not None else kv[:, 0])
            else:
                k, v = cache.get_kvcache(layer)
                rk = cache.get_router_kcache(layer)
                if rk is None:
                    rk = k
                n = k.shape[2] if n is None else n
                assert n == k.shape[2] and self._kv_offset + n <= self.block_desc.chunks()
                sl = slice(self._kv_offset, self._kv_offset + n)
                blk.rk[sl].copy_(rk[0].permute(1, 0, 2), non_blocking=True)
                blk.kv[sl, 0].copy_(k[0].permute(1, 0, 2))
                blk.kv[sl, 1].copy_(v[0].permute(1, 0, 2))
            if layer == self.router_layer_ids[0]:
                self.block_desc.tmp_doc_ids.append(cache.cache_kwargs[layer]["pooled_doc_ids"])
        self._kv_offset += n or 0
        if hasattr(cache, "clear_kvcache"):
            cache.clear_kvcache()        # the receive loop's last step per block (:569); unlinks a shared block file

    def _start_worker(self):
        """Start this GPU's stage-1 worker process and wait until it has loaded its model (src/msa_service.py:323-337)."""
        import multiprocessing as mp
        from .prefill import PrefillStage1Worker
        ctx = mp.get_context("spawn")
        self._worker_req_q, self._worker_rsp_q = ctx.Queue(), ctx.Queue()
        template = getattr(self.generate_config, "template", None) or {"prompt": "<|im_start|>user\n{prompt}<|im_end|>\n"}
        envs = dict(getattr(self.model_config, "envs", None) or {})
        self._worker_process = ctx.Process(
            target=PrefillStage1Worker.prefill_worker_main,
            args=(self.gpu_id, self._worker_req_q, self._worker_rsp_q, self.model_config.model_path, template,
                  self.memory_config.pooling_kernel_size, self.memory_config.block_size, envs),
            name=f"PrefillStage1Worker-{self.gpu_id}")
        self._worker_process.start()
        PrefillStage1Worker.wait_for_ready(self._worker_rsp_q)

    def _stop_worker(self):
        from .prefill import PrefillStage1Worker
        PrefillStage1Worker.close_worker(self._worker_req_q)
        self._worker_process.join()
        self._worker_process = None
        self._worker_req_q = self._worker_rsp_q = None

    def _worker_metas(self, docs: List[Document]):
        """The receive loop of the reference's ``generate_blocks`` (:511-523): send the documents, yield META
        payloads until every document has come back."""
        from .prefill import PrefillStage1Worker
        PrefillStage1Worker.send_documents(self._worker_req_q, docs)
        recv = 0
        while recv < len(docs):
            meta = PrefillStage1Worker.recv_meta(self._worker_rsp_q)
            recv += meta["nr_docs"]
            yield meta

    def generate_blocks(self, docs: List[Document], metas: Optional[Iterable[dict]] = None):
        """``Memory.generate_blocks`` (src/msa_service.py:497-582).  Without ``metas`` the stage-1 results are pulled
        from this GPU's ``PrefillStage1Worker`` process, as in the reference; ``metas`` (an iterable of META payloads)
        feeds a bank from a worker the caller drives itself."""
        data_path = os.environ.get("MEMORY_DATA_PATH", "")
        if data_path:   # same convention as the reference: $MEMORY_DATA_PATH/gpu<world>/<gpu_id> (:498-505)
            world = getattr(self, "world_size", None) or getattr(self.generate_config, "world", 1) or 1
            data_path = os.path.join(data_path, f"gpu{world}", str(self.gpu_id))
            if os.path.exists(os.path.join(data_path, "meta.json")):
                out = self.deserialize(data_path)
                assert len(docs) == self.block_desc.nr_docs
                return out
            if is_reference_bank(data_path):
                # the reference would load this directory (it loads whenever the directory exists, :503-505);
                # rebuilding silently next to its files would hide that the formats differ
                raise A.MsaError(
                    f"{data_path} holds a bank in the reference's format (stub.json / meta.pt / layer_*_k.pt), which "
                    "this package does not read in place: convert it once with "
                    "msa_b200.memory.convert_reference_bank(src_dir, dst_dir) or point MEMORY_DATA_PATH elsewhere")
        own_worker = metas is None and bool(self.model_config.model_path)
        if own_worker:
            self._start_worker()
            metas = self._worker_metas(docs)
        self.begin_blocks(docs)
        try:
            for meta in metas or ():
                self.ingest_meta(meta)
        finally:
            if own_worker:
                self._stop_worker()
        self.block_desc.merge_poolig_doc_id(self.device)
        if data_path:
            self.serialize(data_path)
        return self._post_process()

    def load_pooled(self, docs: List[Document], layers: Dict[int, Tuple[torch.Tensor, torch.Tensor, torch.Tensor]]):
        """Fill the bank from already pooled tensors: ``layers[l] = (k, v, rk)`` each ``[C, Hkv, D]``."""
        first = next(iter(layers.values()))
        self.begin_blocks(docs, first[2].dtype)
        for layer, (k, v, rk) in layers.items():
            blk = self.blocks[layer]
            blk.rk.copy_(rk)
            blk.kv[:, 0].copy_(k)
            blk.kv[:, 1].copy_(v)
        self.block_desc.pool_ids_from_docs(self.device)
        return self._post_process()

    # ------------------------------------------------------------------ on-disk bank
    def serialize(self, path: str):
        """Write the shard under ``path`` (counterpart of ``Memory.serialize``, src/msa_service.py:351-420,
        which stores one ``.pt`` per layer and tensor).  Format: ``meta.json`` (documents, geometry, dtype),
        ``prefix_cache.pt`` (template prefix K/V per layer) and, per router layer, two raw little-endian
        files in exactly the in-memory layouts: ``rk_L<l>.bin`` ``[C, Hkv, D]`` and ``kv_L<l>.bin``
        ``[C, 2, Hkv, D]``.  Raw files can be mapped and pinned in place on load."""
        os.makedirs(path, exist_ok=True)
        g = self.geometry
        first = self.blocks[self.router_layer_ids[0]]
        first_rk = first.get_router_k()
        meta = {"format": "msa_b200-bank-1", "dtype": str(first_rk.dtype).replace("torch.", ""),
                "n_chunks": int(first_rk.shape[0]), "n_kv_heads": g.num_key_value_heads, "head_dim": g.head_dim,
                "router_layer_ids": list(self.router_layer_ids),
                "doc_ids": [d.doc_id for d in self.block_desc.docs],
                "doc_chunks": [d.num_chunks for d in self.block_desc.docs]}
        torch.cuda.synchronize(self.device)
        for layer in self.router_layer_ids:
            blk = self.blocks[layer]
            blk.get_router_k().cpu().contiguous().view(torch.uint8).numpy().tofile(os.path.join(path, f"rk_L{layer}.bin"))
            blk.kv.contiguous().view(torch.uint8).numpy().tofile(os.path.join(path, f"kv_L{layer}.bin"))
        torch.save({l: (k.cpu(), v.cpu()) for l, (k, v) in self.template_prefix_kvcache.items()},
                   os.path.join(path, "prefix_cache.pt"))
        with open(os.path.join(path, "meta.json"), "w") as f:   # written last: its presence marks a complete bank
            json.dump(meta, f)

    def deserialize(self, path: str, map_host_bank: bool = True):
        """Load a shard written by ``serialize`` (src/msa_service.py:422-479).  Router keys go to the GPU.
        The K/V bank is not copied: with ``map_host_bank`` its file is memory-mapped and the mapping is
        pinned and made device-visible (``msa_bank_register_host``), so the first fetch of a document
        pulls it from the page cache; if the file system does not allow pinning its pages (the driver
        refuses ext4 mappings, accepts tmpfs ones) or ``map_host_bank`` is false, the bank is read into
        pinned memory instead.  ``self.bank_placement`` says which happened."""
        with open(os.path.join(path, "meta.json")) as f:
            meta = json.load(f)
        if meta.get("format") != "msa_b200-bank-1":
            raise A.MsaError(f"{path}: not an msa_b200 bank")
        dtype = getattr(torch, meta["dtype"])
        c, h, d = meta["n_chunks"], meta["n_kv_heads"], meta["head_dim"]
        if (h, d) != (self.geometry.num_key_value_heads, self.geometry.head_dim):
            raise A.MsaError(f"{path}: bank geometry {h}x{d} does not match the model")
        if sorted(meta["router_layer_ids"]) != list(self.router_layer_ids):
            raise A.MsaError(f"{path}: bank holds layers {meta['router_layer_ids']}, model routes in {self.router_layer_ids}")
        docs = [Document(doc_id=i, num_chunks=n) for i, n in zip(meta["doc_ids"], meta["doc_chunks"])]
        self.block_desc.init_docs(docs, self.device)
        self.block_desc.pool_ids_from_docs(self.device)
        esize = torch.empty((), dtype=dtype).element_size()
        self._mapped_banks = []
        for layer in self.router_layer_ids:
            blk = self.blocks[layer]
            n_rk, n_kv = c * h * d * esize, c * 2 * h * d * esize
            raw = torch.from_file(os.path.join(path, f"rk_L{layer}.bin"), shared=False, size=max(n_rk, 1), dtype=torch.uint8)
            blk.rk = raw[:n_rk].view(dtype).view(c, h, d).to(self.device)
            kv_path = os.path.join(path, f"kv_L{layer}.bin")
            mapped_ok = False
            if map_host_bank and n_kv > 0:
                import ctypes
                mapped = torch.from_file(kv_path, shared=True, size=n_kv, dtype=torch.uint8)
                addr = ctypes.c_uint64(0)
                rc = A.lib().msa_bank_register_host(mapped.data_ptr(), n_kv, ctypes.byref(addr))
                if rc == 0:   # tmpfs / hugetlbfs mappings can be pinned in place; most disk file systems cannot
                    blk.kv, blk.kv_device_address = mapped.view(dtype).view(c, 2, h, d), int(addr.value)
                    self._mapped_banks.append(mapped)
                    mapped_ok = True
                else:
                    del mapped
            if not mapped_ok:
                raw = torch.from_file(kv_path, shared=False, size=max(n_kv, 1), dtype=torch.uint8)
                blk.kv = raw[:n_kv].view(dtype).view(c, 2, h, d).pin_memory()
                blk.kv_device_address = blk.kv.data_ptr()
            self.bank_placement = "mapped in place" if mapped_ok else "copied to pinned memory"
        prefix = torch.load(os.path.join(path, "prefix_cache.pt"))
        self.template_prefix_kvcache = {int(l): (k.to(self.device), v.to(self.device)) for l, (k, v) in prefix.items()}
        return self._post_process()

    def release_mapped_banks(self):
        """Unpin the file mappings taken by ``deserialize`` (call before the process drops the bank)."""
        torch.cuda.synchronize(self.device)
        for m in getattr(self, "_mapped_banks", []):
            A.lib().msa_bank_unregister_host(m.data_ptr())
        self._mapped_banks = []

    def _post_process(self):
        first = self.blocks[self.router_layer_ids[0]]
        rk = first.rk if first.rk is not None else first.rk_blocked
        kv_bytes = rk.nbytes * len(self.router_layer_ids)
        return kv_bytes, (1, self.geometry.num_key_value_heads, self.block_desc.chunks(), self.geometry.head_dim)

    def block_router_keys(self, free_rows: bool = False):
        """Re-lay every router layer's keys in 128-chunk tiles (``ops.block_router_keys``): the bandwidth-bound
        routing of decode steps then streams them ~19 % faster from HBM, with identical results.  Call once after
        the bank is built.  ``free_rows`` drops the row-major copy layer by layer (a bank that fills most of HBM);
        every routing call then reads the blocked copy (prefill-shaped calls on the one-CTA tensor-core kernel)."""
        for layer in self.router_layer_ids:
            blk = self.blocks[layer]
            if blk.rk is None or blk.rk.dtype != torch.bfloat16 or blk.rk[0].numel() % 64 != 0:
                continue
            blk.n_chunks = blk.rk.shape[0]
            blk.rk_blocked = ops.block_router_keys(blk.rk)
            if free_rows:
                torch.cuda.current_stream(self.device).synchronize()
                blk.rk = None

    def get_max_local_pool_doc_id(self) -> int:
        return int(self.block_desc.pool_ids_cpu[-1])

    def get_template_prefix_kvcaches(self, layer_idx: int):
        return self.template_prefix_kvcache[layer_idx]

    # ------------------------------------------------------------------ scoring + selection
    def prepare_table(self, n_seq: int):
        """Reset the score table for ``n_seq`` sequences on a side stream, NOW, so that the reset overlaps whatever the
        caller issues next on the current stream (the fold kernel, the query all-gather); the next ``score_folded``
        call for ``n_seq`` sequences joins it.  A dependent launch costs a few microseconds even when the kernel is
        tiny, which matters for decode-time routing (a layer-step of ~90 us).  Fork and join both happen inside the
        routing call, so the pattern can be captured in a CUDA graph."""
        desc = self.block_desc
        tbl = self.__dict__.get("_table")
        if tbl is None or tbl.shape[0] != n_seq or tbl.shape[1] != desc.nr_docs + 1:
            tbl = self._table = torch.empty((n_seq, desc.nr_docs + 1), dtype=torch.int32, device=self.device)
        if "_side" not in self.__dict__:
            self._side = torch.cuda.Stream(self.device)
        main = torch.cuda.current_stream(self.device)
        fork = torch.cuda.Event()
        fork.record(main)
        self._side.wait_event(fork)
        dtype = next(b.rk if b.rk is not None else b.rk_blocked for b in self.blocks.values()).dtype
        with torch.cuda.stream(self._side):
            ops.route_table_reset(tbl, desc.nr_docs, torch.finfo(dtype).min)      # status is not touched from here
            done = torch.cuda.Event()
            done.record(self._side)
        self._table_ready = (n_seq, done)

    def _take_prepared_table(self, n_seq: int):
        ready = self.__dict__.pop("_table_ready", None)
        if ready is None:
            return None
        torch.cuda.current_stream(self.device).wait_event(ready[1])      # join, whatever happens next
        return self._table if ready[0] == n_seq else None

    def score_folded(self, layer_idx: int, q_folded, row_bias, n_seq: int, s_pad: int, n_heads: int, top_k: int,
                     scale: float = 1.0, out=None):
        """Score ``n_seq`` folded sequences (head_reduce "mean") against this shard and select ``top_k``
        documents each (``out``: see ``ops.topk_select``).  chunk_reduce "max" is one fused kernel; "mean"
        fills a per-chunk table with the same kernel (every chunk its own document) and reduces it."""
        desc = self.block_desc
        blk = self.blocks[layer_idx]
        use_blocked = blk.rk_blocked is not None and (blk.rk is None or s_pad == 1)   # bandwidth-bound shapes, or no rows left
        keys_src = blk.rk_blocked if use_blocked else blk.rk
        min_val = torch.finfo(keys_src.dtype).min
        if self.chunk_reduce_method == "max" and self.fused_decode_routing and \
                ops.route_score_select_supported(keys_src, n_seq, s_pad, top_k, use_blocked):
            # one token per sequence: scoring and per-CTA selection in one launch, no score table
            need = (n_seq, top_k)
            ws = self.__dict__.get("_select_ws")
            if ws is None or ws[0] != need:
                n_bytes = int(A.lib().msa_route_score_select_workspace_bytes(n_seq, top_k))
                ws = self._select_ws = (need, torch.empty((max(n_bytes, 8) + 7) // 8, dtype=torch.int64, device=self.device))
            self._take_prepared_table(n_seq)      # joins a table reset that a caller may have started
            return ops.route_score_select(q_folded, row_bias, n_seq, keys_src, desc.chunk_doc, desc.nr_docs, scale / n_heads,
                                          top_k, desc.doc_ids, min_val, self._status, ws[1], out, blocked=use_blocked)
        prepared = self._take_prepared_table(n_seq)
        if self.chunk_reduce_method == "max":
            keys, _ = ops.route_scores(q_folded, row_bias, n_seq, s_pad, keys_src, desc.chunk_doc, desc.nr_docs,
                                       alpha=scale / n_heads, min_val=min_val, status=self._status, blocked=use_blocked,
                                       keys=prepared, flags=A.ROUTE_NO_INIT if prepared is not None else 0)
        else:
            c = desc.chunk_doc.numel()
            ident = self.__dict__.get("_identity_ids")
            if ident is None or ident.numel() != c:
                ident = self._identity_ids = torch.arange(1, c + 1, dtype=torch.int32, device=self.device)
            chunk_keys, _ = ops.route_scores(q_folded, row_bias, n_seq, s_pad, keys_src, ident, c, alpha=scale / n_heads,
                                             min_val=min_val, status=self._status, blocked=use_blocked)
            keys = ops.route_reduce_chunks(chunk_keys, desc.chunk_doc, desc.nr_docs, "mean", min_val, status=self._status)
        return self._select(keys, n_seq, top_k, out)

    def score_unfolded(self, layer_idx: int, query_states, query_mask, top_k: int, scale: float = 1.0, out=None):
        """head_reduce "max": the heads cannot be folded, so the unfolded queries ``[B, Hq, S, D]`` are scored per
        head (``ops.route_chunk_scores``) and the chunk table is reduced to documents."""
        desc = self.block_desc
        blk = self.blocks[layer_idx]
        rk = blk.get_router_k()
        min_val = torch.finfo(rk.dtype).min
        self._status.zero_()
        chunk_keys = ops.route_chunk_scores(query_states, query_mask, self.num_key_value_groups, rk,
                                            self.head_reduce_method, self.query_reduce_method, scale, min_val)
        keys = ops.route_reduce_chunks(chunk_keys, desc.chunk_doc, desc.nr_docs, self.chunk_reduce_method, min_val,
                                       status=self._status)
        return self._select(keys, query_states.shape[0], top_k, out)

    def _select(self, keys, n_seq: int, top_k: int, out=None):
        desc = self.block_desc
        need = ops.topk_workspace_bytes(n_seq, desc.nr_docs + 1, top_k)
        ws = getattr(self, "_topk_ws", None)
        if need and (ws is None or ws.numel() * 8 < need):
            ws = self._topk_ws = torch.empty((need + 7) // 8, dtype=torch.int64, device=self.device)
        return ops.topk_select(keys, top_k, desc.doc_ids, workspace=ws if need else None, out=out)

    def prefill_stage2(self, layer_idx: int, query_states: torch.Tensor, query_mask: torch.Tensor):
        """src/msa_service.py:703-828.  query_states ``[B, Hkv, G, S, D]``, query_mask
        ``[B, 1, 1, S, 1]`` bool.  Returns ``(scores[B,k'], local_ids[B,k'], global_ids[B,k'])``,
        ``k' = min(doc_top_k, nr_docs + 1)``; scores are float32."""
        b, hkv, grp, s, d = query_states.shape
        q = query_states.reshape(b, hkv * grp, s, d)
        if self.head_reduce_method == "max":
            return self.score_unfolded(layer_idx, q, query_mask.reshape(b, s), self.model_config.doc_top_k)
        qf, bias, s_pad = ops.fold_queries(q, query_mask.reshape(b, s), grp, query_reduce=self.query_reduce_method)
        return self.score_folded(layer_idx, qf, bias, b, s_pad, hkv * grp, self.model_config.doc_top_k)

    @staticmethod
    def _raise_on_status(st):
        if st[0] != 0:
            raise A.MsaError(f"routing kernel gave up on a barrier wait (code {st[0]}): the score table is incomplete")
        if st[2] != 0:
            raise A.MsaError(f"{st[2]} out-of-range index(es) were skipped on the device (chunk -> document ids outside "
                             "1..nr_docs, or winners outside the directory): bank tables and directory disagree")

    def check_status(self):
        """Raise if a kernel reported a barrier wait that ran out or an index outside its table (reads 16
        bytes back).  ``MSAService.fetch`` / ``doc_query`` check the same words in the read-back they make anyway."""
        self._raise_on_status(self._status.cpu().tolist())

"""Stage-1 worker: encodes blocks of memory documents and ships their pooled K / V / K_r to the service
(mirror of ``src/prefill.py``: ``BlockModelInput`` :22-29, the ``PREFILL_WORKER_*`` tags :31-35,
``PrefillStage1Worker`` :37-305, and of ``ProtocolConstants``, src/types.py:11-21).

Same process protocol as the reference: the service starts ``PrefillStage1Worker.prefill_worker_main`` in its own
process with a request and a response queue; messages are ``(tag, payload)`` tuples; the worker answers READY,
waits for MEMORY_DOCS (the documents of its GPU), cuts them into blocks of at most ``block_size`` chunks
(``split_docs``), runs stage 1 on each block and answers one META per block, then waits for CLOSE.  A META payload
has the reference's keys: ``chunk_sizes, past_key_values, nr_docs, doc_ids, nr_chunks``.

What differs: ``past_key_values`` is not the CPU cache itself, pickled tensor by tensor through the queue, but a
``SharedPooledCache``: the pooled tensors are written once, already in the bank's chunk-major layouts, into a
shared-memory file that the service maps and copies from (``Memory.ingest_meta``).  The model is this package's
decoder stack (``msa_b200.model``) unless ``envs["MSA_B200_MODEL_FACTORY"] = "module:function"`` names another
``function(model_path, device) -> (model, tokenizer)``; the model's ``.model(...)`` call takes the reference's
keyword arguments.
"""
from __future__ import annotations

import importlib
import itertools
import os
from dataclasses import dataclass
from typing import Dict, List

import torch

from .cache import SharedPooledCache, SparseCacheOnCPU
from .memory import Document
from .tools import compose_input

PREFILL_WORKER_READY = "PREFILL_WORKER_READY"
PREFILL_WORKER_CLOSE = "PREFILL_WORKER_CLOSE"
PREFILL_WORKER_MEMORY_DOCS = "PREFILL_WORKER_MEMORY_DOCS"
PREFILL_WORKER_NUM_CHUNKS_REPORT = "PREFILL_WORKER_NUM_CHUNKS_REPORT"
PREFILL_WORKER_META = "PREFILL_WORKER_META"


class ProtocolConstants:
    """``(tag, payload)`` messages on a queue (src/types.py:11-21)."""

    @staticmethod
    def expect(q, constant):
        k, v = q.get()
        assert k == constant, f"expect {constant} but got {k}"
        return v

    @staticmethod
    def send(q, constant, data=None, block=True):
        q.put((constant, data), block=block)


@dataclass
class BlockModelInput:
    doc_input_ids: torch.Tensor
    doc_attention_mask: torch.Tensor
    doc_ids: torch.Tensor
    position_ids: torch.Tensor
    num_chunks: int
    chunk_sizes: List[int]


def default_model_factory(model_path: str, device):
    """Tokenizer and decoder stack from a checkpoint directory in the reference's format (``config.json`` with an
    ``msa_config`` entry, safetensors weights)."""
    import glob
    import json

    from safetensors.torch import load_file
    from transformers import AutoTokenizer

    from .configuration import MSAConfig
    from .model import MSAForCausalLM
    tokenizer = AutoTokenizer.from_pretrained(model_path)
    with open(os.path.join(model_path, "config.json")) as f:
        raw = json.load(f)
    config = MSAConfig(**{k: v for k, v in raw.items() if k not in ("architectures", "model_type", "auto_map")})
    model = MSAForCausalLM(config).to(torch.bfloat16)
    state = {}
    for shard in sorted(glob.glob(os.path.join(model_path, "*.safetensors"))):
        state.update(load_file(shard))
    missing, unexpected = model.load_state_dict(state, strict=False)
    if missing:
        raise RuntimeError(f"{model_path}: checkpoint lacks {missing[:5]} ...")
    return model.to(device).eval(), tokenizer


class PrefillStage1Worker:
    _file_counter = itertools.count()

    def __init__(self, gpu_id: int, model_path: str, template: dict, pooling_kernel_size: int, envs: dict):
        self.gpu_id = gpu_id
        for k, v in (envs or {}).items():        # src/utils/gpu_worker.py:12-15
            os.environ[k] = v
        if torch.cuda.is_available():
            torch.cuda.set_device(gpu_id)
            self.device = f"cuda:{gpu_id}"
        else:                                    # a host-only factory (tests) still runs the protocol
            self.device = "cpu"
        self.model_path = model_path
        self.pooling_kernel_size = pooling_kernel_size
        factory = os.environ.get("MSA_B200_MODEL_FACTORY", "")
        if factory:
            mod, fn = factory.split(":")
            self.model, self.tokenizer = getattr(importlib.import_module(mod), fn)(model_path, self.device)
        else:
            self.model, self.tokenizer = default_model_factory(model_path, self.device)
        self.model_config = self.model.config
        ridx = self.model_config.msa_config.router_layer_idx
        self.router_layer_ids = (list(range(self.model_config.num_hidden_layers)) if ridx == "all"
                                 else sorted(int(i) for i in str(ridx).split(",")))
        self.template_id = -2
        self._prepare_template(template)

    def num_model_layers(self):
        return self.model_config.num_hidden_layers

    # ------------------------------------------------------------------ protocol (static, as in the reference)
    @staticmethod
    def split_docs(docs: List[Document], block_size: int):
        """Greedy blocks of at most ``block_size`` chunks; a document larger than that is a block of its own
        (src/prefill.py:75-91)."""
        sub_blocks, curr_block, sz = [], [], 0
        for doc in docs:
            chunks = doc.num_chunks
            if sz + chunks > block_size and curr_block:
                sub_blocks.append(curr_block)
                sz, curr_block = 0, []
            curr_block.append(doc)
            sz += chunks
        if curr_block:
            sub_blocks.append(curr_block)
        return sub_blocks

    @staticmethod
    def wait_for_ready(q):
        ProtocolConstants.expect(q, PREFILL_WORKER_READY)

    @staticmethod
    def close_worker(q):
        ProtocolConstants.send(q, PREFILL_WORKER_CLOSE, block=True)

    @staticmethod
    def send_documents(q, docs):
        ProtocolConstants.send(q, PREFILL_WORKER_MEMORY_DOCS, data=docs, block=False)

    @staticmethod
    def recv_meta(q):
        return ProtocolConstants.expect(q, PREFILL_WORKER_META)

    @staticmethod
    def prefill_worker_main(gpu_id: int, request_queue, response_queue, model_path: str, template: Dict,
                            pooling_kernel_size: int, block_size: int, envs):
        """Process entry point (src/prefill.py:112-140).  An error while encoding is printed and the worker still
        waits for CLOSE, as the reference does; the service then sees fewer documents than it sent."""
        worker = PrefillStage1Worker(gpu_id, model_path, template, pooling_kernel_size, envs)
        ProtocolConstants.send(response_queue, PREFILL_WORKER_READY, block=False)
        docs: List[Document] = ProtocolConstants.expect(request_queue, PREFILL_WORKER_MEMORY_DOCS)
        try:
            for block in PrefillStage1Worker.split_docs(docs, block_size):
                ProtocolConstants.send(response_queue, PREFILL_WORKER_META, data=worker.inference(block), block=False)
        except Exception as e:
            print(f"[prefill worker {gpu_id}] error: {e}")
            import traceback
            traceback.print_exc()
        ProtocolConstants.expect(request_queue, PREFILL_WORKER_CLOSE)

    # ------------------------------------------------------------------ one block
    def inference(self, block: List[Document]):
        kv_meta = self._inference(self._prepare_block_inputs(block))
        kv_meta["nr_docs"] = len(block)
        kv_meta["doc_ids"] = [item.doc_id for item in block]
        kv_meta["nr_chunks"] = [item.num_chunks for item in block]
        return kv_meta

    def _prepare_template(self, template: Dict):
        """Token ids of the prompt template before and after the ``{prompt}`` slot (src/prefill.py:159-186)."""
        self.pad_token = self.tokenizer.pad_token
        self.pad_token_id = self.tokenizer.pad_token_id
        prompt_template = template["prompt"].replace("{prompt}", self.pad_token)
        inputs = self.tokenizer(prompt_template, add_special_tokens=False)
        ids, mask = list(inputs["input_ids"]), list(inputs["attention_mask"])
        self.pad_index = ids.index(self.pad_token_id)
        self.template_head_input_ids, self.template_head_attention_mask = ids[:self.pad_index], mask[:self.pad_index]
        self.template_tail_input_ids, self.template_tail_attention_mask = ids[self.pad_index + 1:], mask[self.pad_index + 1:]

    def _prepare_block_inputs(self, block: List[Document]) -> BlockModelInput:
        """One row: template head (doc id -2, positions 0..), then every document as ``compose_input`` writes it,
        with doc id = 1-based index INSIDE the block and positions restarting at 0 per document
        (src/prefill.py:188-246)."""
        doc_ids = [self.template_id] * len(self.template_head_input_ids)
        input_ids = list(self.template_head_input_ids)
        attention_mask = list(self.template_head_attention_mask)
        position_ids = list(range(self.pad_index))
        chunk_sizes = []
        for doc_idx, item in enumerate(block):
            _, doc_inputs = compose_input(item.doc, item.doc_id, self.tokenizer)
            ids = list(doc_inputs["input_ids"])
            chunk_size = (len(ids) + self.pooling_kernel_size - 1) // self.pooling_kernel_size
            assert chunk_size == item.num_chunks, \
                f"pre calculated chunk {item.num_chunks} got {chunk_size} for document {item.doc_id} ({len(ids)} tokens)"
            chunk_sizes.append(chunk_size)
            doc_ids.extend([doc_idx + 1] * len(ids))
            input_ids.extend(ids)
            attention_mask.extend(doc_inputs["attention_mask"])
            position_ids.extend(range(len(ids)))
        return BlockModelInput(doc_input_ids=torch.LongTensor([input_ids]), doc_attention_mask=torch.LongTensor([attention_mask]),
                               doc_ids=torch.LongTensor([doc_ids]), position_ids=torch.LongTensor([position_ids]),
                               num_chunks=sum(chunk_sizes), chunk_sizes=chunk_sizes)

    def _inference(self, model_input: BlockModelInput) -> Dict:
        """Stage 1 of the whole stack on one block (src/prefill.py:248-305); the pooled tensors end up in a
        shared-memory file (see ``SharedPooledCache``)."""
        dev = self.device
        cache = SparseCacheOnCPU()
        for layer_idx in range(self.num_model_layers()):
            cache.record_kwargs(layer_idx, {"stage": "prefill_stage1"})
        with torch.no_grad():
            outputs = self.model.model(
                input_ids=model_input.doc_input_ids.to(dev), attention_mask=model_input.doc_attention_mask.to(dev),
                position_ids=model_input.position_ids.to(dev), past_key_values=cache, use_cache=True,
                output_attentions=False, output_hidden_states=False, output_docs_score=False,
                doc_ids=model_input.doc_ids.to(dev))
        cache = outputs.past_key_values
        status = cache.meta.get("_msa_b200_attn_status")
        if status is not None and int(status[0].item()) != 0:      # the last layer's launch is checked here, at block end
            raise RuntimeError("a bounded barrier wait ran out inside the stage-1 attention kernel: block output invalid")
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
        shm_dir = os.environ.get("MSA_B200_SHM_DIR", "/dev/shm")
        path = os.path.join(shm_dir, f"msa_b200_stage1_{os.getpid()}_{next(self._file_counter)}.blk")
        shared = SharedPooledCache.write(path, cache, self.router_layer_ids)
        return {"chunk_sizes": model_input.chunk_sizes, "past_key_values": shared}

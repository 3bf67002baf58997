"""Engine front end: the parent process that owns the memory documents and the per-GPU service processes
(mirror of ``MSAEngine``, src/msa_service.py:1368-1906, its message types :37-169, ``MSAService.generate`` :1316-1364
and ``GenerateConfig``, src/config/memory_config.py:6-26).

    engine = MSAEngine(generate_config, model_config, memory_config)
    texts, recall_topk, userdata = engine.generate(["question", ...])

The parent tokenises the memory file once to count chunks, deals the documents over the GPUs (least loaded bucket
first), starts one ``service_main`` process per GPU and hands each its bucket; a ``generate`` call templates the
prompts, pads the batch to a multiple of the world size, left-pads every GPU's share, sends one ``GenerateRequest``
per GPU, and a receiver thread merges the ``GenerateResponse``s in GPU order and calls back.  Message names, tuple
protocol, dataclass fields and the arithmetic of the request preparation are the reference's (pinned by
``tests/golden/front_end.json``).

Each service process builds its shard with this package's stage-1 worker and bank, loads the decoder stack, and
answers requests with the Memory-Interleave loop (``msa_b200.generate``).  Tokenizer and model come from a factory
``(model_path, device) -> (model, tokenizer)`` (``msa_b200.prefill.default_model_factory`` unless
``model_config.envs["MSA_B200_MODEL_FACTORY"] = "module:function"`` names another); ``MSAEngine(...,
service_main=...)`` swaps the whole service process (the tests run the protocol with a text-only stand-in).
"""
from __future__ import annotations

import importlib
import json
import multiprocessing as mp
import os
import pickle
import queue
import threading
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Union

import torch

from .memory import Document, MemoryConfig, ModelConfig
from .prefill import ProtocolConstants
from .tools import RequestLimiter, compose_input

MEMORY_WORKER_READY = "MEMORY_WORKER_READY"
MEMORY_WORKER_CLOSE = "MEMORY_WORKER_CLOSE"
MEMORY_WORKER_BLOCKS = "MEMORY_WORKER_BLOCKS"
MEMORY_WORKER_IDX_TO_DOC = "MEMORY_WORKER_IDX_TO_DOC"

QWEN3_TEMPLATE = {"prompt": "<|im_start|>user\n{prompt}<|im_end|>\n"}
QWEN3_INSTRUCT_TEMPLATE = QWEN3_TEMPLATE
QUESTION_HEAD = "\nPlease answer the question based on the above historical document information\n\n"
QUESTION_TAIL = "Please return all documents related to the question"


@dataclass
class GenerateConfig:
    devices: Optional[List[int]] = None
    template: Union[str, Dict, None] = None
    max_generate_tokens: int = 256
    max_seq_len: int = 0          # total sequence length in a batch
    max_query_seq_len: int = 0    # longest single query
    max_batch_size: int = 0       # 0 = unlimited
    top_p: float = 0.9
    temperature: float = 0.0
    qa_mode: bool = False

    def __post_init__(self):
        if isinstance(self.template, str):
            assert self.template in ("QWEN3_TEMPLATE", "QWEN3_INSTRUCT_TEMPLATE")
            self.template = {"QWEN3_TEMPLATE": QWEN3_TEMPLATE, "QWEN3_INSTRUCT_TEMPLATE": QWEN3_INSTRUCT_TEMPLATE}[self.template]
        if self.template is None:
            self.template = QWEN3_TEMPLATE
        assert isinstance(self.template, dict)

    @property
    def world(self):
        return len(self.devices) if self.devices else 0


@dataclass
class CmdBase:
    name: str = ""


@dataclass
class GenerateRequest(CmdBase):
    """One user call becomes ``world`` of these, ``seq_id`` = position of the GPU's share in the batch."""
    msg_id: int = 0
    seq_id: int = 0
    input_ids: List[List[int]] = None
    attention_mask: List[List[int]] = None
    doc_ids: List[List[int]] = None
    positions: List[List[int]] = None
    require_recall_topk: bool = False
    prompts: List[str] = None

    def __post_init__(self):
        self.name = "generate_request"


@dataclass
class GenerateResponse:
    msg_id: int = -1
    seq_id: int = -1
    gpu_id: int = 0
    generated_texts: List[str] = None
    recall_topk: Optional[Dict[int, List]] = None


@dataclass
class ReportDocID:
    gpu_id: int = 0
    pooled_doc_id_bias: Any = 0
    name: str = "report_doc_id"


GenerateReceiver = Callable[[List[str], Any, Any], None]


@dataclass
class GenerateStub:
    msg_id: int = 0
    userdata: Any = None
    responses: List[GenerateResponse] = field(default_factory=list)
    nr_dummy: int = 0             # prompts appended to fill the last GPU's share
    callback: Optional[GenerateReceiver] = None

    def respond(self):
        """Texts in GPU order without the fill-ins, recall lists concatenated per layer (src/msa_service.py:150-169)."""
        if self.callback is None:
            return
        self.responses.sort(key=lambda r: r.seq_id)
        texts: List[str] = []
        recall_topk: Dict[int, List] = {}
        for rsp in self.responses:
            texts.extend(rsp.generated_texts)
            for layer, topks in (rsp.recall_topk or {}).items():
                recall_topk.setdefault(layer, []).extend(topks)
        self.callback(texts[:len(texts) - self.nr_dummy], recall_topk, self.userdata)


def _resolve_factory(envs: Optional[dict]):
    spec = (envs or {}).get("MSA_B200_MODEL_FACTORY") or os.environ.get("MSA_B200_MODEL_FACTORY", "")
    if spec:
        mod, fn = spec.split(":")
        return getattr(importlib.import_module(mod), fn)
    from .prefill import default_model_factory
    return default_model_factory


class MSAEngine:
    def __init__(self, generate_config: GenerateConfig, model_config: ModelConfig, memory_config: MemoryConfig,
                 service_main: Optional[Callable] = None, tokenizer=None, start: bool = True):
        if not generate_config.devices:
            # NCCL wants the global device numbering; select GPUs with CUDA_VISIBLE_DEVICES (src/msa_service.py:1376-1379)
            generate_config.devices = list(range(torch.cuda.device_count()))
        self.world_size = generate_config.world
        self.generate_config, self.model_config, self.memory_config = generate_config, model_config, memory_config
        self._service_main = service_main or MSAEngine.service_main
        self.tokenizer = tokenizer
        self.worker_processes: List[mp.Process] = []
        self.worker_qs: Dict[int, Any] = {}
        self._ctx = mp.get_context("spawn")          # CUDA in the children
        self.response_queue = self._ctx.Queue()
        self.request_queue = self._ctx.Queue()
        self.msg_id = 0
        self.limiter = RequestLimiter(4)
        self.requests: Dict[int, GenerateStub] = {}
        self.lock = threading.Lock()
        self.sync_event = threading.Event()
        self.sync_rsp = None
        self.running = False
        self.recv_rsp_thread = None
        if start:
            self.start_workers()
            self.initialize()

    # ------------------------------------------------------------------ start-up
    def initialize(self):
        if self.tokenizer is None:
            _, self.tokenizer = None, self._load_tokenizer()
        self._prepare_template()
        self._load_memory_file()
        self._wait_ready_signal()          # every service is up before the buckets are sent
        self._process_buckets()
        self.running = True                # the receiver starts only after the buckets are processed
        self.recv_rsp_thread = threading.Thread(target=self.receive_response, daemon=True)
        self.recv_rsp_thread.start()

    def _load_tokenizer(self):
        from transformers import AutoTokenizer
        return AutoTokenizer.from_pretrained(self.model_config.model_path)

    def start_workers(self):
        for gpu_id in self.generate_config.devices:
            q = self._ctx.Queue()
            p = self._ctx.Process(target=self._service_main, name=f"MSAService-{gpu_id}",
                                  args=(gpu_id, q, self.response_queue, self.generate_config, self.model_config,
                                        self.memory_config))
            p.start()
            self.worker_processes.append(p)
            self.worker_qs[gpu_id] = q

    def stop_workers(self):
        self.running = False
        for q in self.worker_qs.values():
            q.put(None)
        self.worker_qs = {}
        for p in self.worker_processes:
            p.join()
        self.worker_processes = []
        if self.recv_rsp_thread is not None:
            self.recv_rsp_thread.join()
            self.recv_rsp_thread = None

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc_val, exc_tb):
        self.stop_workers()
        return False

    def _next_response(self):
        """The next message of a service process; raises instead of waiting forever when one of them has died."""
        while True:
            try:
                return self.response_queue.get(timeout=1.0)
            except queue.Empty:
                dead = [p.name for p in self.worker_processes if not p.is_alive()]
                if dead:
                    raise RuntimeError(f"service process(es) {dead} exited during start-up")

    def _wait_ready_signal(self):
        for _ in range(len(self.worker_qs)):
            tag, _ = self._next_response()
            assert tag == MEMORY_WORKER_READY, f"expect {MEMORY_WORKER_READY} but got {tag}"

    def _worker_all_gather(self, cmdname: str):
        responses = []
        while len(responses) < len(self.worker_qs):
            rsp = self._next_response()
            assert rsp.name == cmdname, f"worker all gather got response {rsp.name} expect {cmdname}"
            responses.append(rsp)
        responses.sort(key=lambda r: r.gpu_id)
        return responses

    @staticmethod
    def balanced_bucket_partition(docs: List[Document], n_buckets: int) -> List[List[Document]]:
        """Every document goes to the bucket that holds the fewest chunks so far (src/msa_service.py:1451-1476)."""
        buckets: List[List[Document]] = [[] for _ in range(n_buckets)]
        load = [0] * n_buckets
        for doc in docs:
            b = load.index(min(load))
            buckets[b].append(doc)
            load[b] += doc.num_chunks
        return buckets

    def _sort_reference(self, docs: List[str]) -> List[List[Document]]:
        """Chunk counts from the tokenised documents as the stage-1 worker will write them (src/msa_service.py:1478-1500)."""
        pool = self.model_config.pooling_kernel_size
        documents = []
        for idx, doc in enumerate(docs):
            _, inputs = compose_input(doc, idx, self.tokenizer)
            documents.append(Document(doc=doc, doc_id=idx, num_chunks=(len(inputs["input_ids"]) + pool - 1) // pool))
        return MSAEngine.balanced_bucket_partition(documents, self.generate_config.world)

    def _load_memory_file(self):
        path = self.memory_config.memory_file_path
        if path.endswith(".json"):
            with open(path, "r") as f:
                context_list = json.load(f)
        elif path.endswith(".pkl"):
            with open(path, "rb") as f:
                context_list = list(pickle.load(f))
        else:
            raise ValueError(f"Unsupported file format: {path}")
        self.buckets = self._sort_reference(context_list)
        self.docs: List[Document] = [d for bucket in self.buckets for d in bucket]

    def get_idx_to_doc(self):
        return {doc.doc_id: doc.doc for doc in self.docs}

    def _process_buckets(self):
        idx_to_doc = self.get_idx_to_doc()
        for idx, gpu_id in enumerate(self.generate_config.devices):
            ProtocolConstants.send(self.worker_qs[gpu_id], MEMORY_WORKER_BLOCKS, data=self.buckets[idx], block=False)
            ProtocolConstants.send(self.worker_qs[gpu_id], MEMORY_WORKER_IDX_TO_DOC, data=idx_to_doc, block=False)
        self._worker_all_gather("report_doc_id")      # every shard is built and its model loaded

    # ------------------------------------------------------------------ request preparation
    def _prepare_template(self):
        """Token ids that follow every question: the template's tail and the response head (src/msa_service.py:1703-1721)."""
        head = self.tokenizer("<|im_start|>", add_special_tokens=False)
        pad_token, pad_token_id = self.tokenizer.pad_token, self.tokenizer.pad_token_id
        templ = self.tokenizer(self.generate_config.template["prompt"].replace("{prompt}", pad_token), add_special_tokens=False)
        cut = templ["input_ids"].index(pad_token_id)
        tail_ids, tail_mask = templ["input_ids"][cut + 1:], templ["attention_mask"][cut + 1:]
        self.prompt_tail_input_ids = tail_ids + head["input_ids"]
        self.prompt_tail_attention_mask = tail_mask + head["attention_mask"]
        self.tail_doc_ids = [-2] * len(tail_ids) + [-1] * len(head["input_ids"])

    def _apply_template(self, prompt: str):
        """Question tokens are routing-query tokens (doc id 0), the template tail -2, the response head -1."""
        question = QUESTION_HEAD + prompt + "\n" + QUESTION_TAIL + "\n"
        q = self.tokenizer(question, add_special_tokens=False)
        return (q["input_ids"] + self.prompt_tail_input_ids, q["attention_mask"] + self.prompt_tail_attention_mask,
                [0] * len(q["input_ids"]) + self.tail_doc_ids)

    def _apply_template_regenerate(self, prompt: str):
        """A continued round: the text after ``<regenerate>`` is fed as is; routing-query tokens are the question (up to
        and including the instruction line) and the last list of document numbers, the rest are response tokens
        (src/msa_service.py:1732-1772)."""
        question = prompt.split("<regenerate>")[1]
        q = self.tokenizer(question, add_special_tokens=False)
        n_tok = lambda text: len(self.tokenizer(text, add_special_tokens=False)["input_ids"])
        doc_ids = [-1] * len(q["input_ids"])
        marker = "]<|object_ref_end|>["
        last = question.rfind(marker)
        if last != -1:
            start = last + len(marker) - 1
            nxt = question.find("<|object_ref_end|>", start)
            if nxt != -1:
                first = n_tok(question[:start])
                for i in range(first, first + n_tok(question[start:nxt])):
                    if i < len(doc_ids):
                        doc_ids[i] = 0
        anchor = question.find(QUESTION_TAIL)
        if anchor != -1:
            for i in range(n_tok(question[:anchor + len(QUESTION_TAIL)])):
                if i < len(doc_ids):
                    doc_ids[i] = 0
        return q["input_ids"], q["attention_mask"], doc_ids

    def _validate_inputs(self, input_ids: List[List[int]]):
        if any(len(sub) == 0 for sub in input_ids):
            raise ValueError("empty query is not acceptable")
        # the reference sums the token ids here, not the lengths (src/msa_service.py:1692-1700); kept, limits default to 0 = off
        if self.generate_config.max_seq_len > 0:
            seqlen = sum(sum(sub) for sub in input_ids)
            if seqlen > self.generate_config.max_seq_len:
                raise ValueError(f"total sequence length {seqlen} exceeds limitation {self.generate_config.max_seq_len}")
        if self.generate_config.max_query_seq_len > 0:
            longest = max(sum(sub) for sub in input_ids)
            if longest > self.generate_config.max_query_seq_len:
                raise ValueError(f"max query sequence length {longest} exceeds limitation {self.generate_config.max_query_seq_len}")

    def prepare_requests(self, prompts: List[str], msg_id: int, require_recall_topk: bool = False):
        """``(requests per GPU, number of fill-in prompts)``: the host arithmetic of ``generate``
        (src/msa_service.py:1804-1899).  Positions start after the template and the retrieved slots
        (``3 + doc_top_k``) for every prompt; a GPU's share is left-padded to its own longest prompt, padding repeats
        the first position and has doc id 0 and mask 0."""
        world = self.generate_config.world
        bsz = (len(prompts) + world - 1) // world
        if self.generate_config.max_batch_size > 0 and bsz > self.generate_config.max_batch_size:
            raise ValueError(f"Batch size exceeds maximum allowed batch size {self.generate_config.max_batch_size}")
        pads = bsz * world - len(prompts)
        prompts = list(prompts) + [prompts[-1]] * pads
        first_position = 3 + self.model_config.doc_top_k
        rows = []
        for prompt in prompts:
            ids, mask, docs = (self._apply_template_regenerate if "<regenerate>" in prompt else self._apply_template)(prompt)
            rows.append((ids, mask, docs, [first_position + i for i in range(len(ids))]))
        pad_id = self.tokenizer.pad_token_id if self.tokenizer.pad_token_id else self.tokenizer.eos_token_id
        padded = []
        for i, (ids, mask, docs, pos) in enumerate(rows):
            if i % bsz == 0:
                width = max(len(r[0]) for r in rows[i:i + bsz])
            n = width - len(ids)
            padded.append(([pad_id] * n + ids, [0] * n + mask, [0] * n + docs, [pos[0]] * n + pos))
        self._validate_inputs([p[0] for p in padded][0:-1:bsz])
        requests = []
        for idx in range(world):
            share = padded[idx * bsz:(idx + 1) * bsz]
            requests.append(GenerateRequest(msg_id=msg_id, seq_id=idx, prompts=prompts[idx * bsz:(idx + 1) * bsz],
                                            input_ids=[s[0] for s in share], attention_mask=[s[1] for s in share],
                                            doc_ids=[s[2] for s in share], positions=[s[3] for s in share],
                                            require_recall_topk=require_recall_topk))
        return requests, pads

    # ------------------------------------------------------------------ requests and responses
    def default_callback(self, texts, recall_topk, userdata):
        self.sync_rsp = (texts, recall_topk, userdata)
        self.sync_event.set()

    def generate(self, prompts: Union[str, List[str]], userdata=None, require_recall_topk: bool = False,
                 callback: Optional[GenerateReceiver] = None):
        """Blocking without ``callback`` (returns ``(texts, recall_topk, userdata)``); with one, returns at once and
        the receiver thread calls ``callback(texts, recall_topk, userdata)``.  At most four requests are in flight."""
        if isinstance(prompts, str):
            prompts = [prompts]
        requests, pads = self.prepare_requests(prompts, self.msg_id + 1, require_recall_topk)
        self.limiter.acquire()
        sync = callback is None
        self.msg_id += 1
        with self.limiter.lock:
            self.requests[self.msg_id] = GenerateStub(msg_id=self.msg_id, userdata=userdata, nr_dummy=pads, responses=[],
                                                      callback=callback or self.default_callback)
        for req, gpu_id in zip(requests, self.generate_config.devices):
            self.worker_qs[gpu_id].put(req, block=False)
        if sync:
            self.sync_event.wait()
            self.sync_event.clear()
            return self.sync_rsp

    def receive_response(self):
        while self.running:
            try:
                rsp: GenerateResponse = self.response_queue.get(timeout=0.5)
            except queue.Empty:
                continue
            done = None
            with self.limiter.lock:
                assert rsp.msg_id in self.requests
                stub = self.requests[rsp.msg_id]
                stub.responses.append(rsp)
                if len(stub.responses) == self.world_size:
                    done = self.requests.pop(rsp.msg_id)
            if done is not None:
                self.limiter.release()
                done.respond()

    # ------------------------------------------------------------------ the per-GPU process
    @staticmethod
    def service_main(gpu_id: int, request_queue, response_queue, generate_config: GenerateConfig,
                     model_config: ModelConfig, memory_config: MemoryConfig):
        """One rank (src/msa_service.py:1590-1642): join the NCCL group, build the shard from the documents the parent
        sends, load the model, then answer requests until ``None`` arrives.  An error while answering is printed and
        the loop goes on, as in the reference."""
        import torch.distributed as dist

        from .memory import AttentionGeometry
        from .service import MSAService
        for k, v in (model_config.envs or {}).items():
            os.environ[k] = v
        world = generate_config.world
        torch.cuda.set_device(gpu_id)
        if world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29500")
            dist.init_process_group("nccl", rank=gpu_id, world_size=world, device_id=torch.device("cuda", gpu_id))
        model, tokenizer = _resolve_factory(model_config.envs)(model_config.model_path, f"cuda:{gpu_id}")
        cfg = model.config
        geometry = AttentionGeometry(
            num_hidden_layers=cfg.num_hidden_layers, num_attention_heads=cfg.num_attention_heads,
            num_key_value_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
            head_reduce_method=cfg.msa_config.head_reduce_method, query_reduce_method=cfg.msa_config.query_reduce_method,
            chunk_reduce_method=cfg.msa_config.chunk_reduce_method, aux_loss_method=cfg.msa_config.aux_loss_method,
            decouple_router=cfg.msa_config.decouple_router, dtype=next(model.parameters()).dtype)
        service = MSAService(gpu_id, generate_config, model_config, memory_config, geometry=geometry)
        ProtocolConstants.send(response_queue, MEMORY_WORKER_READY, block=False)
        docs: List[Document] = ProtocolConstants.expect(request_queue, MEMORY_WORKER_BLOCKS)
        idx_to_doc: Dict[int, str] = ProtocolConstants.expect(request_queue, MEMORY_WORKER_IDX_TO_DOC)
        service.generate_blocks(docs)
        if world > 1:
            service.share_host_banks(f"engine{os.getppid()}")
        else:
            service.publish_directory()
        service.setup_memory_client(model)
        response_queue.put(ReportDocID(gpu_id=gpu_id, pooled_doc_id_bias=service.block_desc.nr_docs), block=False)
        while True:
            cmd = request_queue.get()
            if cmd is None:
                if world > 1:
                    service.close_host_banks()
                    dist.destroy_process_group()
                return
            try:
                if cmd.name == "generate_request":
                    response_queue.put(service_generate(service, model, tokenizer, idx_to_doc, generate_config, cmd))
                else:
                    print(f"GPU_ID {gpu_id} recv unknown cmd {cmd.name}")
            except Exception as e:
                print(f"[subprocess {gpu_id}] error: {e}")
                import traceback
                traceback.print_exc()


def create_generate_args(generate_config: GenerateConfig) -> dict:
    """Sampling settings of a request (src/msa_service.py:1042-1054): greedy at temperature 0."""
    if generate_config.temperature == 0.0:
        return {"do_sample": False, "temperature": None, "top_p": None}
    return {"do_sample": True, "temperature": generate_config.temperature, "top_p": generate_config.top_p}


def service_generate(service, model, tokenizer, idx_to_doc, generate_config: GenerateConfig,
                     req: GenerateRequest) -> GenerateResponse:
    """One GPU's share of a request (``MSAService.generate``, src/msa_service.py:1316-1364): a fresh cache whose
    layers start in stage 2 of the prefill, the interleave loop, the decoded sequences and, if asked for, the
    documents every router layer recalled."""
    from .cache import create_cache
    from .generate import interleave_generate
    dev = service.device
    cache = create_cache()
    cache.meta.update({"require_recall_topk": req.require_recall_topk, "qa_mode": generate_config.qa_mode,
                       "max_generate_tokens": generate_config.max_generate_tokens, "tokenizer": tokenizer,
                       "idx_to_doc": idx_to_doc, "pattern": r"\[(\d+)\]",
                       "response_string": ["" for _ in range(len(req.input_ids))]})
    for layer_idx in range(model.config.num_hidden_layers):
        cache.record_kwargs(layer_idx, {"stage": "prefill_stage2"})
    eos = tokenizer.eos_token_id
    sequences = interleave_generate(
        model, torch.LongTensor(req.input_ids).to(dev), torch.LongTensor(req.attention_mask).to(dev),
        torch.LongTensor(req.doc_ids).to(dev), torch.LongTensor(req.positions).to(dev), cache,
        eos_token_ids=[eos] if isinstance(eos, int) else list(eos or []),
        pad_token_id=tokenizer.pad_token_id if tokenizer.pad_token_id is not None else 0, **create_generate_args(generate_config))
    texts = tokenizer.batch_decode(sequences, skip_special_token=True)
    # the entries travel to the parent through a process queue: host tensors, not handles to this process's memory
    to_host = lambda v: v.detach().cpu() if torch.is_tensor(v) else v
    recall = ({layer: [{k: to_host(v) for k, v in entry.items()} for entry in args["recall_topk"]]
               for layer, args in cache.cache_kwargs.items() if "recall_topk" in args} if req.require_recall_topk else None)
    return GenerateResponse(msg_id=req.msg_id, seq_id=req.seq_id, gpu_id=service.gpu_id, generated_texts=texts,
                            recall_topk=recall)

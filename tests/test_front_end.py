"""Engine front end and Memory-Interleave loop against what the reference's own code produced for the same inputs
(tests/golden/front_end.json, recorded by tests/golden/make_golden.py::gen_front_end with the tokenizer and the
scripted model of tests/fake_text.py), plus the parent <-> service process protocol with a text-only service."""
import json
import os
import threading

import pytest
import torch

from msa_b200.engine import GenerateConfig, GenerateResponse, GenerateStub, MSAEngine
from msa_b200.generate import interleave_generate
from msa_b200.memory import MemoryConfig, ModelConfig
from tests import fake_text as F

HERE = os.path.dirname(os.path.abspath(__file__))
with open(os.path.join(HERE, "golden", "front_end.json")) as f:
    GOLD = json.load(f)


def engine(world, top_k):
    return_engine = MSAEngine(GenerateConfig(devices=list(range(world)), template=F.TEMPLATE), ModelConfig(doc_top_k=top_k),
                              MemoryConfig(), tokenizer=F.CharTokenizer(), start=False)
    return_engine._prepare_template()
    return return_engine


@pytest.mark.parametrize("case", GOLD["requests"], ids=lambda c: f"world{c['world']}_n{len(c['prompts'])}")
def test_request_preparation_matches_reference(case):
    e = engine(case["world"], case["top_k"])
    assert e.prompt_tail_input_ids == case["tail_input_ids"] and e.tail_doc_ids == case["tail_doc_ids"]
    reqs, pads = e.prepare_requests(list(case["prompts"]), msg_id=1, require_recall_topk=True)
    assert pads == case["nr_dummy"] and len(reqs) == case["world"]
    for mine, ref in zip(reqs, case["per_gpu"]):
        for key in ("msg_id", "seq_id", "prompts", "input_ids", "attention_mask", "doc_ids", "positions", "require_recall_topk"):
            assert getattr(mine, key) == ref[key], key
        assert mine.name == "generate_request"


def test_request_limits():
    e = engine(2, 16)
    with pytest.raises(ValueError):
        e._validate_inputs([[1, 2], []])
    e.generate_config.max_batch_size = 1
    with pytest.raises(ValueError):
        e.prepare_requests(["a", "b", "c"], 1)


def test_respond_merges_in_gpu_order():
    got = {}
    stub = GenerateStub(msg_id=7, userdata="ud", nr_dummy=1, responses=[], callback=lambda t, r, u: got.update(t=t, r=r, u=u))
    stub.responses.append(GenerateResponse(msg_id=7, seq_id=1, gpu_id=1, generated_texts=["c", "d"], recall_topk={18: [{"x": 3}]}))
    stub.responses.append(GenerateResponse(msg_id=7, seq_id=0, gpu_id=0, generated_texts=["a", "b"],
                                           recall_topk={18: [{"x": 1}], 19: [{"x": 2}]}))
    stub.respond()
    assert got["t"] == GOLD["respond"]["texts"] and got["u"] == GOLD["respond"]["userdata"]
    assert {str(k): v for k, v in got["r"].items()} == GOLD["respond"]["recall"]


@pytest.mark.parametrize("case", GOLD["interleave"], ids=lambda c: c["name"])
def test_interleave_loop_matches_reference_call_by_call(case):
    tok = F.CharTokenizer()
    e = engine(1, 16)
    (req,), _ = e.prepare_requests(list(case["prompts"]), 1)
    lm = F.ScriptedLM(case["scripts"], tok)
    cache = F.StubCache()
    cache.meta.update({"require_recall_topk": False, "qa_mode": True, "max_generate_tokens": 64, "tokenizer": tok,
                       "idx_to_doc": F.IDX_TO_DOC, "pattern": r"\[(\d+)\]", "response_string": ["" for _ in case["prompts"]]})
    for layer in range(lm.config.num_hidden_layers):
        cache.record_kwargs(layer, {"stage": "prefill_stage2"})
    seqs = interleave_generate(lm, torch.LongTensor(req.input_ids), torch.LongTensor(req.attention_mask),
                               torch.LongTensor(req.doc_ids), torch.LongTensor(req.positions), cache,
                               eos_token_ids=[tok.eos_token_id], pad_token_id=tok.pad_token_id)
    assert len(lm.calls) == len(case["calls"])
    for i, (mine, ref) in enumerate(zip(lm.calls, case["calls"])):
        for key in ("input_ids", "attention_mask", "position_ids", "doc_ids"):
            assert mine[key].tolist() == ref[key], (i, key)
        assert mine["stages"] == ref["stages"], i
    assert seqs.tolist() == case["sequences"]
    assert cache.meta["response_string"] == case["response_string"]


def test_sampling_path_runs_and_respects_top_p():
    from msa_b200.generate import _process_logits
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0]])
    kept = torch.isfinite(_process_logits(logits, 1.0, 0.7))
    assert kept.tolist() == [[True, True, False, False]]          # 0.64 + 0.24 >= 0.7
    assert torch.isfinite(_process_logits(logits, 0.5, None)).all()


def test_engine_processes_speak_the_protocol(tmp_path):
    """Parent and two service processes (text-only stand-ins): buckets by least-loaded chunk count, requests split
    per GPU, responses merged in GPU order without the fill-in prompt, the callback path and the blocking path."""
    from tests import fake_engine_worker
    docs = ["d%d " % i * (3 + 5 * (i % 4)) for i in range(9)]
    mem = tmp_path / "memory.json"
    mem.write_text(json.dumps(docs))
    cfg = GenerateConfig(devices=[0, 1], template=F.TEMPLATE)
    with MSAEngine(cfg, ModelConfig(doc_top_k=16, pooling_kernel_size=4), MemoryConfig(memory_file_path=str(mem)),
                   service_main=fake_engine_worker.service_main, tokenizer=F.CharTokenizer()) as e:
        loads = [sum(d.num_chunks for d in b) for b in e.buckets]
        assert sum(len(b) for b in e.buckets) == 9 and abs(loads[0] - loads[1]) <= max(d.num_chunks for d in e.docs)
        texts, recall, userdata = e.generate(["one", "two", "three"], userdata=5, require_recall_topk=True)
        assert userdata == 5 and len(texts) == 3                      # the fourth (fill-in) answer is dropped
        assert [t.split("|")[0] for t in texts] == ["gpu0", "gpu0", "gpu1"]
        assert [t.split("|")[4] for t in texts] == ["one", "two", "three"]
        assert all(t.split("|")[3] == "known9" for t in texts)
        assert [r["topk_doc_ids"] for r in recall[18]] == [[0], [0], [1], [1]]
        done = threading.Event()
        got = {}
        e.generate("solo", callback=lambda t, r, u: (got.update(t=t), done.set()))
        assert done.wait(30) and len(got["t"]) == 1 and got["t"][0].startswith("gpu0|")

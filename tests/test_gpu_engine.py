"""The whole front-to-back path on one GPU: engine parent -> service process -> stage-1 worker process -> bank ->
decoder stack with routing, host fetch and sparse attention -> Memory-Interleave loop -> merged response.  The model
is a tiny seeded stack (tests/fake_text.py::factory), so the text is meaningless; what is checked is that every
process speaks the protocol, that the bank the service built holds the documents the parent counted, that the
router layer recalled documents of that bank for every prompt, and that the same request gives the same answer."""
import json

import pytest
import torch

from msa_b200.engine import GenerateConfig, MSAEngine
from msa_b200.memory import MemoryConfig, ModelConfig
from tests import fake_text as F

pytestmark = pytest.mark.gpu


@pytest.mark.timeout(420)
def test_engine_end_to_end_on_one_gpu(tmp_path):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    docs = [f"document {i} is about topic {i % 7}; " * (5 + i % 6) for i in range(14)]
    mem = tmp_path / "memory.json"
    mem.write_text(json.dumps(docs))
    envs = {"MSA_B200_MODEL_FACTORY": "tests.fake_text:factory"}
    gen_cfg = GenerateConfig(devices=[0], template=F.TEMPLATE, max_generate_tokens=10, temperature=0.0)
    model_cfg = ModelConfig(model_path="unused-by-the-factory", doc_top_k=2, pooling_kernel_size=64, router_layer_idx="1", envs=envs)
    with MSAEngine(gen_cfg, model_cfg, MemoryConfig(block_size=64, memory_file_path=str(mem)), tokenizer=F.CharTokenizer()) as e:
        assert len(e.docs) == 14 and all(d.num_chunks >= 1 for d in e.docs)
        prompts = ["what is topic 3 about?", "name a document"]
        texts, recall, userdata = e.generate(prompts, userdata="tag", require_recall_topk=True)
        assert userdata == "tag" and len(texts) == 2 and all(isinstance(t, str) and t for t in texts)
        assert set(recall) == {1} and len(recall[1]) == 2               # the router layer, one entry per prompt
        for entry in recall[1]:
            ids = [int(i) for i in entry["topk_doc_ids"].tolist()] if torch.is_tensor(entry["topk_doc_ids"]) else list(entry["topk_doc_ids"])
            assert len(ids) == 2 and all(0 <= i < 14 for i in ids)
        again, _, _ = e.generate(prompts)
        assert again == texts                                             # greedy decoding is reproducible

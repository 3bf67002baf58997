"""A character-level tokenizer and a scripted language model for the front-end tests (engine request preparation and
the Memory-Interleave generation loop).  Both the fixture generator (which drives the reference's own code with them)
and the tests (which drive this package's code with them) import this file, so the two sides see identical inputs.

Tokenizer: the chat markers and the two control strings of the interleave loop are single tokens, every other
character is one token (id = 16 + code point, capped), pad = 0.
Model: emits, for sample i at its c-th forward call, the token ``script[i][c]`` as a one-hot logit row (EOS once the
script is exhausted), and logs what it was called with.
"""
from types import SimpleNamespace

import torch

SPECIALS = ["<pad>", "<|im_start|>", "<|im_end|>", "<|object_ref_end|>", "<End-of-Retrieve>", "<eos>"]
VOCAB = 16 + 256


class CharTokenizer:
    pad_token, pad_token_id = "<pad>", 0
    eos_token, eos_token_id = "<eos>", 5

    def encode(self, text):
        ids, i = [], 0
        while i < len(text):
            for t, s in enumerate(SPECIALS):
                if text.startswith(s, i):
                    ids.append(t)
                    i += len(s)
                    break
            else:
                ids.append(16 + min(ord(text[i]), 255))
                i += 1
        return ids

    def decode_one(self, tok):
        tok = int(tok)
        return SPECIALS[tok] if tok < len(SPECIALS) else (chr(tok - 16) if tok >= 16 else "")

    def __call__(self, text, add_special_tokens=False, padding=None, truncation=None, return_tensors=None,
                 padding_side="right", **unused):
        if isinstance(text, str):
            ids = self.encode(text)
            return {"input_ids": ids, "attention_mask": [1] * len(ids)}
        rows = [self.encode(t) for t in text]
        width = max(len(r) for r in rows)
        ids, mask = [], []
        for r in rows:
            pad = [self.pad_token_id] * (width - len(r))
            ids.append(pad + r if padding_side == "left" else r + pad)
            mask.append([0] * len(pad) + [1] * len(r) if padding_side == "left" else [1] * len(r) + [0] * len(pad))
        return {"input_ids": torch.tensor(ids, dtype=torch.long), "attention_mask": torch.tensor(mask, dtype=torch.long)}

    def batch_decode(self, ids, **unused):
        ids = torch.as_tensor(ids)
        if ids.dim() == 1:
            return [self.decode_one(t) for t in ids.tolist()]
        return ["".join(self.decode_one(t) for t in row) for row in ids.tolist()]


class ScriptedLM:
    """``forward`` of a causal LM whose next token is scripted per sample and per call."""

    def __init__(self, scripts, tokenizer, num_hidden_layers=2):
        self.scripts = [tokenizer.encode(s) if isinstance(s, str) else list(s) for s in scripts]
        self.tok = tokenizer
        self.config = SimpleNamespace(is_encoder_decoder=False, num_hidden_layers=num_hidden_layers)
        self.calls = []

    def forward(self, input_ids=None, attention_mask=None, position_ids=None, doc_ids=None, past_key_values=None, **kw):
        c = len(self.calls)
        stages = sorted({v.get("stage") for v in past_key_values.cache_kwargs.values()}) if past_key_values is not None else []
        self.calls.append({"input_ids": input_ids.clone(), "attention_mask": attention_mask.clone(),
                           "position_ids": position_ids.clone(), "doc_ids": doc_ids.clone(), "stages": stages})
        b = input_ids.shape[0]
        logits = torch.full((b, input_ids.shape[1], VOCAB), -10.0)
        for i in range(b):
            tok = self.scripts[i][c] if c < len(self.scripts[i]) else self.tok.eos_token_id
            logits[i, -1, tok] = 10.0
        return SimpleNamespace(logits=logits, past_key_values=past_key_values)

    __call__ = forward


class StubCache:
    """The cache duck type the loop touches: ``meta``, ``cache_kwargs``, ``record_kwargs``."""

    def __init__(self):
        self.meta, self.cache_kwargs = {}, {}

    def record_kwargs(self, layer_idx, kwargs):
        self.cache_kwargs.setdefault(layer_idx, {}).update(kwargs)


QUESTION_HEAD = "\nPlease answer the question based on the above historical document information\n\n"
QUESTION_TAIL = "\nPlease return all documents related to the question\n"
TEMPLATE = {"prompt": "<|im_start|>user\n{prompt}<|im_end|>\n"}
IDX_TO_DOC = {1: "alpha doc", 3: "gamma doc", 12: "twelfth doc", 40: "fortieth"}

# (name, prompts, per-sample scripts: the text the model emits, one token per forward call; '#' marks a call whose
# output the loop discards, blanks keep a sample that has finished its part from emitting EOS early)
INTERLEAVE_CASES = [
    ("ids_then_round_end", ["who wrote alpha?", "what is twelve"],
     ["[3]<|object_ref_end|>      ", "[12][1]<|object_ref_end|>  "]),
    ("end_of_retrieve_then_answer", ["q one", "second q"],
     ["<End-of-Retrieve>#yes<eos>", "<End-of-Retrieve>#no.<eos>"]),
    ("mixed_lengths", ["a", "a much longer question than the first one"],
     ["[1]<|object_ref_end|>            ", "[40][3][99]<|object_ref_end|>  "]),
    ("one_ends_retrieval_other_lists", ["first", "second"],
     ["<End-of-Retrieve>        ", "[3]<|object_ref_end|>   "]),
    ("malformed_list", ["x", "y"],
     ["[3]oops<|object_ref_end|>   ", "[1]<|object_ref_end|>        "]),
]


def factory(model_path, device):
    """``MSA_B200_MODEL_FACTORY`` target for the engine's end-to-end test: a tiny seeded decoder stack of this package
    (2 layers, router layer 1, head_dim 128, chunk 64) with the character tokenizer above."""
    from msa_b200.configuration import MSAConfig
    from msa_b200.model import MSAForCausalLM
    cfg = MSAConfig(
        msa_config=dict(router_layer_idx="1", aux_loss=False, aux_loss_method="INFONCE", decouple_router=True,
                        top_k_docs=2, pooling_kernel_size=64, head_reduce_method="mean", query_reduce_method="max",
                        chunk_reduce_method="max", decouple_pooling_mode="mean"),
        hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=128, num_hidden_layers=2,
        intermediate_size=128, vocab_size=VOCAB, max_position_embeddings=8192)
    cfg._attn_implementation = "eager"
    torch.manual_seed(4321)
    model = MSAForCausalLM(cfg).to(torch.bfloat16).to(device).eval()
    return model, CharTokenizer()

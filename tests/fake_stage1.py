"""Model factories for the stage-1 worker tests (``MSA_B200_MODEL_FACTORY = "tests.fake_stage1:factory"``).

``factory(model_path, device)`` returns ``(model, tokenizer)``:
  * on a CUDA device: a tiny, seeded ``msa_b200.model.MSAForCausalLM`` (2 layers, router layer 1, head_dim 128), i.e.
    the real stage-1 path on this package's kernels;
  * on the CPU: a stand-in whose ``.model(...)`` fills the cache with chunk means of token-derived states computed in
    plain torch, enough to exercise the worker protocol and the shared-memory transfer without a GPU.
The tokenizer is byte level: one id per character (+ 3), ``<|im_start|>`` / ``<|im_end|>`` as single ids, pad = 0.
"""
from types import SimpleNamespace

import torch

HKV, D, POOL = 2, 128, 4
SPECIAL = {"<|im_start|>": 1, "<|im_end|>": 2}


class ByteTokenizer:
    pad_token, pad_token_id = "\x00", 0

    def __call__(self, text, add_special_tokens=False):
        ids, i = [], 0
        while i < len(text):
            for s, t in SPECIAL.items():
                if text.startswith(s, i):
                    ids.append(t)
                    i += len(s)
                    break
            else:
                ids.append(0 if text[i] == self.pad_token else 3 + (ord(text[i]) % 250))
                i += 1
        return {"input_ids": ids, "attention_mask": [1] * len(ids)}


def config(device_is_cuda: bool):
    from msa_b200.configuration import MSAConfig
    cfg = MSAConfig(
        msa_config=dict(router_layer_idx="1", aux_loss=False, aux_loss_method="INFONCE", decouple_router=True,
                        top_k_docs=2, pooling_kernel_size=POOL if not device_is_cuda else 64, head_reduce_method="mean",
                        query_reduce_method="max", chunk_reduce_method="max", decouple_pooling_mode="mean"),
        hidden_size=64, num_attention_heads=4, num_key_value_heads=HKV, head_dim=D, num_hidden_layers=2,
        intermediate_size=128, vocab_size=256, max_position_embeddings=4096)
    cfg._attn_implementation = "eager"
    return cfg


def token_states(input_ids, salt):
    """Deterministic [1, HKV, T, D] fp32 states from token ids and positions."""
    t = input_ids.shape[1]
    base = (input_ids[0].float().view(1, t, 1) * 0.37 + torch.arange(t).view(1, t, 1) * 0.011 + salt)
    grid = torch.arange(HKV * D).view(1, 1, HKV * D).float() * 0.05
    return torch.sin(base + grid).view(1, t, HKV, D).permute(0, 2, 1, 3).contiguous()


class CpuStandIn:
    """Fills the cache like a 2-layer model whose layer 1 routes: pooled K / V / K_r per chunk of POOL tokens."""

    def __init__(self):
        self.config = config(False)
        self.model = self._forward

    def _forward(self, input_ids=None, attention_mask=None, position_ids=None, past_key_values=None, doc_ids=None, **kw):
        from oracle import msa_oracle as O
        cache = past_key_values
        doc_indices, gci, pooled_doc_ids, lengths = O.chunk_bookkeeping(doc_ids, attention_mask, POOL)
        n_t = int((doc_ids == -2).sum())
        for layer in range(2):
            k, v, rk = (token_states(input_ids, 10 * layer + j) for j in range(3))
            kw_l = {"template_prefix_kcache": k[:, :, :n_t], "template_prefix_vcache": v[:, :, :n_t]}
            if layer == 1:
                pk, pv = O.sequence_pooling_kv(k, v, doc_indices, gci)
                prk = O.pool_chunks_cumsum(rk[doc_indices[:, 0], :, doc_indices[:, 1]], lengths)
                to_ref = lambda x: x.transpose(0, 1).unsqueeze(0)
                cache.update(to_ref(pk), to_ref(pv), layer)
                cache.update_router_kcache(O.l2_normalize(to_ref(prk)), layer)
                kw_l.update({"doc_id_bias": doc_ids.shape[1], "pooled_doc_ids": pooled_doc_ids,
                             "prefill_stage1_kvcache_size": pk.shape[0]})
            cache.record_kwargs(layer, kw_l)
        return SimpleNamespace(last_hidden_state=None, past_key_values=cache)


def gpu_model(device):
    from msa_b200.model import MSAForCausalLM
    torch.manual_seed(1234)
    return MSAForCausalLM(config(True)).to(torch.bfloat16).to(device).eval()


def factory(model_path, device):
    if str(device).startswith("cuda"):
        return gpu_model(device), ByteTokenizer()
    return CpuStandIn(), ByteTokenizer()

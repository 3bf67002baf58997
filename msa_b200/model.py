"""Decoder stack around ``MemorySparseAttention`` for inference (mirror of ``src/msa/model.py``:
``MSADeocoderLayer`` :53-135, ``MSAModel`` :137-262, ``MSAForCausalLM`` :264-330).

Only what the stage-1 worker and the generation loop call: embeddings, N pre-norm decoder layers whose attention
is this package's ``MemorySparseAttention`` (``doc_ids`` handed down to every layer), final norm, ``lm_head``.
Module and parameter names follow the reference (``model.embed_tokens``, ``model.layers.<i>.self_attn.*``,
``model.layers.<i>.mlp.*``, ``model.norm``, ``lm_head``), so a reference checkpoint's state dict loads with
``load_state_dict``.  MLP, RMSNorm and rotary embedding are transformers' Qwen3 modules, as in the reference.
The training losses of the reference's ``MSAForCausalLM.forward`` are out of scope.
"""
from __future__ import annotations

from types import SimpleNamespace

import torch
import torch.nn as nn
from transformers.models.qwen3.modeling_qwen3 import Qwen3MLP, Qwen3RMSNorm, Qwen3RotaryEmbedding

from .attention import MemorySparseAttention
from .cache import create_cache


class MSADecoderLayer(nn.Module):
    def __init__(self, config, layer_idx: int):
        super().__init__()
        self.layer_idx = layer_idx
        self.self_attn = MemorySparseAttention(config=config, layer_idx=layer_idx)
        self.mlp = Qwen3MLP(config)
        self.input_layernorm = Qwen3RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.post_attention_layernorm = Qwen3RMSNorm(config.hidden_size, eps=config.rms_norm_eps)

    def forward(self, hidden_states, attention_mask=None, past_key_value=None, position_embeddings=None, doc_ids=None):
        attn, _ = self.self_attn(self.input_layernorm(hidden_states), doc_ids, attention_mask=attention_mask,
                                 position_embeddings=position_embeddings, past_key_value=past_key_value)
        hidden_states = hidden_states + attn
        return hidden_states + self.mlp(self.post_attention_layernorm(hidden_states))


class MSAModel(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.config = config
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size, getattr(config, "pad_token_id", None))
        self.layers = nn.ModuleList([MSADecoderLayer(config, i) for i in range(config.num_hidden_layers)])
        self.norm = Qwen3RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.rotary_emb = Qwen3RotaryEmbedding(config=config)

    def forward(self, input_ids=None, attention_mask=None, position_ids=None, past_key_values=None, inputs_embeds=None,
                use_cache=True, doc_ids=None, **unused):
        """Same call as the reference's ``MSAModel.forward`` (the flags it only forwards to outputs are accepted and
        ignored).  ``past_key_values`` must carry the stage of every layer (``cache_kwargs[layer]["stage"]``)."""
        if (input_ids is None) == (inputs_embeds is None):
            raise ValueError("You must specify exactly one of input_ids or inputs_embeds")
        hidden = self.embed_tokens(input_ids) if inputs_embeds is None else inputs_embeds
        if past_key_values is None:
            past_key_values = create_cache()
        if position_ids is None:
            position_ids = torch.arange(hidden.shape[1], device=hidden.device).unsqueeze(0)
        position_embeddings = self.rotary_emb(hidden, position_ids)
        for layer in self.layers:
            hidden = layer(hidden, attention_mask=attention_mask, past_key_value=past_key_values,
                           position_embeddings=position_embeddings, doc_ids=doc_ids)
        return SimpleNamespace(last_hidden_state=self.norm(hidden), past_key_values=past_key_values if use_cache else None)


class MSAForCausalLM(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.config = config
        self.model = MSAModel(config)
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)

    def forward(self, input_ids=None, attention_mask=None, position_ids=None, past_key_values=None, doc_ids=None,
                use_cache=True, logits_to_keep: int = 0, **unused):
        out = self.model(input_ids=input_ids, attention_mask=attention_mask, position_ids=position_ids,
                         past_key_values=past_key_values, use_cache=use_cache, doc_ids=doc_ids)
        hidden = out.last_hidden_state[:, -logits_to_keep:] if logits_to_keep else out.last_hidden_state
        return SimpleNamespace(logits=self.lm_head(hidden), past_key_values=out.past_key_values)

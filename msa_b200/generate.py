"""The Memory-Interleave generation loop (mirror of ``MSAGenerationMixin._sample``, src/msa/generate.py:23-354).

One call is one retrieval round of a batch of questions.  The model first lists document numbers
(``[3][12]<|object_ref_end|>``); when every live sample has closed its list, the loop looks the numbers up in
``idx_to_doc``, tokenises the documents' text and appends it to the context as one multi-token segment (the layer
sees it as routing-query tokens, ``doc_ids == 0``) -- the round ends there and the caller continues with a
``<regenerate>`` prompt.  A sample that answers ``<End-of-Retrieve>`` stops listing; when all have, the question is
restated once and the answer is decoded until EOS.  Samples that wait for the others are fed with attention mask 0
and keep their position.  The stage of every layer is switched to ``"generate"`` after the first (prefill) call.

What differs from the reference: this is a plain function over ``model(**inputs) -> .logits`` instead of an override
inside transformers' ``GenerationMixin`` (whose private helpers changed between releases); the per-sample string
bookkeeping, the stage machine and the tensors handed to the model are the same, call by call (pinned by
``tests/golden/front_end.json``, which was recorded from the reference's own loop).
"""
from __future__ import annotations

import re
from typing import Optional, Sequence

import torch
import torch.nn.functional as F

END_OF_LIST = "<|object_ref_end|>"
END_OF_RETRIEVE = "<End-of-Retrieve>"
MAX_RETRIEVAL_CHARS = 1000           # src/msa/generate.py:311
_ID_PREFIX = r"^\[\d*\]?$"           # a document number that is still being written (src/msa/generate.py:306)


def _question_of(text: str) -> str:
    """The user's question inside a templated prompt (src/msa/generate.py:188-189)."""
    q = text.split("historical document information\n\n")[-1]
    return q.split("\nPlease return all documents related to the question")[0]


def _process_logits(logits: torch.Tensor, temperature: Optional[float], top_p: Optional[float]) -> torch.Tensor:
    """Temperature, then nucleus filtering (what transformers' warpers do for ``do_sample=True``)."""
    if temperature is not None and temperature > 0 and temperature != 1.0:
        logits = logits / temperature
    if top_p is not None and 0.0 < top_p < 1.0:
        sorted_logits, order = torch.sort(logits, descending=False, dim=-1)
        cum = sorted_logits.softmax(dim=-1).cumsum(dim=-1)
        remove = cum <= (1.0 - top_p)
        remove[..., -1:] = False
        logits = logits.masked_fill(remove.scatter(-1, order, remove), float("-inf"))
    return logits


@torch.no_grad()
def interleave_generate(model, input_ids: torch.Tensor, attention_mask: torch.Tensor, doc_ids: torch.Tensor,
                        position_ids: torch.Tensor, past_key_values, *, eos_token_ids: Sequence[int], pad_token_id: int,
                        do_sample: bool = False, temperature: Optional[float] = None, top_p: Optional[float] = None,
                        generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """Runs the loop and returns every token the model was fed, ``[B, total]``, masked positions sorted to the left
    (what the reference's ``generate`` returns).  ``past_key_values.meta`` carries ``max_generate_tokens``,
    ``tokenizer``, ``response_string`` (updated in place), ``idx_to_doc`` and ``pattern``, as the reference's service
    sets them (src/msa_service.py:1324-1333)."""
    meta = past_key_values.meta
    max_generate_tokens = meta["max_generate_tokens"]
    tokenizer, response_string = meta["tokenizer"], meta["response_string"]
    idx_to_doc, pattern = meta["idx_to_doc"], meta["pattern"]
    dev = input_ids.device
    bsz = input_ids.shape[0]
    eos = torch.as_tensor(list(eos_token_ids), dtype=torch.long, device=dev)
    n_layers = model.config.num_hidden_layers

    # per-sample state lives on the host: every step needs the new tokens there anyway (to decode them into text),
    # so the flags cost no extra synchronisation and no swarm of one-element device kernels
    unfinished = torch.ones(bsz, dtype=torch.long)
    retrieval_end = torch.zeros(bsz, dtype=torch.bool)                  # the sample said <End-of-Retrieve>
    round_end = torch.zeros(bsz, dtype=torch.bool)                      # the sample closed its list of this round
    inner = [""] * bsz                                                  # text since the last appended context
    all_input_str = [""] * bsz
    last_valid = input_ids[:, -1:].clone()
    eos_host = eos.cpu()
    kw = {"attention_mask": attention_mask, "doc_ids": doc_ids, "position_ids": position_ids}
    hist = {}
    pos = None
    source_copied = has_stage3 = round_over = finished = False
    is_first = is_prefill = True
    step_all_valid = False          # the first call is the prefill
    stage, cnt = 1, 0

    while not finished:
        pos = kw.pop("position_ids") if "position_ids" in kw else (pos[:, -1:] + kw["attention_mask"]).to(dev)
        step_ids = input_ids if is_first else last_valid
        am = kw["attention_mask"]
        for i, s in enumerate(tokenizer.batch_decode(step_ids)):
            all_input_str[i] += s
        if not is_prefill:
            for layer_idx in range(n_layers):
                past_key_values.record_kwargs(layer_idx, {"stage": "generate"})
        # everything the model is fed, in order (src/msa/generate.py:124-133)
        if not hist:
            hist = {"doc_ids": kw["doc_ids"].clone(), "attention_mask": am.clone(), "input_ids": step_ids.clone(),
                    "position_ids": pos.clone()}
        else:
            hist["doc_ids"] = torch.cat((hist["doc_ids"], kw["doc_ids"][:, -am.shape[1]:]), dim=1)
            hist["attention_mask"] = torch.cat((hist["attention_mask"], am), dim=1)
            hist["input_ids"] = torch.cat((hist["input_ids"], step_ids), dim=1)
            hist["position_ids"] = torch.cat((hist["position_ids"], pos), dim=1)
        if round_over:
            break

        # lets a decode branch pick its single-token kernel without looking at the mask on the device
        meta["step_all_valid"] = step_all_valid
        out = model(input_ids=step_ids, attention_mask=am, position_ids=pos, doc_ids=kw["doc_ids"],
                    past_key_values=past_key_values, use_cache=True)
        is_prefill = is_first = False
        kw["attention_mask"] = torch.cat([am, am.new_ones((bsz, 1))], dim=-1)
        scores = out.logits[:, -1, :].to(dtype=torch.float32, device=dev)
        if do_sample:
            probs = F.softmax(_process_logits(scores, temperature, top_p), dim=-1)
            next_tokens = torch.multinomial(probs, num_samples=1, generator=generator).squeeze(1)
        else:
            next_tokens = torch.argmax(scores, dim=-1)
        next_tokens = next_tokens.cpu()
        if eos.numel():
            next_tokens = next_tokens * unfinished + pad_token_id * (1 - unfinished)
        new_text = tokenizer.batch_decode(next_tokens)

        if stage in (2, 3):
            # this call's token is dropped; the next input is a block of context text per sample
            sources = []
            if stage == 2:
                for i, listed in enumerate(inner):
                    if END_OF_RETRIEVE in listed:
                        sources.append("<|im_start|>" + "The user's question is: %s\n%s" % (_question_of(all_input_str[i]), END_OF_LIST))
                    else:
                        ids = sorted(set(map(int, re.findall(pattern, listed))))
                        ids = [k for k in ids if k in idx_to_doc]
                        sources.append("".join(f"[{k}]. {idx_to_doc[k]}\n" for k in ids) + END_OF_LIST)
            else:
                for i, said in enumerate(response_string):
                    sources.append("<|im_start|>" + "The user's question is: %s\n%s" % (_question_of(all_input_str[i]), END_OF_LIST)
                                   if END_OF_RETRIEVE in said else "")
            batch = tokenizer(sources, padding="longest", truncation=True, return_tensors="pt", add_special_tokens=True,
                              padding_side="left")
            src_ids = batch["input_ids"].clone().detach().long().to(dev)
            src_mask = batch["attention_mask"].clone().detach().long().to(dev)
            width = src_ids.shape[1]
            src_pos = torch.arange(width, dtype=torch.long, device=dev).unsqueeze(0).expand(bsz, -1)
            src_pos = src_pos + pos + src_mask.sum(dim=1, keepdim=True) - width + 1      # continues after this step's position
            input_ids = src_ids
            kw["attention_mask"], kw["doc_ids"], kw["position_ids"] = src_mask, torch.zeros_like(src_ids), src_pos
            source_copied, finished, is_first = True, False, True
            step_all_valid = False                                  # a multi-token, left-padded segment
            inner = [""] * bsz
            if stage == 2:
                round_over, stage = True, 1
            else:
                stage = 4
            round_end = torch.zeros(bsz, dtype=torch.bool)
        else:
            if eos.numel():
                unfinished = unfinished & ~torch.isin(next_tokens, eos_host)
            finished = bool(unfinished.max() == 0)
            input_ids = next_tokens[:, None].to(dev)
            kw["doc_ids"] = F.pad(kw["doc_ids"], (0, 1), value=-1)
            step_mask = torch.ones(bsz, 1, dtype=torch.long)
            if stage == 1:
                waiting = retrieval_end | round_end               # waits for the others: fed nothing, keeps its position
                step_mask[waiting, 0] = 0
                last_valid = torch.where(waiting.to(dev).unsqueeze(1), last_valid, input_ids)
            else:
                last_valid = input_ids.clone()
            step_all_valid = bool(step_mask.min() == 1)
            kw["attention_mask"] = step_mask.to(dev)
            for i in range(bsz):
                response_string[i] += new_text[i]
                inner[i] += new_text[i]
                round_end[i] |= END_OF_LIST in inner[i]
                retrieval_end[i] |= END_OF_RETRIEVE in response_string[i]
                if source_copied and stage == 1:
                    is_id = bool(re.fullmatch(_ID_PREFIX, inner[i]))
                    is_eor = inner[i] == END_OF_RETRIEVE[:len(inner[i])]
                    round_end[i] |= (not is_id and not is_eor)
                if not source_copied:
                    retrieval_end[i] |= len(response_string[i]) > MAX_RETRIEVAL_CHARS
            live = unfinished * (~retrieval_end)
            if int((round_end * live).sum()) == int(live.sum()) and not has_stage3:
                stage = 2
                for i in range(bsz):
                    if source_copied and round_end[i]:
                        if END_OF_LIST not in inner[i] or not re.fullmatch(_ID_PREFIX, inner[i].split(END_OF_LIST)[0]):
                            retrieval_end[i] = True
            if int((retrieval_end * unfinished).sum()) == int(unfinished.sum()) and not has_stage3:
                stage, has_stage3 = 3, True
        cnt += 1
        if cnt > max_generate_tokens:
            break

    mask, order = hist["attention_mask"].sort(dim=1, descending=False, stable=True)
    return hist["input_ids"].gather(dim=1, index=order)

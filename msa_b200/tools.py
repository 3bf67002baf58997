"""Small host-side helpers shared by the stage-1 worker and the engine front end (mirrors of
``src/utils/tools.py``: ``compose_input`` :101-104, ``RequestLimiter`` :59-99, ``cumulative_concat`` :34-55)."""
from __future__ import annotations

import threading

import torch


def compose_input(doc: str, doc_idx: int, tokenizer):
    """How a memory document is written into a block: ``<|im_start|>[i]. text[i]<|im_end|>`` (src/utils/tools.py:101-104).
    Returns ``(text, tokenizer output)``."""
    new_doc = "<|im_start|>" + f"[{doc_idx}]. {doc}[{doc_idx}]<|im_end|>"
    return new_doc, tokenizer(new_doc, add_special_tokens=False)


def cumulative_concat(tensors):
    """Concatenate per-block id lists that each count from 1 into ids that keep counting across blocks."""
    out, base = [], 0
    for t in tensors:
        out.append(t + base)
        base += int(t[-1])
    return torch.cat(out) if out else torch.empty(0, dtype=torch.long)


class RequestLimiter:
    """At most ``max_concurrent`` requests in flight; ``acquire`` blocks, ``release`` wakes one waiter."""

    def __init__(self, max_concurrent: int = 10):
        self.max_concurrent = max_concurrent
        self.current_count = 0
        self.lock = threading.Lock()
        self.condition = threading.Condition(self.lock)

    def acquire(self) -> bool:
        with self.lock:
            while self.current_count >= self.max_concurrent:
                self.condition.wait()
            self.current_count += 1
            return True

    def release(self) -> None:
        with self.lock:
            if self.current_count > 0:
                self.current_count -= 1
                self.condition.notify()

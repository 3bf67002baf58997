"""A Qwen3-shaped decoder whose attention layers decode over the MSA sparse context.

This is the decode loop of the reference (``src/msa/generate.py:101-186`` driving
``MSADeocoderLayer`` / ``MemorySparseAttention`` in its "generate" stage,
``src/msa/model.py:67-135``, ``src/msa/memory_sparse_attention.py:361-405``) reduced to what a
throughput measurement needs: random-initialised weights of the real shapes, greedy sampling, no
tokenizer and no string handling.  The GEMMs (projections, MLP, lm_head) are cuBLAS as in the reference;
the elementwise work between them (RMSNorm, q/k norm + RoPE, residual adds, SiLU*up) runs on three small
fused kernels; attention runs on this package's flash-decode kernel with
in-place append, and the router layers route every step through ``MSAService``:

    route(step t, layer l)  ->  fetch of the winners' pooled K/V from the pinned host bank on a
    side stream, started with the scoring of the next router layer  ->  written into the "retrieved" segment of layer l's cache, where the attention
    of step t+1 reads it.

So the host fetch never sits on the critical path: it overlaps the rest of the step, and with
``step_pipelined`` (the loop rotated to start at the first router layer) also the router-free lower
layers of the next step.  (The
reference routes once per round, in prefill stage 2; per-step routing is the variant benchmark
config 5 asks to time.)  KV layout per layer: ``[template t | retrieved k*c | local + generated]``.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn.functional as F

from . import ops
from .service import MSAService


@dataclass
class DecoderShape:
    num_layers: int = 36
    hidden: int = 2560
    n_q_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 9728
    vocab: int = 151_936
    rope_theta: float = 1_000_000.0
    rms_eps: float = 1e-6
    template_len: int = 3


class SparseDecodeModel:
    def __init__(self, shape: DecoderShape, service: Optional[MSAService], router_layers: List[int], batch: int,
                 local_ctx: int, max_new: int, retrieved_entries: int, device, dtype=torch.bfloat16, seed: int = 0):
        self.s, self.svc, self.device, self.dtype = shape, service, device, dtype
        self.router_layers = set(router_layers)
        self.batch, self.max_new, self.retrieved = batch, max_new, retrieved_entries
        s = shape
        g = torch.Generator(device=device)
        g.manual_seed(seed)

        def w(*dims, scale=None):
            scale = scale if scale is not None else 1.0 / math.sqrt(dims[0])
            return (torch.randn(dims, generator=g, device=device, dtype=torch.float32) * scale).to(dtype)

        qkv_out = (s.n_q_heads + 2 * s.n_kv_heads) * s.head_dim
        self.layers = []
        for l in range(s.num_layers):
            extra = s.n_q_heads * s.head_dim if l in self.router_layers else 0
            self.layers.append(dict(
                w_in=torch.ones(s.hidden, device=device, dtype=dtype),
                w_qkv=w(s.hidden, qkv_out + extra),            # q | k | v | (router q): one GEMM
                q_norm=torch.ones(s.head_dim, device=device, dtype=dtype),
                k_norm=torch.ones(s.head_dim, device=device, dtype=dtype),
                w_o=w(s.n_q_heads * s.head_dim, s.hidden),
                w_post=torch.ones(s.hidden, device=device, dtype=dtype),
                w_gate_up=w(s.hidden, 2 * s.ffn),
                w_down=w(s.ffn, s.hidden),
            ))
        self.embed = w(s.vocab, s.hidden, scale=1.0)
        self.w_final = torch.ones(s.hidden, device=device, dtype=dtype)
        self.lm_head = w(s.hidden, s.vocab)

        # caches: [template | retrieved | local context + generated tokens], filled synthetically
        self.ctx0 = s.template_len + retrieved_entries + local_ctx
        cap = self.ctx0 + max_new + 1
        self.k_cache = [torch.randn((batch, s.n_kv_heads, cap, s.head_dim), generator=g, device=device,
                                    dtype=torch.float32).to(dtype) for _ in range(s.num_layers)]
        self.v_cache = [torch.randn((batch, s.n_kv_heads, cap, s.head_dim), generator=g, device=device,
                                    dtype=torch.float32).to(dtype) for _ in range(s.num_layers)]
        self.kv_len = torch.full((batch,), self.ctx0, dtype=torch.int32, device=device)
        self.positions = torch.full((batch,), s.template_len + 16 + local_ctx, dtype=torch.long, device=device)
        self.inv_freq = 1.0 / (s.rope_theta ** (torch.arange(0, s.head_dim, 2, device=device, dtype=torch.float32)
                                                / s.head_dim))
        self.tokens = torch.randint(0, s.vocab, (batch,), generator=g, device=device)
        self.query_mask = torch.ones((batch, 1), dtype=torch.bool, device=device)
        self.n_splits = ops.decode_splits(batch, s.n_kv_heads, cap)
        need = batch * s.n_q_heads * self.n_splits * (s.head_dim + 2)
        self.workspace = torch.empty(max(need, 1), dtype=torch.float32, device=device)
        self.attn_out = torch.empty((batch, s.n_q_heads * s.head_dim), dtype=dtype, device=device)
        self.fetch_stream = torch.cuda.Stream(device, priority=-1)   # its small copies go ahead of queued compute
        self.fetch_enabled = True
        self._fetch_issued = False
        # Where a router layer's host gather starts.  "routing": with the NEXT router layer's scoring kernel, which its
        # zero-copy reads slow by a tenth; "dense": right after the layer's attention, beside the output / MLP GEMMs,
        # which ran 2.1x slower while 24 CTAs of PCIe reads were in flight (1.3x beside 8 CTAs; 1.2x beside the same
        # gather reading device memory).  Beside the scoring pays while the scoring of this rank's shard lasts at
        # least as long as the gather (measured, 1.56M chunks, batch 32: 1 GPU 13.64 -> 13.57 ms per step, 2 GPUs
        # 11.13 -> 10.60 ms); with a shorter scoring kernel the gather runs into the routing's collectives and the
        # selection (4 GPUs: 7.5-7.6 ms beside the GEMMs, 8.2 ms beside the scoring).
        self.fetch_beside = os.environ.get("MSA_B200_DECODE_FETCH_BESIDE") or self._fetch_placement()
        self.gather_ctas = int(os.environ.get("MSA_B200_DECODE_GATHER_CTAS", "24"))   # CTAs of the host gather beside the step's kernels
        # the decode loop is cut at the first router layer (see step_pipelined)
        self.split_layer = min(self.router_layers) if (self.router_layers and service is not None) else s.num_layers
        self._x_mid = torch.zeros((batch, s.hidden), dtype=dtype, device=device)
        self._pending_mid = torch.zeros((batch, s.hidden), dtype=dtype, device=device)
        # norms, rotary embedding, residual adds and SiLU*up on this package's fused kernels (bf16, head_dim 128)
        self.fused = dtype == torch.bfloat16 and s.head_dim == 128 and s.hidden % 2 == 0 and s.ffn % 2 == 0
        self._cos = torch.zeros((batch, 1, s.head_dim), dtype=dtype, device=device)
        self._sin = torch.zeros((batch, 1, s.head_dim), dtype=dtype, device=device)
        self.probe = None  # set to a dict to collect per-layer CUDA events (a profiled step)
        self.probe_external = False  # True: event-record nodes, readable after the replay of a graph that captured them
        # The cache layout [template | retrieved | local] gives every sequence exactly `retrieved_entries`
        # positions for fetched entries; a step whose winners hold fewer would leave the previous step's entries
        # in the tail of the segment.  The smallest count seen per router layer is tracked on the device and
        # checked by check_fetch_counts().
        self._n_sel_min = {l: torch.full((), retrieved_entries, dtype=torch.int64, device=device)
                           for l in self.router_layers}
        # Which document every slot of a sequence's retrieved segment holds, per router layer: a document that is
        # selected again in the next step keeps its entries and is not read from the host again.
        self._resident = {}
        top_k = service.model_config.doc_top_k if service is not None else 0
        if top_k and retrieved_entries % top_k == 0 and os.environ.get("MSA_B200_DECODE_RESIDENT", "1") != "0":
            self._resident = {l: torch.full((batch, top_k), -1, dtype=torch.int64, device=device) for l in self.router_layers}

    # ------------------------------------------------------------------------------------
    def _rope(self, x, cos, sin):
        d = x.shape[-1]
        rot = torch.cat([-x[..., d // 2:], x[..., : d // 2]], dim=-1)
        return x * cos + rot * sin

    def _mark(self, name, layer, stream=None):
        if self.probe is not None:
            e = torch.cuda.Event(enable_timing=True, external=self.probe_external)
            e.record(stream if stream is not None else torch.cuda.current_stream(self.device))
            self.probe.setdefault(name, {})[layer] = e

    def _layers(self, x, pending, lo, hi, fetch_done):
        """Layers lo..hi-1.  ``x`` is the residual stream, ``pending`` a branch output not yet added to it
        (None at the start); returns the same pair, so that the add fuses with the next RMSNorm."""
        s, B = self.s, self.batch
        main = torch.cuda.current_stream(self.device)
        cos, sin = self._cos, self._sin
        nq, nkv, d = s.n_q_heads, s.n_kv_heads, s.head_dim
        deferred = None
        for l in range(lo, hi):
            p = self.layers[l]
            self._mark("layer_start", l)
            if self.fused:
                x, h = ops.add_rmsnorm(x, pending, p["w_in"], s.rms_eps)
            else:
                x = x if pending is None else x + pending
                h = F.rms_norm(x, (s.hidden,), p["w_in"], s.rms_eps)
            qkv = h @ p["w_qkv"]
            v = qkv[:, (nq + nkv) * d: (nq + 2 * nkv) * d].reshape(B, nkv, d)
            if self.fused:
                q, k = ops.qk_norm_rope(qkv, nq, nkv, p["q_norm"], p["k_norm"], s.rms_eps, cos, sin)
            else:
                q = qkv[:, : nq * d].view(B, nq, d)
                k = qkv[:, nq * d: (nq + nkv) * d].view(B, nkv, d)
                q = self._rope(F.rms_norm(q, (d,), p["q_norm"], s.rms_eps), cos, sin)
                k = self._rope(F.rms_norm(k, (d,), p["k_norm"], s.rms_eps), cos, sin)
            routed = None
            if l in self.router_layers and self.svc is not None:
                self._mark("route_start", l)
                if deferred is not None:        # the previous router layer's fetch starts with this layer's routing
                    self._issue_fetch(*deferred, fetch_done)
                    deferred = None
                rq = qkv[:, (nq + 2 * nkv) * d:].view(B, nq, 1, d)      # L2-normalised inside the fold kernel
                routed = self.svc.route(rq, self.query_mask, l, l2_normalize=True, all_valid=True)
                self._mark("route_end", l)
            self._mark("attn_start", l)
            ops.sparse_decode_attn(q, self.k_cache[l], self.v_cache[l], self.kv_len, k, v, n_splits=self.n_splits,
                                   workspace=self.workspace, out=self.attn_out)
            self._mark("attn_end", l)
            if routed is not None and self.fetch_enabled:
                # the retrieved segment may only be overwritten once this step's attention has read it
                if deferred is not None:
                    self._issue_fetch(*deferred, fetch_done)
                    deferred = None
                if self.fetch_beside == "routing" and l + 1 < hi:
                    deferred = (routed, l)
                else:
                    self._issue_fetch(routed, l, fetch_done)
            attn = self.attn_out @ p["w_o"]
            if self.fused:
                x, h = ops.add_rmsnorm(x, attn, p["w_post"], s.rms_eps)
                pending = ops.silu_mul(h @ p["w_gate_up"], s.ffn) @ p["w_down"]
            else:
                x = x + attn
                h = F.rms_norm(x, (s.hidden,), p["w_post"], s.rms_eps)
                gu = h @ p["w_gate_up"]
                pending = (F.silu(gu[:, : s.ffn]) * gu[:, s.ffn:]) @ p["w_down"]
        if deferred is not None:
            self._issue_fetch(*deferred, fetch_done)
        return x, pending

    def _fetch_placement(self):
        """"routing" when streaming this rank's router keys of one layer (at 6.5 TB/s) takes at least as long as reading
        this rank's share of a layer's winners from host memory, else "dense".  Host reads: 48 GB/s for one GPU, and
        about 80 GB/s for all GPUs of the node together (measured per GPU: 35 GB/s at 2, 28 at 4, 10 at 8)."""
        if self.svc is None or not self.router_layers:
            return "dense"
        blk = self.svc.blocks[min(self.router_layers)]
        rk = blk.rk if blk.rk is not None else blk.rk_blocked
        if rk is None:
            return "dense"
        s = self.s
        world = max(1, self.svc.world_size)
        scoring_s = rk.numel() * rk.element_size() / 6.5e12
        fetch_bytes = self.batch * self.retrieved * 2 * s.n_kv_heads * s.head_dim * self.dtype.itemsize   # this rank's sequences
        gather_s = fetch_bytes / min(48e9, 80e9 / world)
        return "routing" if scoring_s >= gather_s else "dense"

    def _issue_fetch(self, routed, l, fetch_done):
        """Fetch the winners' K/V of router layer ``l`` on the side stream, from this point of the main stream on,
        and refresh the layer's retrieved segment."""
        s = self.s
        _, local, _, rank = routed
        gate = torch.cuda.Event()
        gate.record(torch.cuda.current_stream(self.device))
        self.fetch_stream.wait_event(gate)
        with torch.cuda.stream(self.fetch_stream):
            self._mark("fetch_start", l, self.fetch_stream)
            # the gather writes every sequence's entries into its own retrieved segment of the cache
            n_sel = self.svc.fetch_into(local, rank, l, self.k_cache[l], self.v_cache[l], s.template_len,
                                        self.retrieved, max_ctas=self.gather_ctas, resident=self._resident.get(l))
            torch.minimum(self._n_sel_min[l], n_sel.min(), out=self._n_sel_min[l])
            for t_ in (local, rank, n_sel):
                t_.record_stream(self.fetch_stream)
            done = torch.cuda.Event(enable_timing=self.probe is not None,
                                    external=self.probe is not None and self.probe_external)
            done.record(self.fetch_stream)
            fetch_done.append(done)
            self._fetch_issued = True
            if self.probe is not None:
                self.probe.setdefault("fetch_end", {})[l] = done

    def _front(self):
        """Embedding, rotary tables and the layers below the first router layer -> ``self._x_mid``."""
        self._mark("front_start", 0)
        ang = self.positions.to(torch.float32).unsqueeze(-1) * self.inv_freq
        emb = torch.cat([ang, ang], dim=-1)
        self._cos.copy_(emb.cos().unsqueeze(1))
        self._sin.copy_(emb.sin().unsqueeze(1))
        x, pending = self._layers(self.embed[self.tokens], None, 0, self.split_layer, [])
        self._x_mid.copy_(x)
        if pending is not None:
            self._pending_mid.copy_(pending)

    def _back(self):
        """Router layers and everything above them, lm_head, greedy token, cache-length update."""
        s = self.s
        fetch_done = []
        self._mark("back_start", 0)
        x, pending = self._layers(self._x_mid, self._pending_mid if self.split_layer > 0 else None, self.split_layer,
                                  s.num_layers, fetch_done)
        if self.fused:
            _, x = ops.add_rmsnorm(x, pending, self.w_final, s.rms_eps)
        else:
            x = F.rms_norm(x if pending is None else x + pending, (s.hidden,), self.w_final, s.rms_eps)
        nxt = (x @ self.lm_head).argmax(dim=-1)
        self._mark("compute_end", 0)
        if self.probe is not None:
            self.probe["fetch_done"] = fetch_done
        self.tokens.copy_(nxt)
        self.kv_len += 1
        self.positions += 1
        return nxt

    def step(self):
        """One decode step for the whole batch; returns the next tokens ``[B]``.  The step ends when
        the refreshed retrieved segments are in place."""
        self._front()
        nxt = self._back()
        self._join_fetch()
        return nxt

    def prime(self):
        """Run the lower layers of the first step, so that ``step_pipelined`` can start at the router layers."""
        self._front()

    def step_pipelined(self):
        """The same decode loop rotated by half a step: [router layers and above of step t, sampling, lower
        layers of step t+1].  The tokens are those of ``step``; the host fetch issued by step t's router layers
        now has the lower (router-free) layers of step t+1 to hide behind before anything reads what it
        refreshes.  Call ``prime`` once before the first call.  One call = one token per sequence."""
        nxt = self._back()
        self._front()
        self._mark("front_end", 0)
        self._join_fetch()
        self._mark("step_end", 0)
        return nxt

    def _join_fetch(self):
        """The step ends when the refreshed segments are in place.  Only a step that issued a fetch waits: inside a
        stream capture, waiting on the fetch stream when nothing was forked into it would tie the captured graph to
        work outside the capture, which invalidates the capture."""
        if self._fetch_issued:
            torch.cuda.current_stream(self.device).wait_stream(self.fetch_stream)
            self._fetch_issued = False

    def check_fetch_counts(self):
        """Raise if some step fetched fewer entries for a sequence than its retrieved segment holds (documents of
        varying length, invalid winners): this loop's fixed cache layout needs ``retrieved_entries`` per step."""
        torch.cuda.synchronize(self.device)
        low = {l: int(v.item()) for l, v in self._n_sel_min.items() if int(v.item()) < self.retrieved}
        if low:
            raise RuntimeError(f"router layers {sorted(low)} fetched as few as {min(low.values())} entries for a sequence; "
                               f"the decode loop's cache layout holds exactly {self.retrieved} retrieved entries")

    def reset(self):
        for table in self._resident.values():      # the caller may refill the caches: no segment's content is known any more
            table.fill_(-1)
        self.kv_len.fill_(self.ctx0)
        self.positions.fill_(self.s.template_len + 16 + (self.ctx0 - self.s.template_len - self.retrieved))

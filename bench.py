"""Routing benchmark: queries/s over a 100M-token pooled memory bank (benchmark config 4).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (fixed for every N, so scaling is STRONG): 195,313 documents x 8 chunks =
1,562,504 pooled router keys per layer, 18 routing layers, bf16, sharded by document over
the N ranks; 128 queries x 256 routing tokens, split over the ranks (each rank scores ALL
queries against its shard).  A step = all 18 layers: fold -> (all-gather queries) -> fused
score/reduce -> per-shard top-k -> (all-gather candidates) -> merge to the global top-16.
Inputs are seeded synthetic (cosine mode: unit-norm heads; keys = per-document mean N(0,0.5)
+ noise of std 1/8 per chunk, the pooled statistics of benchmark config 3's distribution).

`value` times the step with queries resident in HBM; `e2e` times the same step through
MSAService.route with the queries in pinned HOST memory (H2D of every layer's queries and
D2H of every layer's winners inside the timed region).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_DOCS, CHUNKS_PER_DOC, N_LAYERS = 195_313, 8, 18
N_QUERIES, Q_TOKENS, HQ, HKV, D, TOP_K = 128, 256, 32, 8, 128, 16
METRIC = "routing queries/s over 100M-token memory"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--docs", type=int, default=N_DOCS, help="shrink the bank (development only)")
    ap.add_argument("--layers", type=int, default=N_LAYERS)
    ap.add_argument("--queries", type=int, default=N_QUERIES)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--new-tokens", type=int, default=256, help="generate workload: tokens to decode")
    ap.add_argument("--workload", default="routing", choices=["routing", "pooling", "decode", "fetch", "route-decode", "prefill", "stage1", "generate"],
                    help="routing = the headline (default); the others time one secondary kernel each")
    return ap.parse_args()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "tflops": p["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of GPU `index`, sampled during the timed region."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
            t0 = time.time()
            while not self.rows and time.time() - t0 < 2.0:   # sampling is live before the timed region starts
                time.sleep(0.02)
            self.rows.clear()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ------------------------------------------------------------------------------------------
def cpu_reference_sample(threads: int, target_s: float = 12.0):
    """The oracle port of Memory.prefill_stage2 (matmul over all 32 heads, masked_fill, head mean,
    token max, scatter amax, topk) on the host cores, fp32, on a bounded sample; extrapolated
    linearly in chunks and layers to the full workload."""
    import torch
    from oracle import msa_oracle as O
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(4000)
    n_q, docs = 2, 2048
    chunks = docs * CHUNKS_PER_DOC
    rk = torch.nn.functional.normalize(torch.randn(HKV, chunks, D, generator=g), dim=-1)
    pool_ids = torch.repeat_interleave(torch.arange(1, docs + 1), CHUNKS_PER_DOC)
    table = torch.arange(docs + 1)
    q = torch.nn.functional.normalize(torch.randn(n_q, HKV, HQ // HKV, Q_TOKENS, D, generator=g), dim=-1)
    mask = torch.ones(n_q, Q_TOKENS, dtype=torch.bool)

    def once():
        t0 = time.perf_counter()
        O.prefill_stage2(q, mask, rk, pool_ids, table, TOP_K)
        return time.perf_counter() - t0
    once()
    t1 = once()
    reps = max(1, min(20, int(target_s / max(t1, 1e-3))))
    t = statistics.median([once() for _ in range(reps)])
    per_query_full = t / n_q * (N_DOCS * CHUNKS_PER_DOC / chunks) * N_LAYERS
    sample = (f"oracle port of prefill_stage2, fp32, {n_q} queries x {Q_TOKENS} tokens x {chunks} chunks x 1 layer, "
              f"median of {reps}, scaled x{N_DOCS * CHUNKS_PER_DOC / chunks:.1f} chunks x{N_LAYERS} layers")
    return 1.0 / per_query_full, sample, t


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    vals, sample, t_last = [], "", 0.0
    for i in range(args.warmup + args.steps):
        v, sample, t_last = cpu_reference_sample(threads, target_s=2.0)
        if i >= args.warmup:
            vals.append(v)
    v = statistics.median(vals)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": "queries/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * N_QUERIES / v, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "benchmark config 4: 100M-token bank, 18 layers, 128 queries x 256 tokens, top-16",
                   "note": "CPU: bounded sample, extrapolated linearly"},
        "cpu_baseline": {"value": v, "unit": "queries/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------------------------------
def make_bank(torch, dev, docs_local: int, layers: int, seed: int):
    """Pooled router keys [C, Hkv, D] bf16 per layer, generated on the device in slices."""
    out = []
    g = torch.Generator(device=dev)
    for layer in range(layers):
        g.manual_seed(seed + layer)
        rk = torch.empty((docs_local * CHUNKS_PER_DOC, HKV, D), dtype=torch.bfloat16, device=dev)
        step = 8192
        for d0 in range(0, docs_local, step):
            n = min(step, docs_local - d0)
            mu = torch.randn((n, 1, HKV, D), generator=g, device=dev) * 0.5
            x = mu + torch.randn((n, CHUNKS_PER_DOC, HKV, D), generator=g, device=dev) * 0.125
            x = torch.nn.functional.normalize(x, dim=-1)
            rk[d0 * CHUNKS_PER_DOC:(d0 + n) * CHUNKS_PER_DOC] = x.view(-1, HKV, D).to(torch.bfloat16)
        out.append(rk)
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist
    from msa_b200 import ops
    from msa_b200.memory import AttentionGeometry, Document, ModelConfig
    from msa_b200.service import MSAService, all_gather_cat

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    n_docs, layers, n_q = args.docs, args.layers, args.queries
    per = (n_docs + world - 1) // world
    d_lo, d_hi = min(n_docs, rank * per), min(n_docs, (rank + 1) * per)
    docs_local = d_hi - d_lo
    b = n_q // world
    assert b * world == n_q, "queries must divide over the ranks"
    shard_k = TOP_K if world == 1 else 2 * TOP_K

    model_cfg = ModelConfig(doc_top_k=TOP_K, router_layer_idx=",".join(str(18 + i) for i in range(layers)))
    svc = MSAService(local_rank, None, model_cfg, None, AttentionGeometry(), world_size=world, rank=rank,
                     shard_top_k=shard_k)
    docs = [Document(doc_id=d_lo + i, num_chunks=CHUNKS_PER_DOC) for i in range(docs_local)]
    svc.block_desc.init_docs(docs, dev)
    svc.block_desc.pool_ids_from_docs(dev)
    bank = make_bank(torch, dev, docs_local, layers, seed=4000 + 100 * rank)
    for i, layer in enumerate(svc.router_layer_ids):
        svc.blocks[layer].rk = bank[i]

    # queries: pinned host copy (e2e) and device copy (kernel-resident value)
    gq = torch.Generator(device=dev)
    gq.manual_seed(504_000 + rank)
    q_host, q_dev = [], []
    for layer in range(layers):
        q = torch.nn.functional.normalize(torch.randn((b, HQ, Q_TOKENS, D), generator=gq, device=dev), dim=-1)
        q_dev.append(q.to(torch.bfloat16))
        host = torch.empty(q.shape, dtype=torch.bfloat16).pin_memory()
        host.copy_(q_dev[-1])
        q_host.append(host)
    mask_host = torch.ones((b, Q_TOKENS), dtype=torch.bool).pin_memory()
    mask_dev = mask_host.to(dev)

    n_all = n_q
    s_pad = ops.route_s_pad(Q_TOKENS)
    c_local = docs_local * CHUNKS_PER_DOC
    keys = torch.empty((n_all, docs_local + 1), dtype=torch.int32, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    min_val = torch.finfo(torch.bfloat16).min
    route_events = []
    launches = [0]
    cand = ops.candidate_buffer(n_all, min(shard_k, docs_local + 1), dev) if world > 1 else None

    def layer_resident(i, layer, timed):
        qf, bias, _ = ops.fold_queries(q_dev[i], mask_dev, HQ // HKV, s_pad=s_pad)
        if world > 1:
            qf = all_gather_cat(qf, world).view(-1, qf.shape[1])
            bias = all_gather_cat(bias, world).view(-1)
        ops.route_table_reset(keys, docs_local, min_val, status)
        if timed:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        ops.route_scores(qf, bias, n_all, s_pad, svc.blocks[layer].rk, svc.block_desc.chunk_doc, docs_local,
                         alpha=1.0 / HQ, min_val=min_val, keys=keys, status=status, flags=2)
        if timed:
            e1.record()
            route_events.append((e0, e1))
        if world > 1:
            ops.topk_select(keys, shard_k, svc.block_desc.doc_ids, out=cand[1:])
            sc, li, gi = ops.candidate_views(all_gather_cat(cand[0], world))
        else:
            sc, li, gi = ops.topk_select(keys, shard_k, svc.block_desc.doc_ids)
            sc, li, gi = sc.unsqueeze(0), li.unsqueeze(0), gi.unsqueeze(0)
        launches[0] += 5
        return ops.topk_merge(sc, li, gi, TOP_K, seq_offset=rank * b, n_seq=b)

    def step_resident(timed):
        out = None
        for i, layer in enumerate(svc.router_layer_ids):
            out = layer_resident(i, layer, timed)
        return out

    copy_stream = torch.cuda.Stream(dev)
    stage = [torch.empty_like(q_dev[0]) for _ in range(2)]
    res_host = [(torch.empty((b, TOP_K), dtype=torch.float32).pin_memory(),
                 torch.empty((b, TOP_K), dtype=torch.int64).pin_memory()) for _ in range(layers)]

    # host-resident content bank (K then V per chunk), one layer's worth shared by all layers:
    # docs_local x 8 chunks x 4 KiB per rank (6.4 GB over all ranks), mapped by every rank
    fetch_note = None
    try:
        g_kv = torch.Generator(device=dev)
        g_kv.manual_seed(77 + rank)
        for layer in svc.router_layer_ids[:1]:
            kv = torch.empty((c_local, 2, HKV, D), dtype=torch.bfloat16).pin_memory()
            step_c = 1 << 18
            for c0 in range(0, c_local, step_c):
                n = min(step_c, c_local - c0)
                kv[c0:c0 + n].copy_(torch.randn((n, 2, HKV, D), generator=g_kv, device=dev).to(torch.bfloat16))
            svc.blocks[layer].kv = kv
            svc.blocks[layer].kv_device_address = kv.data_ptr()
        first = svc.router_layer_ids[0]
        for layer in svc.router_layer_ids[1:]:
            svc.blocks[layer].kv = svc.blocks[first].kv
            svc.blocks[layer].kv_device_address = svc.blocks[first].kv_device_address
        if world > 1:
            shm = "/dev/shm"
            need = c_local * 2 * HKV * D * 2
            st = os.statvfs(shm)
            if st.f_bavail * st.f_frsize < need * 1.1:
                raise RuntimeError(f"{shm} has {st.f_bavail * st.f_frsize >> 20} MiB free, {need >> 20} MiB needed")
            keep_ids = svc.router_layer_ids
            svc.router_layer_ids = keep_ids[:1]          # one bank file per rank
            svc.share_host_banks(tag=f"bench{os.environ.get('MASTER_PORT', '0')}")
            svc.router_layer_ids = keep_ids
            base_, offs_, ln_, kvb = svc._directory
            svc._directory = (base_, offs_, ln_, {layer: kvb[first] for layer in keep_ids})
            for layer in keep_ids[1:]:
                svc.blocks[layer].kv = svc.blocks[first].kv
        else:
            svc.publish_directory()
    except Exception as e:  # the routing numbers stand without the fetch leg
        fetch_note = f"fetch leg skipped: {e}"
    fetch_stream = torch.cuda.Stream(dev)
    max_entries = b * TOP_K * CHUNKS_PER_DOC
    timeline = {}

    def step_e2e():
        """Through MSAService.route / .fetch with host-resident queries: the copy stream brings layer
        l+1's queries over PCIe while layer l is scored; layer l's winners' K/V are fetched from the
        pinned host bank on a side stream while layer l+1 is scored; winners go back to host memory."""
        main = torch.cuda.current_stream(dev)
        ready = [torch.cuda.Event() for _ in range(layers)]
        freed = [torch.cuda.Event() for _ in range(layers)]
        ev = {k_: [torch.cuda.Event(enable_timing=True) for _ in range(layers)] for k_ in ("rs", "re", "fs", "fe")}
        t0 = torch.cuda.Event(enable_timing=True)
        t0.record(main)
        for i, layer in enumerate(svc.router_layer_ids):
            with torch.cuda.stream(copy_stream):
                if i >= 2:
                    copy_stream.wait_event(freed[i - 2])
                stage[i % 2].copy_(q_host[i], non_blocking=True)
                ready[i].record(copy_stream)
            main.wait_event(ready[i])
            ev["rs"][i].record(main)
            sc, li, gi, rk_ = svc.route(stage[i % 2], mask_dev, layer)
            ev["re"][i].record(main)
            freed[i].record(main)
            res_host[i][0].copy_(sc, non_blocking=True)
            res_host[i][1].copy_(gi, non_blocking=True)
            if fetch_note is None:
                fetch_stream.wait_event(ev["re"][i])
                with torch.cuda.stream(fetch_stream):
                    ev["fs"][i].record(fetch_stream)
                    fk, fv, n_sel, total = svc.fetch(li, rk_, layer, max_entries=max_entries)
                    ev["fe"][i].record(fetch_stream)
                    for t_ in (li, rk_, fk, fv):
                        t_.record_stream(fetch_stream)
        main.wait_stream(fetch_stream)
        timeline["ev"], timeline["t0"] = ev, t0

    def sync_all():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    def timed_region(fn, steps):
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        sync_all()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(args.warmup):
        step_resident(False)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches[0] = 0
    ms_total = timed_region(lambda: step_resident(True), args.steps)
    clocks = sampler.stop() if rank == 0 else None
    n_launch = launches[0]
    svc._status = status
    svc.check_status()
    route_ms = [a.elapsed_time(b_) for a, b_ in route_events]
    route_avg_ms = sum(route_ms) / len(route_ms)

    for _ in range(max(1, args.warmup // 2)):
        step_e2e()
    ms_e2e = timed_region(step_e2e, args.steps)
    svc.check_status()

    fetch_report = {"note": fetch_note}
    if fetch_note is None:
        ev, t0 = timeline["ev"], timeline["t0"]
        rs = [t0.elapsed_time(e) for e in ev["rs"]]
        re_ = [t0.elapsed_time(e) for e in ev["re"]]
        fs = [t0.elapsed_time(e) for e in ev["fs"]]
        fe = [t0.elapsed_time(e) for e in ev["fe"]]
        fetch_ms = [b_ - a_ for a_, b_ in zip(fs, fe)]
        hidden = sum(1 for i in range(layers - 1) if fe[i] <= re_[i + 1])
        fetch_bytes = b * TOP_K * CHUNKS_PER_DOC * 2 * HKV * D * 2
        fetch_report = {
            "bytes_per_layer_per_gpu": fetch_bytes, "avg_ms": sum(fetch_ms) / layers,
            "pcie_gbs": fetch_bytes / (sum(fetch_ms) / layers / 1e3) / 1e9,
            "layers_hidden_behind_next_layer_scoring": f"{hidden}/{layers - 1}",
            "exposed_ms_after_last_layer": max(0.0, fe[-1] - re_[-1]),
            "timeline_ms_first_3_layers": [{"route": [round(rs[i], 3), round(re_[i], 3)],
                                            "fetch": [round(fs[i], 3), round(fe[i], 3)]} for i in range(min(3, layers))],
            "host_bank": "one layer's K/V bank (docs x 8 chunks x 4 KiB), pinned, shared by the 18 layers"}
        if world > 1:
            svc.close_host_banks()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    pk = peaks()
    ms_step = ms_total / args.steps
    value = n_q / (ms_step / 1e3)
    e2e_value = n_q / (ms_e2e / args.steps / 1e3)
    flops = 2.0 * n_all * s_pad * c_local * (HKV * D)
    achieved_tf = flops / (route_avg_ms / 1e3) / 1e12
    alg_bytes = c_local * HKV * D * 2 + n_all * s_pad * HKV * D * 2
    n_qtiles = (n_all * s_pad + 255) // 256
    pair = ((c_local + 127) // 128) * n_qtiles >= 2 * 148          # the library's rule for the 2-CTA kernel
    kernel_name = "route_tc_pair_kernel" if pair else "route_tc_kernel"
    traffic = ((n_qtiles + 63) // 64) * c_local * HKV * D * 2 + n_all * s_pad * HKV * D * 2
    line = {
        "metric": METRIC, "value": value, "unit": "queries/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"benchmark config 4: {n_docs} docs x {CHUNKS_PER_DOC} chunks (100M tokens), {layers} routing "
                               f"layers, {n_q} queries x {Q_TOKENS} tokens, top-{TOP_K}, cosine scores",
                   "sharding": f"bank by document over {world} rank(s); every rank scores all queries; "
                               f"per-shard top-{shard_k}, all-gather merge",
                   "l2": "inputs per layer (router keys %.0f MB) exceed L2; 18 distinct layers per step" % (c_local * 2048 / 1e6)},
        "e2e": {"value": e2e_value, "unit": "queries/s",
                "h2d_bytes_per_step": layers * (q_host[0].numel() * 2) * world,
                "d2h_bytes_per_step": layers * b * TOP_K * 12 * world,
                "host_to_device_fetch_bytes_per_step": 0 if fetch_note else layers * world * b * TOP_K * CHUNKS_PER_DOC * 2 * HKV * D * 2},
        "gpu_launches": n_launch,
        "fetch": fetch_report,
        "clocks": clocks,
        "roofline": {"kernel": kernel_name, "bound": "tensor", "achieved": achieved_tf, "peak": pk["tflops"],
                     "unit": "TFLOP/s", "frac": achieved_tf / pk["tflops"], "traffic": traffic,
                     "traffic_source": "ncu dram__bytes_read+write of a 160,000-chunk launch (846 MB = keys x query "
                                       "groups + queries), scaled by the chunk count of this launch",
                     "peak_source": pk["source"] + " (bf16 sustained)", "avg_launch_ms": route_avg_ms,
                     "flops_per_launch": flops,
                     "hbm": {"algorithmic_bytes_per_launch": alg_bytes,
                             "achieved_gbs": alg_bytes / (route_avg_ms / 1e3) / 1e9,
                             "frac_of_hbm": alg_bytes / (route_avg_ms / 1e3) / 1e9 / pk["hbm_gbs"]}},
    }
    if not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        v, sample, _ = cpu_reference_sample(threads)
        line["cpu_baseline"] = {"value": v, "unit": "queries/s", "cores": threads, "kind": "port", "sample": sample}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------
# Secondary kernels: one JSON line each (single GPU), HBM or PCIe roofline.
# ------------------------------------------------------------------------------------------
def _time_ms(torch, fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def _secondary_line(args, metric, unit, value, ms, workload, kernel, alg_bytes, peak, peak_name, clocks, launches,
                    extra=None):
    gbs = alg_bytes / (ms / 1e3) / 1e9
    line = {"metric": metric, "value": value, "unit": unit, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": {"workload": workload}, "gpu_launches": launches, "clocks": clocks,
            "roofline": {"kernel": kernel, "bound": "hbm" if peak_name == "hbm" else peak_name, "achieved": gbs,
                         "peak": peak, "unit": "GB/s", "frac": gbs / peak, "traffic": None,
                         "algorithmic_bytes_per_step": alg_bytes}}
    if extra:
        line.update(extra)
    print(json.dumps(line))


def run_secondary(args):
    import torch
    from msa_b200 import ops
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    pk = peaks()
    g = torch.Generator(device=dev)
    g.manual_seed(2000)
    sampler = ClockSampler(0)
    steps, warmup = max(args.steps, 50), max(args.warmup, 3)   # short kernels: time many launches
    args.steps, args.warmup = steps, warmup

    if args.workload == "pooling":
        # benchmark config 2: 2,048 documents x 512 tokens, K / V / K_r bf16 [1, 8, T, 128], chunk 64
        n_docs, doc_len, p = (2048 if args.docs == N_DOCS else args.docs), 512, 64
        t = n_docs * doc_len
        doc_ids = torch.arange(1, n_docs + 1, device=dev).repeat_interleave(doc_len).view(1, t)
        tok, off, pooled = ops.chunk_bookkeeping(doc_ids, None, p)
        ms_bk = _time_ms(torch, lambda: ops.chunk_bookkeeping(doc_ids, None, p, max_chunks=t // p + 1), 3, 1)
        states = [torch.randn((1, HKV, t, D), generator=g, device=dev).to(torch.bfloat16) for _ in range(3)]

        def step():
            ops.pool_chunks(states[0], off, tok)
            ops.pool_chunks(states[1], off, tok)
            ops.pool_chunks(states[2], off, tok, l2_normalize=True)
        sampler.start()
        ms = _time_ms(torch, step, steps, warmup)
        clocks = sampler.stop()
        c = off.numel() - 1
        alg = 3 * (t * HKV * D * 2 + c * HKV * D * 2)
        _secondary_line(args, "chunk-mean pooling tokens/s (K, V, K_r)", "tokens/s", t / (ms / 1e3), ms,
                        f"benchmark config 2: {n_docs} docs x {doc_len} tokens, chunk {p}, bf16, 3 tensors "
                        f"({t * HKV * D * 2 / 1e9:.2f} GB each, > L2)", "pool_kernel", alg, pk["hbm_gbs"], "hbm", clocks, 3 * steps,
                        {"bookkeeping_ms": ms_bk})

    elif args.workload == "decode":
        # benchmark config 5: batch 32, 32 q / 8 kv heads, L = 3 template + 128 retrieved + 2048 local
        b, L, n_layers = 32, 3 + 128 + 2048, 4
        caches = [(torch.randn((b, HKV, L + 8, D), generator=g, device=dev).to(torch.bfloat16),
                   torch.randn((b, HKV, L + 8, D), generator=g, device=dev).to(torch.bfloat16)) for _ in range(n_layers)]
        q = torch.randn((b, HQ, D), generator=g, device=dev).to(torch.bfloat16)
        nk = torch.randn((b, HKV, D), generator=g, device=dev).to(torch.bfloat16)
        nv = torch.randn((b, HKV, D), generator=g, device=dev).to(torch.bfloat16)
        kv_len = torch.full((b,), L, dtype=torch.int32, device=dev)
        n_splits = ops.decode_splits(b, HKV, L)
        ws = torch.empty(max(1, int(b * HQ * n_splits * (D + 2))), dtype=torch.float32, device=dev)
        out = torch.empty((b, HQ * D), dtype=torch.bfloat16, device=dev)

        def step():
            for kc, vc in caches:
                ops.sparse_decode_attn(q, kc, vc, kv_len, nk, nv, n_splits=n_splits, workspace=ws, out=out)
        _time_ms(torch, step, 2, 2)
        graph = torch.cuda.CUDAGraph()      # a decode loop replays its token step from a CUDA graph
        with torch.cuda.graph(graph):
            step()
        kv_len.fill_(L)
        sampler.start()
        ms = _time_ms(torch, graph.replay, 10 * steps, warmup) / n_layers
        clocks = sampler.stop()
        alg = 2 * b * (L + 1) * HKV * D * 2
        _secondary_line(args, "sparse decode attention layer-steps/s", "layer-steps/s", 1e3 / ms, ms,
                        f"benchmark config 5 layer: batch {b}, L={L}+1, 32q/8kv heads, d=128, bf16, {n_splits} KV "
                        f"splits, {n_layers} distinct caches of 285 MB rotate (> L2)", "decode_mma_kernel", alg,
                        pk["hbm_gbs"], "hbm", clocks, 3 * n_layers * steps)

    elif args.workload == "fetch":
        # host bank of 32,768 documents x 8 chunks (1.07 GB pinned); 128 queries x 16 winners per layer
        n_docs, b, k = 32768, N_QUERIES, TOP_K
        bank = torch.empty((n_docs * CHUNKS_PER_DOC, 2, HKV, D), dtype=torch.bfloat16).pin_memory()
        bank.copy_(torch.randn(bank.shape, generator=g, device=dev).to(torch.bfloat16))
        lens = torch.tensor([0] + [CHUNKS_PER_DOC] * n_docs, dtype=torch.int32, device=dev)
        offs = torch.cumsum(torch.cat([torch.zeros(1, dtype=torch.long, device=dev), lens[:-1].long()]), 0)
        base = torch.zeros(1, dtype=torch.long, device=dev)
        kv_base = torch.tensor([bank.data_ptr()], dtype=torch.int64, device=dev)
        gsel = torch.Generator().manual_seed(7)
        sels = [torch.stack([torch.randperm(n_docs, generator=gsel)[:k] + 1 for _ in range(b)]).to(dev) for _ in range(4)]
        n_entries = b * k * CHUNKS_PER_DOC
        state = {"i": 0}

        def step():
            sel = sels[state["i"] % len(sels)]
            state["i"] += 1
            plan, n_sel, total = ops.gather_plan(sel, None, 1, base, offs, lens, kv_base, 2 * HKV * D * 2)
            ops.gather_run(plan, torch.bfloat16, HKV, D, n_entries)
        sampler.start()
        ms = _time_ms(torch, step, steps, warmup)
        clocks = sampler.stop()
        alg = n_entries * 2 * HKV * D * 2
        _secondary_line(args, "host K/V fetch documents/s", "documents/s", b * k / (ms / 1e3), ms,
                        f"{b} queries x top-{k} documents x {CHUNKS_PER_DOC} chunks = {alg / 1e6:.0f} MB per layer from a "
                        f"1.07 GB pinned host bank (plan + gather)", "gather_kernel", alg, 55.0, "pcie", clocks,
                        2 * steps, {"note": "peak = 55 GB/s, a nominal PCIe Gen5 x16 payload rate (not measured)"})

    elif args.workload == "prefill":
        # stage 2 of one layer: 32 queries x 128 tokens, each with 3 template entries and 16 documents x 8 chunks
        # retrieved -> contexts of 259 keys; several layers' tensors rotate so that inputs exceed L2
        b, s_q, t_len, n_ret, n_layers = 32, 128, 3, TOP_K * CHUNKS_PER_DOC, 6
        layers = []
        for _ in range(n_layers):
            layers.append(dict(
                q=torch.randn((b, HQ, s_q, D), generator=g, device=dev).to(torch.bfloat16),
                k=torch.randn((b, HKV, s_q, D), generator=g, device=dev).to(torch.bfloat16),
                v=torch.randn((b, HKV, s_q, D), generator=g, device=dev).to(torch.bfloat16),
                tk=torch.randn((1, HKV, t_len, D), generator=g, device=dev).to(torch.bfloat16),
                tv=torch.randn((1, HKV, t_len, D), generator=g, device=dev).to(torch.bfloat16),
                sk=torch.randn((HKV, b * n_ret, D), generator=g, device=dev).to(torch.bfloat16),
                sv=torch.randn((HKV, b * n_ret, D), generator=g, device=dev).to(torch.bfloat16)))
        valid = torch.ones((b, s_q), dtype=torch.bool, device=dev)
        n_sel = torch.full((b,), n_ret, dtype=torch.int64, device=dev)
        max_kv = t_len + n_ret + s_q
        ev = []

        def step(timed=False):
            for L in layers:
                ks, vs, st, ln, qt, nq, _ = ops.assemble_context(L["tk"], L["tv"], L["sk"], L["sv"], n_sel, L["k"], L["v"],
                                                                 valid, max_kv, 0)
                if timed:
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                ops.sparse_prefill_attn(L["q"], ks, vs, st, ln, qt, nq)
                if timed:
                    e1.record()
                    ev.append((e0, e1))
        _time_ms(torch, lambda: step(True), 5, warmup)
        attn_ms = statistics.mean([a.elapsed_time(b_) for a, b_ in ev[-5 * n_layers:]])
        lib_ms = None
        try:    # the library call the reference makes at this point, on the same packed shapes (context only)
            from flash_attn import flash_attn_varlen_func
            cu_q = torch.arange(0, (b + 1) * s_q, s_q, dtype=torch.int32, device=dev)
            cu_k = torch.arange(0, (b + 1) * max_kv, max_kv, dtype=torch.int32, device=dev)
            qp = torch.randn((b * s_q, HQ, D), generator=g, device=dev).to(torch.bfloat16)
            kp = torch.randn((b * max_kv, HKV, D), generator=g, device=dev).to(torch.bfloat16)
            vp = torch.randn((b * max_kv, HKV, D), generator=g, device=dev).to(torch.bfloat16)
            lib_ms = _time_ms(torch, lambda: flash_attn_varlen_func(qp, kp, vp, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k,
                                                                    max_seqlen_q=s_q, max_seqlen_k=max_kv, causal=True),
                              steps, warmup)
        except Exception:
            pass
        sampler.start()
        ms = _time_ms(torch, step, steps, warmup) / n_layers
        clocks = sampler.stop()
        # bytes one layer must move: q read + out written, K/V of template/retrieved/query read and written once by
        # the assembly and read once more by the attention (they stay in L2 in between)
        kv_bytes = 2 * b * max_kv * HKV * D * 2
        alg = 2 * b * HQ * s_q * D * 2 + 2 * kv_bytes
        flops = 4.0 * b * HQ * D * sum(t_len + n_ret + i + 1 for i in range(s_q))
        _secondary_line(args, "stage-2 sparse prefill layer-steps/s (assembly + attention)", "layer-steps/s", 1e3 / ms, ms,
                        f"{b} queries x {s_q} tokens, {t_len} template + {n_ret} retrieved entries, 32q/8kv heads, d=128, "
                        f"bf16, {n_layers} layers' tensors rotate (> L2)", "prefill_attn_kernel", alg, pk["hbm_gbs"], "hbm",
                        clocks, 2 * n_layers * steps,
                        {"attention_kernel_ms": attn_ms, "attention_tflops": flops / (attn_ms / 1e3) / 1e12,
                         "library_varlen_attention_ms": lib_ms,
                         "note": "contexts of a few hundred keys: the kernel is latency / issue bound, far from either roof"})

    elif args.workload == "stage1":
        # benchmark config 2 shapes: documents of 512 tokens, 32 q / 8 kv heads, d = 128, chunk 64; one block row.
        # 512 documents (262,144 tokens: q and out 2.1 GB each) keep the run short; time scales linearly in documents.
        n_docs, doc_len, p = (512 if args.docs == N_DOCS else args.docs), 512, 64
        t = n_docs * doc_len
        doc_ids = torch.arange(1, n_docs + 1, device=dev).repeat_interleave(doc_len).view(1, t)
        tok, off, _ = ops.chunk_bookkeeping(doc_ids, None, p)
        seg = torch.arange(0, t + 1, doc_len, dtype=torch.int32, device=dev)
        q = torch.randn((1, HQ, t, D), generator=g, device=dev).to(torch.bfloat16)
        k = torch.randn((1, HKV, t, D), generator=g, device=dev).to(torch.bfloat16)
        v = torch.randn((1, HKV, t, D), generator=g, device=dev).to(torch.bfloat16)
        out = torch.zeros((1, t, HQ * D), dtype=torch.bfloat16, device=dev)

        tc_status = torch.zeros(4, dtype=torch.int32, device=dev)

        def step():      # what the layer mirror runs for unmasked documents: tcgen05 attention, then K and V pooled
            ops.doc_attention_tc(q, k, v, tok, seg, doc_len, out=out, status=tc_status)
            ops.pool_chunks(k, off, tok)
            ops.pool_chunks(v, off, tok)
        lib_ms = None
        try:    # what the reference does at this point: the library's varlen attention, then K and V pooled separately
            from flash_attn import flash_attn_varlen_func
            qp, kp, vp = q[0].transpose(0, 1).contiguous(), k[0].transpose(0, 1).contiguous(), v[0].transpose(0, 1).contiguous()
            lib_ms = _time_ms(torch, lambda: flash_attn_varlen_func(qp, kp, vp, cu_seqlens_q=seg, cu_seqlens_k=seg,
                                                                    max_seqlen_q=doc_len, max_seqlen_k=doc_len, causal=True),
                              10, 3)
            del qp, kp, vp
        except Exception:
            pass
        pool_ms = _time_ms(torch, lambda: (ops.pool_chunks(k, off, tok), ops.pool_chunks(v, off, tok)), 10, 3)
        tc_ms = _time_ms(torch, lambda: ops.doc_attention_tc(q, k, v, tok, seg, doc_len, out=out, status=tc_status), 10, 3)
        fused_ms = _time_ms(torch, lambda: ops.doc_attention_pool(q, k, v, tok, seg, doc_len, out=out, chunk_offsets=off,
                                                                  pool_size=p), 10, 3)
        steps = min(steps, 20)
        args.steps = steps
        sampler.start()
        ms = _time_ms(torch, step, steps, warmup)
        clocks = sampler.stop()
        assert tc_status.cpu().tolist()[0] == 0, "a bounded wait ran out inside doc_attn_tc_kernel"
        flops = 4.0 * n_docs * HQ * D * (doc_len * (doc_len + 1) / 2)          # causal: the part below the diagonal
        n_tiles = n_docs * HQ * sum(range(1, doc_len // 128 + 1))                # 128 x 128 tiles the kernel executes
        flops_exec = 4.0 * 128 * 128 * 128 * n_tiles
        alg = 2 * t * HQ * D * 2 + 2 * t * HKV * D * 2 + 2 * (t // p) * HKV * D * 2
        peak_tf = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"] \
            if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else 1590.0
        tf = flops_exec / (tc_ms / 1e3) / 1e12
        _secondary_line(args, "stage-1 document attention + K/V pooling tokens/s", "tokens/s", t / (ms / 1e3), ms,
                        f"{n_docs} documents x {doc_len} tokens in one block row, 32q/8kv heads, d=128, chunk {p}, bf16 "
                        f"(q and out {t * HQ * D * 2 / 1e9:.1f} GB each, > L2)", "doc_attn_tc_kernel", alg, pk["hbm_gbs"],
                        "hbm", clocks, 3 * steps,
                        {"roofline": {"kernel": "doc_attn_tc_kernel", "bound": "tensor", "achieved": tf, "peak": peak_tf,
                                      "unit": "TFLOP/s", "frac": tf / peak_tf, "traffic": None,
                                      "flops_per_launch": flops_exec,
                                      "note": "executed flops (whole 128 x 128 tiles, diagonal tiles included) over the "
                                              "kernel's own time; peak = burst bf16 GEMM rate (kernel timed alone). The kernel "
                                              "is bound by the exponentials: 16,384 per tile at 16 per clock per SM = 0.54 us "
                                              "against 0.28 us of MMA per tile"},
                         "tcgen05_attention_ms": tc_ms, "tcgen05_attention_causal_tflops": flops / (tc_ms / 1e3) / 1e12,
                         "separate_kv_pooling_ms": pool_ms,
                         "mma_sync_attention_with_fused_pooling_ms": fused_ms,
                         "library_varlen_attention_ms": lib_ms})

    else:  # route-decode: benchmark config 5 per-step routing on one of 8 shards
        b, docs_local = 32, (N_DOCS + 7) // 8
        c = docs_local * CHUNKS_PER_DOC
        n_layers = 4
        banks = make_bank(torch, dev, docs_local, n_layers, seed=9000)
        chunk_doc = torch.arange(1, docs_local + 1, device=dev, dtype=torch.int32).repeat_interleave(CHUNKS_PER_DOC)
        q = torch.nn.functional.normalize(torch.randn((b, HQ, 1, D), generator=g, device=dev), dim=-1).to(torch.bfloat16)
        mask = torch.ones((b, 1), dtype=torch.bool, device=dev)
        keys = torch.empty((b, docs_local + 1), dtype=torch.int32, device=dev)
        status = torch.zeros(4, dtype=torch.int32, device=dev)
        topk_ws = torch.empty((ops.topk_workspace_bytes(b, docs_local + 1, TOP_K) + 7) // 8, dtype=torch.int64, device=dev)
        ev = []

        def step(timed=False):
            for rk in banks:
                qf, bias, s_pad = ops.fold_queries(q, mask, HQ // HKV)
                ops.route_table_reset(keys, docs_local, torch.finfo(torch.bfloat16).min, status)
                if timed:
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                ops.route_scores(qf, bias, b, s_pad, rk, chunk_doc, docs_local, 1.0 / HQ, keys=keys, status=status,
                                 flags=2)
                if timed:
                    e1.record()
                    ev.append((e0, e1))
                ops.topk_select(keys, TOP_K, workspace=topk_ws)
        # the scoring kernel alone, eagerly, with events around each launch
        _time_ms(torch, lambda: step(True), 5, warmup)
        route_ms = statistics.mean([a.elapsed_time(b_) for a, b_ in ev[-5 * n_layers:]])
        # the whole layer-step replayed from a CUDA graph: at ~100 us per layer the Python
        # launch path would otherwise be the bottleneck, as it would be in a real decode loop
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step(False)
        sampler.start()
        ms = _time_ms(torch, graph.replay, 10 * steps, warmup) / n_layers
        clocks = sampler.stop()
        alg = c * HKV * D * 2 + b * HKV * D * 2
        _secondary_line(args, "decode-time routing layer-steps/s (one of 8 shards)", "layer-steps/s", 1e3 / ms, ms,
                        f"benchmark config 5 per-step routing: {b} sequences x 1 token against {c} chunks (400 MB shard), "
                        f"{n_layers} distinct layers rotate", "route_tc_kernel", alg, pk["hbm_gbs"], "hbm", clocks,
                        5 * n_layers * 10 * steps, {"launch": "one CUDA graph per step (fold, reset, score, top-k)",
                                                    "route_kernel_ms": route_ms,
                                               "route_kernel_gbs": alg / (route_ms / 1e3) / 1e9,
                                               "route_kernel_frac": alg / (route_ms / 1e3) / 1e9 / pk["hbm_gbs"]})


# ------------------------------------------------------------------------------------------
# benchmark config 5: end-to-end sparse generation step (Qwen3-4B-shaped decoder, random weights)
# ------------------------------------------------------------------------------------------
def run_generate(args):
    import torch
    import torch.distributed as dist
    from msa_b200.decoder import DecoderShape, SparseDecodeModel
    from msa_b200.memory import AttentionGeometry, Document, ModelConfig
    from msa_b200.service import MSAService

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    n_docs, batch_total, local_ctx, new_tokens = args.docs, 32, 2048, args.new_tokens
    router_ids = list(range(18, 36))
    per = (n_docs + world - 1) // world
    d_lo, d_hi = min(n_docs, rank * per), min(n_docs, (rank + 1) * per)
    docs_local, b = d_hi - d_lo, batch_total // world
    c_local = docs_local * CHUNKS_PER_DOC
    shard_k = TOP_K if world == 1 else 2 * TOP_K
    svc = MSAService(local_rank, None, ModelConfig(doc_top_k=TOP_K, router_layer_idx=",".join(map(str, router_ids))),
                     None, AttentionGeometry(), world_size=world, rank=rank, shard_top_k=shard_k)
    svc.uniform_seqlen = True
    svc.block_desc.init_docs([Document(doc_id=d_lo + i, num_chunks=CHUNKS_PER_DOC) for i in range(docs_local)], dev)
    svc.block_desc.pool_ids_from_docs(dev)
    bank = make_bank(torch, dev, docs_local, len(router_ids), seed=4000 + 100 * rank)
    g_kv = torch.Generator(device=dev)
    g_kv.manual_seed(77 + rank)
    kv = torch.empty((c_local, 2, HKV, D), dtype=torch.bfloat16).pin_memory()
    for c0 in range(0, c_local, 1 << 18):
        n = min(1 << 18, c_local - c0)
        kv[c0:c0 + n].copy_(torch.randn((n, 2, HKV, D), generator=g_kv, device=dev).to(torch.bfloat16))
    for i, layer in enumerate(router_ids):
        svc.blocks[layer].rk, svc.blocks[layer].kv, svc.blocks[layer].kv_device_address = bank[i], kv, kv.data_ptr()
    first = router_ids[0]
    if world > 1:
        svc.router_layer_ids = router_ids[:1]
        svc.share_host_banks(tag=f"gen{os.environ.get('MASTER_PORT', '0')}")
        svc.router_layer_ids = router_ids
        base_, offs_, ln_, kvb = svc._directory
        svc._directory = (base_, offs_, ln_, {layer: kvb[first] for layer in router_ids})
        for layer in router_ids[1:]:
            svc.blocks[layer].kv = svc.blocks[first].kv
    else:
        svc.publish_directory()

    model = SparseDecodeModel(DecoderShape(), svc, router_ids, b, local_ctx, new_tokens + 8,
                              TOP_K * CHUNKS_PER_DOC, dev, seed=10 + rank)

    def sync_all():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    # eager: warm up, then one profiled step for the per-layer breakdown
    for _ in range(2):
        model.step()
    model.probe = {}
    t0 = torch.cuda.Event(enable_timing=True)
    t0.record()
    model.step()
    torch.cuda.synchronize(dev)
    pr, model.probe = model.probe, None
    route_ms = [pr["route_start"][l].elapsed_time(pr["route_end"][l]) for l in router_ids]
    attn_ms = [pr["attn_start"][l].elapsed_time(pr["attn_end"][l]) for l in range(36)]
    svc.check_status()

    def timed_run(with_fetch: bool, pipelined: bool = True):
        """Capture one step in a CUDA graph (eager launches if capture is refused) and time new_tokens steps.
        pipelined: the loop rotated to start at the first router layer (same tokens, one token per call)."""
        model.fetch_enabled = with_fetch
        one_step = model.step_pipelined if pipelined else model.step
        mode = "cuda-graph"
        graph = torch.cuda.CUDAGraph()
        model.prime()
        try:
            with torch.cuda.graph(graph):
                one_step()
            run = graph.replay
        except Exception as e:  # e.g. a collective that cannot be captured
            mode, run, graph = f"eager ({type(e).__name__})", one_step, None
            torch.cuda.synchronize(dev)
        model.reset()
        model.prime()
        for _ in range(3):
            run()
        model.reset()
        model.prime()               # outside the timed region: every timed call still runs all 36 layers
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(new_tokens):
            run()
        e1.record()
        sync_all()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        del graph
        torch.cuda.synchronize(dev)
        return float(t.item()), mode

    timed_run(True)                        # untimed pass: settles lazily initialised communicators and the clocks
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms_total, mode = timed_run(True)
    clocks = sampler.stop() if rank == 0 else None
    ms_plain, _ = timed_run(True, pipelined=False)   # unrotated loop: the fetch has only the rest of its own step
    ms_nofetch, _ = timed_run(False)       # same step without the host fetch: what the fetch may hide behind
    svc.check_status()
    tokens_host = model.tokens.cpu()
    if world > 1:
        svc.close_host_banks()
    if rank == 0:
        value = batch_total * new_tokens / (ms_total / 1e3)
        per_step_bytes = (sum(p_.numel() for l_ in model.layers for p_ in l_.values()) + model.lm_head.numel()) * 2
        print(json.dumps({
            "metric": "sparse generation tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": new_tokens, "warmup": 3, "ms_per_step": ms_total / new_tokens, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"benchmark config 5: Qwen3-4B-shaped decoder (36 layers, hidden 2560, 32q/8kv, d 128, FFN 9728, "
                                   f"vocab 151936, random weights), routing in layers 18-35 every step against {n_docs} docs x "
                                   f"{CHUNKS_PER_DOC} chunks, top-{TOP_K}, batch {batch_total}, {local_ctx}-token local context, "
                                   f"{new_tokens} new tokens", "launch": mode,
                       "parallelism": f"sequences and bank split over {world} rank(s); weights replicated"},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                    "note": "tokens are produced and consumed on the device; the only host traffic is the K/V fetch",
                    "host_to_device_fetch_bytes_per_step": 18 * batch_total * TOP_K * CHUNKS_PER_DOC * 2 * HKV * D * 2},
            "per_layer": {"routing_ms_avg": sum(route_ms) / len(route_ms), "attention_ms_avg": sum(attn_ms) / len(attn_ms),
                          "measured": "eager step, CUDA events"},
            "fetch": {"ms_per_step_with_fetch": ms_total / new_tokens, "ms_per_step_without_fetch": ms_nofetch / new_tokens,
                      "ms_per_step_unrotated_loop": ms_plain / new_tokens,
                      "loop": "rotated to start at the first router layer: layers 18-35 of step t, sampling, layers 0-17 "
                              "of step t+1; the fetch issued in step t is needed by layer 18 of step t+1",
                      "exposed_ms_per_step": max(0.0, (ms_total - ms_nofetch) / new_tokens),
                      "note": "the run without the fetch is a diagnostic; on 8 GPUs it has measured slower than the run with it",
                      "pcie_bytes_per_step_per_gpu": 18 * b * TOP_K * CHUNKS_PER_DOC * 2 * HKV * D * 2},
            "dense_weight_bytes_per_step": per_step_bytes, "clocks": clocks,
            # this package's kernels per step: per layer add+norm x2, q/k norm+rope, decode attention (+ combine),
            # SiLU*up; per router layer fold, table fill, scoring, top-k x2, merge, gather plan, gather; final norm
            "gpu_launches": new_tokens * (36 * 5 + 18 * 8 + 1), "last_tokens": tokens_host[:4].tolist()}), flush=True)
    if world > 1:
        # graphs that captured NCCL kernels were alive in this process: leave without tearing the
        # communicator down (its destructor can wait forever on them)
        dist.barrier()
        torch.cuda.synchronize(dev)
        sys.stdout.flush()
        os._exit(0)


if __name__ == "__main__":
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    elif a.workload == "generate":
        run_generate(a)
    elif a.workload != "routing":
        run_secondary(a)
    else:
        run_ours(a)

#!/usr/bin/env python
"""Benchmark of the batched graph beam search (one JSON line on rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3|c2|c1|c4|c5|small]
    python bench.py --impl reference ...      # the reference's CPU best-first search, host cores

A step is one pass of the search over the workload's whole query batch.  The index is built in
this process by the library itself, the way the reference builds it: exact k_b nearest base points
of the training queries (tensor cores), neighbourhood-aware projection, connectivity enhancement,
16 entry points by farthest-point sampling.

Replicated workloads (c1, c2, c3, small): with N GPUs every rank holds the whole index and searches
1/N of the batch -- the N-th part of the batch in its locality ORDER (every rank computes the same
deterministic order of the whole batch), no collective on the data path, total work fixed (strong
scaling).  With N > 1 the run ends with a short sharded leg (one 1M-point shard per GPU, all queries
on every shard, one NCCL all-gather, slice merge), checked against the CPU oracle's merge and
reported under config.sharded_check.  Sharded workload (c4): every rank holds one 12.5M-point shard
with its own graph and searches ALL queries (weak scaling: the index grows with N).

value : queries/s with index and queries resident in HBM, device pointers in and out
        (coral_search_async), CUDA events on the launching stream, max over ranks.
e2e   : queries/s through coral_search with pinned HOST queries in and HOST ids out, the
        copies inside the timed region.
Inputs are seeded synthetic data of the named shapes (coral_b200/synth.py); the index (vectors +
adjacency) is far larger than L2, so no cache flush is needed between iterations.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # data: a configuration of coral_b200.synth.CONFIGS; n: base points (per shard when sharded)
    "c1": dict(data="c1", n=1_000_000, q=10_000, k=10, Ls=[64, 128, 256, 512], train=100_000),
    "c2": dict(data="c2", n=1_000_000, q=10_000, k=10, Ls=[64, 128, 256], train=100_000),
    "c3": dict(data="c3", n=10_000_000, q=100_000, k=10, Ls=[64, 128, 256], train=100_000),
    "c4": dict(data="c4", n=12_500_000, q=100_000, k=100, Ls=[128, 256], train=100_000, sharded=True),
    "small": dict(data="c3", n=1_000_000, q=8_192, k=10, Ls=[64], train=100_000),
    # small-batch latency on the c3 index: batches of 1, 8, 64, 512 queries, L=128
    "c5": dict(data="c3", n=10_000_000, q=8_192, k=10, Ls=[128], train=100_000, latency=[1, 8, 64, 512]),
}
METRIC = "QPS @ recall@10>=0.95, 10Mx512 IP"


def metric_name(workload, w):
    """The headline metric's name for the workload it is quoted on (c3 and its small-batch leg);
    the other workloads are named after their own shape so that a line cannot be mistaken for it."""
    if workload in ("c3", "c5"):
        return METRIC
    from coral_b200 import synth
    cfg = synth.CONFIGS[w["data"]]
    n = w["n"]
    size = f"{n // 1_000_000}M" if n % 1_000_000 == 0 else (f"{n / 1e6:g}M" if n >= 1_000_000 else str(n))
    return (f"QPS @ recall@{w['k']}>=0.95, {size}x{cfg['dim']} {cfg['kind'].upper()}"
            + (" per shard, sharded" if w.get("sharded") else ""))
PEAK_FALLBACK_GBS = 6650.0
# DRAM bytes per algorithmic byte of the search kernel, from the ncu capture of the 1M x 512 case
# summarised under profiles/ (a profile constant, not a measurement of this run): workload -> ratio.
# The 10M x 512 workloads use the same ratio: with a 23 GB index L2 serves less of the gather than
# with 2.3 GB, so for them the figure is a lower bound of the DRAM share.
DRAM_PER_ALGORITHMIC_BYTE = {"small": 0.748, "c3": 0.748}


_RESULT_FD = None


def claim_stdout():
    """Keeps the process's standard output for the one result line: everything else that writes to
    file descriptor 1 from here on (libraries such as NCCL print banners there) goes to stderr."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def emit(obj):
    line = (json.dumps(obj) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(line.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, line)


def log(*a):
    print(*a, file=sys.stderr, flush=True)


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return PEAK_FALLBACK_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        time.sleep(0.15)
        self.proc.terminate()
        clocks, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                clocks.append(float(r[0]))
                mx = float(r[1])
                for nm, v in zip(names, r[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(nm)
            except Exception:
                continue
        clocks.sort()
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(clocks)}


def build_index(w, local, rank=0, seed=20260001, n_test=None, extra=0):
    """Seeded synthetic data of the workload and the index over it, built by the library on this GPU
    (of this rank's shard when sharded).  `extra` more points of the same distribution are kept behind
    the indexed rows, to be inserted later.  Returns (dataset, index handle, build info)."""
    import torch
    from coral_b200 import capi, synth
    t0 = time.time()
    draw = seed + 1000 + rank if w.get("sharded") else None
    cfg = synth.CONFIGS[w["data"]]
    ds = synth.make_config(w["data"], w["train"], n_test or w["q"], n=w["n"] + extra, seed=seed, device=f"cuda:{local}",
                           draw_seed=draw)
    ix = capi.Index(w["n"] + extra, cfg["dim"], cfg["deg"], cfg["kind"], device=local)
    ix.attach_vectors(ds.base)
    if extra:
        ix.set_live(w["n"])
    t1 = time.time()
    info = ix.build(ds.train, kb=100)
    torch.cuda.synchronize()
    info.update(data_s=round(t1 - t0, 1), build_s=round(time.time() - t1, 1), knn_tflops=round(ix.last_dense_tflops, 1))
    log(f"[bench] rank {rank}: {w['data']} n={w['n']}: data {info['data_s']}s, build {info['build_s']}s "
        f"({info['isolated']} isolated nodes enhanced)")
    ds.train = None
    torch.cuda.empty_cache()
    return ds, ix, info


def cpu_reference(base_h, adj_h, start_h, queries_h, gt_h, L0, k, max_L=1024, threads=0, repeat=1):
    """The reference's CPU best-first search at the metric's recall: L is doubled from L0 until
    recall@k on the ground-truth sample reaches 0.95 (the reference's own driver sweeps L the same
    way, tests/test_search_pipeline.cpp:283-310).  Returns the report dict."""
    from oracle import oracle
    threads = threads or (os.cpu_count() or 1)
    out, L = {}, L0
    same_L = None
    while True:
        best = None
        for _ in range(repeat):
            ids, _, hops, secs, kind, used = oracle.cpu_search(base_h, adj_h, start_h, queries_h, L, k, threads=threads)
            best = secs if best is None else min(best, secs)
        m = min(len(queries_h), len(gt_h))
        rec = oracle.recall(ids[:m], gt_h[:m], k)
        row = {"L": L, "qps": len(queries_h) / best, "recall": rec, "seconds": best}
        if same_L is None:
            same_L = row
        out = row
        if rec >= 0.95 or L * 2 > max_L:
            break
        L *= 2
    return {"value": out["qps"], "unit": "queries/s", "cores": used, "kind": kind, "L": out["L"], "recall": out["recall"],
            "reached_recall_target": out["recall"] >= 0.95, "at_same_L": same_L,
            "sample": (f"first {len(queries_h)} queries, k={k}, L doubled from {L0} until recall@{k} >= 0.95: L={out['L']}, "
                       f"recall {out['recall']:.4f}, {out['seconds']:.2f}s per pass; "
                       + ("reference NeighborPriorityQueue + AVX-512 DistanceL2 with the search_in_cpu loop restated"
                          if kind == "reference" else "self-contained port of search_in_cpu"))}


def reference_gpu_kernel(ix, base_h, adj_h, start_h, queries_h, gt_h, L, k, metric, max_degree):
    """The reference's own search kernel (its sources compiled unmodified for sm_100a under
    oracle/_ref) on the same graph, entry points, queries and L, timed over the reference's own window
    (src/search_gpu.cu:861-877).  Reported beside the CPU baseline; None when that build is absent.
    The reference kernel reads out of range for a query whose beam never fills, so it only runs after
    this library's search reported status 0 for every query of the sample."""
    import numpy as np
    from oracle import oracle
    if not oracle.have_ref_gpu():
        return None
    try:
        _, _, st, _ = ix.search(queries_h, L, k, dists=False, stats=True)
        if int(np.abs(st[:, 0]).max()) != 0:
            return {"value": None, "unit": "queries/s", "sample": "skipped: a query of the sample did not fill its beam"}
        best, ids = None, None
        with oracle.RefGpuIndex(base_h, adj_h, start_h, metric, max_degree=max_degree) as ref:
            for _ in range(2):
                ids, _, hops, secs = ref.search(queries_h, L, k)
                best = secs if best is None else min(best, secs)
        m = min(len(queries_h), len(gt_h))
        return {"value": len(queries_h) / best, "unit": "queries/s", "L": L, "recall": oracle.recall(ids[:m], gt_h[:m], k),
                "seconds": best, "hops": hops,
                "sample": f"first {len(queries_h)} queries, best of 2 calls of GPUFuncs::search_gpu (4096 persistent CTAs x 512 threads), "
                          "kernel + hop-count copy as the reference times it, queries and results resident on the device"}
    except Exception as e:
        return {"value": None, "unit": "queries/s", "sample": f"failed: {e}"}


def run_reference(args, w, rank, world):
    """bench.py --impl reference: the reference's CPU search on this box's host cores, rank 0 only."""
    if rank != 0:
        return
    import torch
    if not torch.cuda.is_available():
        emit({"impl": "reference", "unavailable": "the index for the CPU arm is built with the library's GPU "
              "builder; no CUDA device here"})
        return
    from coral_b200 import synth
    ds, ix, info = build_index(w, 0)
    k = w["k"]
    n_gt = min(2000, w["q"])
    gt = ix.exact_knn(ds.test[:n_gt], k, dists=False)[0].cpu().numpy()
    base, adj, start = ds.base.cpu().numpy(), ix.get_adjacency(), ix.get_start_ids()
    test = ds.test.cpu().numpy()
    ix.close()
    sample = min(args.cpu_queries, w["q"])
    L0 = args.L or w["Ls"][0]
    reps = []
    for it in range(args.warmup + args.steps):
        r = cpu_reference(base, adj, start, test[:sample], gt, L0, k)
        if it >= args.warmup:
            reps.append(r)
    qps = sum(r["value"] for r in reps) / len(reps)
    r = reps[-1]
    cfg = synth.CONFIGS[w["data"]]
    out = {
        "impl": "reference", "metric": metric_name(args.workload, w), "value": qps, "unit": "queries/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sample / qps * 1e3, "higher_is_better": True,
        "scaling": "weak" if w.get("sharded") else "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "n": w["n"], "dim": cfg["dim"], "metric": cfg["kind"], "max_degree": cfg["deg"],
                   "queries_per_step": sample, "k": k, "L": r["L"], "recall": r["recall"],
                   "graph": "built by the library (k-NN lists -> NAP -> CE), the same graph as the GPU arm"},
        "cpu_baseline": dict(r, value=qps),
        "e2e": {"value": qps, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(out)


def run_latency(args, w, ix, ds, device, rank):
    """Small-batch latency: per batch size, p50/p99 over many batches, device-resident (CUDA events
    around coral_search_async) and end to end (coral_search, pinned host queries in, host ids out)."""
    import numpy as np
    import torch
    from coral_b200 import capi, synth
    cfg = synth.CONFIGS[w["data"]]
    L, k, dim = args.L or w["Ls"][0], w["k"], cfg["dim"]
    lib, handle = capi.load(), ix._h
    n_gt = 2000
    gt = ix.exact_knn(ds.test[:n_gt], k, dists=False)[0]
    ids, _, _, _ = ix.search(ds.test[:n_gt], L, k, dists=False)
    recall = ix.count_hits(ids, gt, k) / float(k * n_gt)
    stream = torch.cuda.Stream(device=device)
    h_all = ds.test.cpu().pin_memory()
    launches0 = ix.launch_count

    def measure():
        table = {}
        for B in w["latency"]:
            d_ids = torch.empty((B, k), dtype=torch.int32, device=device)
            h_ids = torch.empty((B, k), dtype=torch.int32).pin_memory()
            n_batches = max(20, min(200, w["q"] // B))
            dev_us, e2e_us = [], []
            hops = C.c_int64(0)
            for i in range(n_batches + args.warmup):
                s = (i * B) % (w["q"] - B + 1)
                q = ds.test[s:s + B]
                ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ev0.record(stream)
                ix.search_async(q, L, k, d_ids, None, None, stream.cuda_stream)
                ev1.record(stream)
                stream.synchronize()
                hq = h_all[s:s + B].numpy()
                t0 = time.perf_counter()
                rc = lib.coral_search(handle, C.c_void_p(hq.ctypes.data), B, L, k, C.c_void_p(h_ids.numpy().ctypes.data),
                                      None, None, C.byref(hops))
                t1 = time.perf_counter()
                if rc != 0:
                    raise RuntimeError(lib.coral_last_error(handle).decode())
                if i >= args.warmup:
                    dev_us.append(ev0.elapsed_time(ev1) * 1e3)
                    e2e_us.append((t1 - t0) * 1e6)
            ix.check()
            table[B] = {"p50_us": float(np.percentile(dev_us, 50)), "p99_us": float(np.percentile(dev_us, 99)),
                        "e2e_p50_us": float(np.percentile(e2e_us, 50)), "e2e_p99_us": float(np.percentile(e2e_us, 99)),
                        "qps": B / float(np.percentile(dev_us, 50)) * 1e6, "batches": n_batches,
                        "ctas_per_query": ix.get_option("last_cluster_size")}
        return table

    table = measure()
    ref_latency = None
    if rank == 0 and not args.no_cpu_baseline:
        ref_latency = reference_gpu_latency(ix, ds, w, L, k, cfg)
    # Second leg: 10 % of the points deleted with topology repair, then 5 % new points inserted with
    # neighbours from the same search kernel at L = 128 (src/index_gpu.cpp:138-224), then the same batches.
    n, extra = w["n"], w["n"] // 20
    rng = np.random.default_rng(77)
    del_ids = rng.choice(n, n // 10, replace=False).astype(np.int32)
    dead = np.zeros(n + extra, bool)
    dead[del_ids] = True
    t0 = time.time()
    ix.update_begin()
    ix.delete(del_ids)
    torch.cuda.synchronize()
    t_del = time.time() - t0
    t0 = time.time()
    ix.insert(n, extra, kb=100, L=128, batch=32768)
    torch.cuda.synchronize()
    t_ins = time.time() - t0
    ix.build_end()
    ix.prepare(max(w["q"], n_gt), L, 4 * k)
    gt_wide = ix.exact_knn(ds.test[:n_gt], 4 * k, dists=False)[0].cpu().numpy()      # over all live rows
    gt_alive = np.stack([row[~dead[row]][:k] for row in gt_wide])
    ids_d, _, _, _ = ix.search(ds.test[:n_gt], L, k, dists=False)
    ids_d = ids_d.cpu().numpy() if hasattr(ids_d, "cpu") else np.asarray(ids_d)
    assert not dead[ids_d[ids_d >= 0]].any(), "a deleted id was returned"
    recall_deleted = float(np.mean([len(set(a) & set(b)) / k for a, b in zip(ids_d, gt_alive)]))
    inserted_found = float(np.mean((ids_d >= n).any(1)))
    table_deleted = measure()
    if rank == 0:
        b1 = table[w["latency"][0]]
        out = {"metric": "p50 latency of one query batch, 10Mx512 IP, L=%d" % L, "value": b1["p50_us"], "unit": "us",
               "n_gpus": 1, "steps": b1["batches"], "warmup": args.warmup, "ms_per_step": b1["p50_us"] * 1e-3,
               "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
               "config": {"workload": args.workload, "n": w["n"], "dim": dim, "metric": cfg["kind"], "max_degree": cfg["deg"],
                          "k": k, "L": L, "recall": recall, "batch_sizes": w["latency"], "latency": table,
                          "reference_gpu_kernel_latency": ref_latency,
                          "after_10pct_delete_with_repair_and_5pct_insert": {
                              "latency": table_deleted, "recall": recall_deleted, "delete_s": round(t_del, 1),
                              "insert_s": round(t_ins, 1), "insert_batch": 32768,
                              "queries_with_an_inserted_point_in_their_top_k": inserted_found},
                          "l2_policy": "inputs larger than L2; every batch uses different queries"},
               "e2e": {"value": b1["e2e_p50_us"], "unit": "us", "h2d_bytes_per_step": dim * 4 * w["latency"][0],
                       "d2h_bytes_per_step": k * 4 * w["latency"][0] + 32},
               "gpu_launches": int(ix.launch_count - launches0)}
        emit(out)


def reference_gpu_latency(ix, ds, w, L, k, cfg, batches=10):
    """p50 of the reference's own search kernel (oracle/_ref, its sources compiled unmodified) per batch
    size on the same index, entry points and queries: the reference's timed window, queries and results
    on the device.  None when that build is absent; batches whose queries do not all fill their beam
    are skipped (the reference kernel reads out of range for those)."""
    import numpy as np
    from oracle import oracle
    if not oracle.have_ref_gpu():
        return None
    try:
        out = {}
        with oracle.RefGpuIndex(ds.base.cpu().numpy(), ix.get_adjacency(), ix.get_start_ids(), cfg["kind"],
                                max_degree=cfg["deg"]) as ref:
            for B in w["latency"]:
                us = []
                for i in range(batches + 2):
                    s0 = (i * B) % (w["q"] - B + 1)
                    q = ds.test[s0:s0 + B].cpu().numpy()
                    _, _, st, _ = ix.search(q, L, k, dists=False, stats=True)
                    if int(np.abs(st[:, 0]).max()) != 0:
                        continue
                    _, _, _, secs = ref.search(q, L, k)
                    if i >= 2:
                        us.append(secs * 1e6)
                out[B] = {"p50_us": float(np.percentile(us, 50)), "batches": len(us)} if us else None
        return out
    except Exception as e:
        return {"failed": str(e)}


def quick_workload(name, local, steps=3, warmup=2):
    """One small extra workload measured inside the default run: builds, picks the first configured
    L with recall >= 0.95, times the device-resident search.  Returns a dict for config.extra."""
    import numpy as np
    import torch
    from coral_b200 import capi, synth
    w = WORKLOADS[name]
    cfg = synth.CONFIGS[w["data"]]
    ds, ix, info = build_index(w, local)
    Q, k = w["q"], w["k"]
    n_gt = min(2000, Q)
    gt = ix.exact_knn(ds.test[:n_gt], k, dists=False)[0]
    ix.prepare(Q, max(w["Ls"]), k)
    out = {"build_s": info["build_s"], "by_L": {}}
    peak, _ = measured_peak()
    d_ids = torch.empty((Q, k), dtype=torch.int32, device=ds.test.device)
    d_stats = torch.empty((Q, capi.STATS_W), dtype=torch.int32, device=ds.test.device)
    stream = torch.cuda.Stream(device=ds.test.device)
    chosen = None
    for L in w["Ls"]:
        ix.search_async(ds.test, L, k, d_ids, None, d_stats, stream.cuda_stream)
        stream.synchronize()
        rec = ix.count_hits(d_ids[:n_gt], gt, k) / float(k * n_gt)
        st = d_stats.cpu().numpy().astype(np.int64)
        alg = float((st[:, 1] * cfg["dim"] * 4 + st[:, 2] * ix.get_option("deg_pad") * 4 + cfg["dim"] * 4 + k * 8).sum())
        for _ in range(warmup):
            ix.search_async(ds.test, L, k, d_ids, None, None, stream.cuda_stream)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        for _ in range(steps):
            ix.search_async(ds.test, L, k, d_ids, None, None, stream.cuda_stream)
        ev1.record(stream)
        stream.synchronize()
        ix.check()
        ms = ev0.elapsed_time(ev1) / steps
        out["by_L"][L] = {"qps": Q / (ms * 1e-3), "recall": rec, "alg_gbs": alg / (ms * 1e-3) / 1e9,
                          "frac": alg / (ms * 1e-3) / 1e9 / peak}
        if chosen is None and rec >= 0.95:
            chosen = L
    out["L"] = chosen
    ix.close()
    del ds
    torch.cuda.empty_cache()
    return out


def sharded_check(local, rank, world, comm):
    """A short sharded leg at the end of a replicated multi-GPU run: one 1M x 200 shard per GPU
    (config 4's data), all queries on every shard, k = 100, L = 128, through coral_search_sharded.
    Parity: the merged slice of every rank equals the CPU oracle's merge of the per-shard results
    (checked on rank 0 for its own slice) and per-shard results equal the oracle's search."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from coral_b200 import sharded
    from oracle import oracle
    w = dict(data="c4", n=1_000_000, q=4_096, k=100, Ls=[128], train=100_000, sharded=True)
    ds, ix, info = build_index(w, local, rank)
    Q, k, L = w["q"], w["k"], 128
    id_map = torch.from_numpy(sharded.interleaved_ids(w["n"], world, rank)).to(ds.test.device)
    ix.prepare(Q, L, k)
    sh = sharded.ShardedIndex(ix, id_map, comm)
    stream = torch.cuda.Stream(device=ds.test.device)
    torch.cuda.synchronize()
    out_buf = None
    for _ in range(2):
        ids, d, lo, hi = sh.search(ds.test, L, k, stream.cuda_stream, out_buf)
        out_buf = (ids, d)
    stream.synchronize()
    dist.barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    steps = 3
    for _ in range(steps):
        sh.search(ds.test, L, k, stream.cuda_stream, out_buf)
    ev1.record(stream)
    stream.synchronize()
    ix.check()
    ms = torch.tensor([ev0.elapsed_time(ev1) / steps], dtype=torch.float64, device=ds.test.device)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    # parity: every rank sends its local (global-id) results of a query sample to rank 0 through torch
    sample = np.arange(lo, hi)[:64] if hi > lo else np.arange(0)
    loc_ids, loc_d, _, _ = ix.search(ds.test, L, k)
    gl = torch.where(loc_ids >= 0, id_map[loc_ids.clamp(min=0).long()], loc_ids)
    all_ids = [torch.empty_like(gl) for _ in range(world)]
    all_d = [torch.empty_like(loc_d) for _ in range(world)]
    dist.all_gather(all_ids, gl)
    dist.all_gather(all_d, loc_d)
    ok = True
    if len(sample):
        o_ids, o_d = oracle.merge_shards(torch.stack(all_ids)[:, sample].cpu().numpy(),
                                         torch.stack(all_d)[:, sample].cpu().numpy(), "l2")
        mine_ids, mine_d = ids.cpu().numpy()[sample - lo], d.cpu().numpy()[sample - lo]
        ok = bool(np.array_equal(mine_ids, o_ids) and np.array_equal(mine_d.view(np.uint32), o_d.view(np.uint32)))
        # this shard's own search against the oracle on a few queries
        base_h, adj_h, start_h = ds.base.cpu().numpy(), ix.get_adjacency(), ix.get_start_ids()
        r_ids, r_d, _ = oracle.search(base_h, adj_h, start_h, ds.test[:16].cpu().numpy(), L, k, "l2")
        ok = ok and bool(np.array_equal(loc_ids[:16].cpu().numpy(), r_ids))
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=ds.test.device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    ix.close()
    return {"shards": world, "points_per_shard": w["n"], "queries": Q, "k": k, "L": L, "qps": Q / (float(ms.item()) * 1e-3),
            "ms_per_step": float(ms.item()), "merged_equals_oracle_merge": bool(flag.item()),
            "exchange": "one ncclAllGather of ids+distances, each rank merges its slice (coral_search_sharded)"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS))
    ap.add_argument("--L", type=int, default=0, help="beam capacity; 0 = smallest configured L with recall >= 0.95")
    ap.add_argument("--queries", type=int, default=0, help="override the workload's query batch (profiling)")
    ap.add_argument("--n", type=int, default=0, help="override the number of base points (per shard)")
    ap.add_argument("--cpu-queries", type=int, default=4000, help="query sample of the CPU baseline")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the extra c1/c2 workloads and the sharded leg")
    ap.add_argument("--option", action="append", default=[], help="kernel tuning knob name=value")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)
    claim_stdout()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    w = dict(WORKLOADS[args.workload])
    if args.queries:
        w["q"] = args.queries
    if args.n:
        w["n"] = args.n
    sharded_mode = bool(w.get("sharded"))

    if args.impl == "reference":
        run_reference(args, w, rank, world)
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    from coral_b200 import capi, sharded, synth

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the search path has no CPU fallback")
    torch.cuda.set_device(local)
    device = f"cuda:{local}"
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # The only collectives here are barriers, scalar reductions and one all-gather of a few MB per
        # step in the sharded workloads: in-switch reduction buys nothing, and every figure of this
        # repository was measured with plain peer transport.  An explicit setting wins.
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        # NCCL writes its version banner to stdout at NCCL_DEBUG=VERSION; stdout is for the one JSON line
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(device))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce_ranks(x: float, op) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=op)
        return float(t.item())

    cfg = synth.CONFIGS[w["data"]]
    extra_rows = w["n"] // 20 if w.get("latency") else 0
    ds, ix, build_info = build_index(w, local, rank, extra=extra_rows)   # replicated: same seed on every rank; sharded: own shard
    Q, k, dim = w["q"], w["k"], cfg["dim"]
    for kv in args.option:
        name, val = kv.split("=")
        ix.set_option(name, int(val))
    n_gt = min(2000, Q)
    comm = sharded.Communicator.from_torch(local) if world > 1 or sharded_mode else None
    id_map = torch.from_numpy(sharded.interleaved_ids(w["n"], world, rank)).to(device) if sharded_mode else None
    ix.prepare(Q, max(w["Ls"] + [args.L]), k)
    torch.cuda.synchronize()
    sh = sharded.ShardedIndex(ix, id_map, comm) if sharded_mode else None
    stream = torch.cuda.Stream(device=device)

    if w.get("latency"):
        run_latency(args, w, ix, ds, device, rank)
        ix.close()
        return

    # ---- ground truth (exact, tensor-core scan + exact re-rank) for the first n_gt queries; global when sharded
    gt_ids, gt_d, _ = ix.exact_knn(ds.test[:n_gt], k)
    if sharded_mode:
        ix.map_ids(gt_ids, id_map)
        torch.cuda.synchronize()
        a_ids, a_d = sharded.all_gather_results(gt_ids, gt_d)
        torch.cuda.synchronize()
        gt_ids, _ = ix.merge_shards(a_ids, a_d)
        torch.cuda.synchronize()

    # ---- beam capacity: smallest configured L whose recall@k on the ground-truth sample reaches 0.95
    recalls, L = {}, args.L
    for cand in ([args.L] if args.L else w["Ls"]):
        if sharded_mode:
            ids, _, lo_, hi_ = sh.search(ds.test[:n_gt], cand, k)
            torch.cuda.synchronize()
            hits = torch.tensor([ix.count_hits(ids, gt_ids[lo_:hi_], k) if hi_ > lo_ else 0], dtype=torch.float64, device=device)
            if world > 1:
                dist.all_reduce(hits)
            recalls[cand] = float(hits.item()) / float(k * n_gt)
        else:
            ids, _, _, _ = ix.search(ds.test[:n_gt], cand, k, dists=False)
            recalls[cand] = ix.count_hits(ids, gt_ids, k) / float(k * n_gt)
        L = cand
        if recalls[cand] >= 0.95:
            break
    log(f"[bench] rank {rank}: recall by L {recalls}, using L={L}")

    # ---- this rank's part of the batch
    if sharded_mode:
        my_rows = None
        my_q = ds.test
        lo, hi = sharded.query_slice(Q, world, rank)
        nq, n_out = Q, hi - lo
    else:
        if world > 1:
            # every rank orders the whole batch (deterministic, identical everywhere) and takes its range
            order = ix.query_order(ds.test)
            torch.cuda.synchronize()
            my_rows = sharded.sorted_slice(order, world, rank).long()
            my_q = ds.test[my_rows].contiguous()
        else:
            my_rows = None
            my_q = ds.test
        nq = n_out = int(my_q.shape[0])

    d_ids = torch.empty((n_out, k), dtype=torch.int32, device=device)
    d_dists = torch.empty((n_out, k), dtype=torch.float32, device=device) if sharded_mode else None
    d_stats = torch.empty((nq, capi.STATS_W), dtype=torch.int32, device=device)
    h_q = my_q.cpu().pin_memory()
    h_ids = torch.empty((n_out, k), dtype=torch.int32).pin_memory()
    h_q_np, h_ids_np = h_q.numpy(), h_ids.numpy()
    lib, handle = capi.load(), ix._h

    def device_step():
        if sharded_mode:
            sh.search(my_q, L, k, stream.cuda_stream, (d_ids, d_dists))
        else:
            ix.search_async(my_q, L, k, d_ids, None, None, stream.cuda_stream)

    # ---- algorithmic bytes of one step (deterministic for the query set): untimed pass with counters
    scratch_ids = torch.empty((nq, k), dtype=torch.int32, device=device)
    ix.search_async(my_q, L, k, scratch_ids, None, d_stats, stream.cuda_stream)
    stream.synchronize()
    ix.check()
    st = d_stats.cpu().numpy().astype(np.int64)
    row_bytes, deg_pad = dim * 4, ix.get_option("deg_pad")
    alg_bytes = float((st[:, 1] * row_bytes + st[:, 2] * deg_pad * 4 + row_bytes + k * 8).sum())
    del scratch_ids

    # ---- device-resident timing
    for _ in range(args.warmup):
        device_step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = ix.launch_count
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for _ in range(args.steps):
        device_step()
    ev1.record(stream)
    barrier()
    ix.check()
    launches = ix.launch_count - launches0
    clocks = sampler.stop() if rank == 0 else None
    my_ms = ev0.elapsed_time(ev1) / args.steps
    dev_ms = reduce_ranks(my_ms, dist.ReduceOp.MAX)
    fastest_ms = reduce_ranks(my_ms, dist.ReduceOp.MIN)
    ref_ids = d_ids.cpu().numpy()

    # ---- end to end: pinned host queries in, host ids out
    hops = C.c_int64(0)

    def e2e_step():
        if sharded_mode:
            with torch.cuda.stream(stream):
                dq = h_q.to(device, non_blocking=True)
            rc = lib.coral_search_sharded(handle, comm._c, C.c_void_p(id_map.data_ptr()), C.c_void_p(dq.data_ptr()), nq, L, k,
                                          C.c_void_p(h_ids_np.ctypes.data), None, C.c_void_p(stream.cuda_stream))
            if rc != 0:
                raise RuntimeError(lib.coral_comm_last_error(comm._c).decode())
            return
        rc = lib.coral_search(handle, C.c_void_p(h_q_np.ctypes.data), nq, L, k, C.c_void_p(h_ids_np.ctypes.data),
                              None, None, C.byref(hops))
        if rc != 0:
            raise RuntimeError(lib.coral_last_error(handle).decode())

    for _ in range(min(args.warmup, 2)):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_ms = reduce_ranks((time.perf_counter() - t0) * 1e3, dist.ReduceOp.MAX) / args.steps
    if not np.array_equal(h_ids_np, ref_ids):
        raise SystemExit("host-pointer and device-pointer searches disagree")

    total_alg = reduce_ranks(alg_bytes, dist.ReduceOp.SUM)
    peak, peak_kind = measured_peak()
    achieved = reduce_ranks(alg_bytes / (my_ms * 1e-3) / 1e9, dist.ReduceOp.MIN)   # per GPU, against one GPU's peak

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            sample = min(args.cpu_queries, Q)
            base_h, adj_h, start_h = ds.base.cpu().numpy(), ix.get_adjacency(), ix.get_start_ids()
            q_h, g_h = ds.test[:sample].cpu().numpy(), gt_ids[:min(sample, n_gt)].cpu().numpy()
            cpu = cpu_reference(base_h, adj_h, start_h, q_h, g_h, L, k)
            cpu["reference_gpu_kernel"] = reference_gpu_kernel(ix, base_h, adj_h, start_h, q_h, g_h, L, k, cfg["kind"], cfg["deg"])
            del base_h, adj_h
        except Exception as e:  # the baseline is a report, never a reason to lose the measurement
            cpu = {"value": None, "unit": "queries/s", "cores": 0, "kind": "port", "sample": f"failed: {e}"}

    index_gb = w["n"] * (row_bytes + deg_pad * 4) / 1e9
    plan = {n_: ix.get_option(n_) for n_ in ("plan_stages", "plan_chunk_bytes", "plan_smem_bytes", "plan_hash_bits",
                                               "plan_ctas_per_sm", "plan_warps")}
    ix.close()
    del ds
    torch.cuda.empty_cache()

    extra, shard_leg = None, None
    if not args.no_extra and args.workload == "c3" and not args.queries and not args.n:
        if world == 1:
            extra = {}
            for name in ("c2", "c1"):
                try:
                    extra[name] = quick_workload(name, local)
                except Exception as e:
                    extra[name] = {"failed": str(e)}
        else:
            try:
                shard_leg = sharded_check(local, rank, world, comm)
            except Exception as e:
                shard_leg = {"failed": str(e)}

    if rank == 0:
        ratio = DRAM_PER_ALGORITHMIC_BYTE.get(args.workload)
        out = {
            "metric": metric_name(args.workload, w), "value": Q / (dev_ms * 1e-3), "unit": "queries/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dev_ms, "higher_is_better": True,
            "scaling": "weak" if sharded_mode else "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "n": w["n"] * (world if sharded_mode else 1), "dim": dim,
                       "metric": cfg["kind"], "max_degree": cfg["deg"], "queries_per_step": Q, "k": k, "L": L,
                       "recall": recalls[L], "recall_by_L": recalls, "entry_points": 16,
                       "graph": "built in this run by the library: tensor-core exact k-NN lists of 100k training queries "
                                "(k_b=100) -> NAP -> CE -> 16 FPS entry points",
                       "build": build_info,
                       "parallelism": (f"{world} shards of {w['n']} points, all queries on every shard, one NCCL "
                                       f"all-gather + slice merge" if sharded_mode else
                                       f"replicated index, locality-ordered batch split x{world}"),
                       "kernel_ms_per_rank": {"min": fastest_ms, "max": dev_ms},
                       "l2_policy": "inputs larger than L2 (index %.1f GB per GPU)" % index_gb,
                       "plan": plan, "extra_workloads": extra, "sharded_check": shard_leg},
            "e2e": {"value": Q / (e2e_ms * 1e-3), "unit": "queries/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": nq * dim * 4 * world, "d2h_bytes_per_step": (n_out * k * 4 + 32) * world},
            "gpu_launches": int(launches * world),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": peak_kind,
                         "traffic": (ratio * alg_bytes if ratio and world == 1 else None),
                         "traffic_source": (("profile constant: 0.748 DRAM bytes per algorithmic byte in the ncu capture of the "
                                             "1M x 512 case (profiles/), scaled to this launch by its algorithmic bytes"
                                             + ("; a lower bound at 10M, where L2 serves less" if w["n"] > 1_000_000 else ""))
                                            if ratio else None),
                         "dram_frac": (ratio * achieved / peak if ratio else None),
                         "algorithmic_bytes_per_step": total_alg, "kernel": "beam_search_kernel",
                         "note": "per GPU (slowest rank); frac = ALGORITHMIC bytes (n_dist*dim*4 + n_exp*deg_pad*4 + dim*4 "
                                 "+ k*8 per query) / time / measured copy peak -- part of those bytes is served by L2, "
                                 "dram_frac = the DRAM share of it"},
            "cpu_baseline": cpu,
            "clocks": clocks,
        }
        emit(out)
    if comm is not None:
        comm.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

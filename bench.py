#!/usr/bin/env python
"""Benchmark of the batched graph beam search (one JSON line on rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3|c2|c1|c4|small]
    python bench.py --impl reference ...      # the reference's CPU best-first search, host cores

A step is one pass of the search over the workload's whole query batch.

Replicated workloads (c1, c2, c3, small): with N GPUs every rank holds the whole index and
searches a contiguous 1/N slice of the batch -- no collective on the data path, total work
fixed (strong scaling).  Sharded workload (c4): every rank holds one 12.5M-point shard with
its own graph, searches ALL queries, and the per-shard top-k are exchanged with one NCCL
all-gather and merged (weak scaling: the index grows with N).

value : queries/s with index and queries resident in HBM, device pointers in and out
        (coral_search_async), CUDA events on the launching stream, max over ranks.
e2e   : queries/s through coral_search with pinned HOST queries in and HOST ids out, the
        copies inside the timed region.
Inputs are seeded synthetic data of the named shapes (coral_b200/synth.py); the index
(vectors + adjacency) is far larger than L2, so no cache flush is needed between iterations.
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
    # n: base points (per shard when sharded), groups: mixture centres / clusters
    "c1": dict(n=1_000_000, dim=200, metric="l2", deg=32, groups=1000, q=10_000, k=10, Ls=[64, 128, 256, 512], train=100_000),
    "c2": dict(n=1_000_000, dim=512, metric="ip", deg=32, groups=410, q=10_000, k=10, Ls=[64, 128, 256], train=100_000),
    "c3": dict(n=10_000_000, dim=512, metric="ip", deg=64, groups=4096, q=100_000, k=10, Ls=[64, 128, 256], train=100_000),
    "c4": dict(n=12_500_000, dim=200, metric="l2", deg=32, groups=10_000, q=100_000, k=100, Ls=[128, 256], train=100_000,
               sharded=True),
    "small": dict(n=1_000_000, dim=512, metric="ip", deg=64, groups=410, q=8_192, k=10, Ls=[64], train=50_000),
    # small-batch latency on the c3 index: batches of 1, 8, 64, 512 queries, L=128
    "c5": dict(n=10_000_000, dim=512, metric="ip", deg=64, groups=4096, q=8_192, k=10, Ls=[128], train=100_000,
               latency=[1, 8, 64, 512]),
}
METRIC = "QPS @ recall@10>=0.95, 10Mx512 IP"
PEAK_FALLBACK_GBS = 6650.0
# DRAM bytes moved by one full-size launch, from the single-pass ncu capture recorded in
# profiles/ (workload, L) -> bytes; absent -> null in the JSON line.
MEASURED_TRAFFIC = {
    ("c3", 64): 3.916e11,      # dram__bytes_read 366.0 GB + dram__bytes_write 25.6 GB for 100k queries (locality-ordered)
    ("small", 64): 1.201e10,   # 10.64 GB + 1.37 GB for 8192 queries
}


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


def build_inputs(w, device, rank=0, seed=20260001):
    """Seeded synthetic vectors, queries, graph and entry points (of this rank's shard when sharded)."""
    import torch
    from coral_b200 import synth
    t0 = time.time()
    draw = seed + 1000 + rank if w.get("sharded") else None
    if w["metric"] == "ip":
        ds = synth.make_ip_cones(w["n"], w["train"], w["q"], dim=w["dim"], clusters=w["groups"], seed=seed,
                                 device=device, draw_seed=draw)
    else:
        ds = synth.make_l2_mixture(w["n"], w["train"], w["q"], dim=w["dim"], centers=w["groups"], seed=seed,
                                   device=device, draw_seed=draw)
    g = synth.build_graph(ds.base, ds.train, ds.metric, max_degree=w["deg"], k_b=100, cell_size=512)
    if device != "cpu":
        torch.cuda.synchronize()
    log(f"[bench] rank {rank}: inputs ready in {time.time() - t0:.1f}s")
    ds.train = None
    if device != "cpu":
        torch.cuda.empty_cache()      # the builder's workspace is not part of the benchmark's footprint
    return ds, g


def exact_topk(base, queries, k, metric):
    """Exact ids and distances (fp32) of the k closest base rows: ground truth."""
    import torch
    from coral_b200 import synth
    ids = synth.exact_knn(base, queries, k, metric)
    rows = base[ids.long()]                                         # [Q, k, dim]
    if metric == "ip":
        d = (rows * queries[:, None, :]).sum(2)
    else:
        d = (rows - queries[:, None, :]).pow(2).sum(2)
    return ids, d.to(torch.float32)


def run_reference(args, w, rank, world):
    """The reference's CPU best-first search (src/search_in_cpu.cpp) on the host cores."""
    if rank != 0:
        return
    import torch
    from oracle import oracle
    device = "cuda" if torch.cuda.is_available() else "cpu"   # inputs are synthesised wherever it is fastest
    ds, g = build_inputs(w, device)
    n_gt = min(2000, w["q"])
    gt, _ = exact_topk(ds.base, ds.test[:n_gt], w["k"], w["metric"])
    base, adj = ds.base.cpu().numpy(), g.adj.cpu().numpy()
    start, test = g.start_ids.cpu().numpy(), ds.test.cpu().numpy()
    gt = gt.cpu().numpy()
    L = args.L or w["Ls"][0]
    sample = min(args.cpu_queries, w["q"])
    threads = os.cpu_count() or 1
    times, rec, kind, used = [], None, "port", threads
    for it in range(args.warmup + args.steps):
        ids, _, hops, secs, kind, used = oracle.cpu_search(base, adj, start, test[:sample], L, w["k"], threads=threads)
        if it >= args.warmup:
            times.append(secs)
        m = min(sample, gt.shape[0])
        rec = oracle.recall(ids[:m], gt[:m], w["k"])
    secs = sum(times) / len(times)
    qps = sample / secs
    desc = (f"first {sample} of {w['q']} queries per step, L={L}, k={w['k']}, recall@{w['k']}={rec:.4f}"
            + (" on one shard" if w.get("sharded") else "") + "; "
            + ("reference NeighborPriorityQueue + AVX-512 DistanceL2 with the search_in_cpu loop restated"
               if kind == "reference" else "self-contained port of search_in_cpu"))
    out = {
        "impl": "reference", "metric": METRIC, "value": qps, "unit": "queries/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": secs * 1e3, "higher_is_better": True,
        "scaling": "weak" if w.get("sharded") else "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "n": w["n"], "dim": w["dim"], "metric": w["metric"], "max_degree": w["deg"],
                   "queries_per_step": sample, "k": w["k"], "L": L, "recall": rec},
        "cpu_baseline": {"value": qps, "unit": "queries/s", "cores": used, "kind": kind, "sample": desc},
        "e2e": {"value": qps, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(out), flush=True)


def run_latency(args, w, ix, ds, g, device, rank):
    """Small-batch latency: per batch size, p50/p99 over many batches, device-resident (CUDA events
    around coral_search_async) and end to end (coral_search, pinned host queries in, host ids out)."""
    import numpy as np
    import torch
    from coral_b200 import capi, synth
    L, k, dim = args.L or w["Ls"][0], w["k"], w["dim"]
    lib, handle = capi.load(), ix._h
    n_gt = 2000
    gt = synth.exact_knn(ds.base, ds.test[:n_gt], k, w["metric"])
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
    # The same batches with 10 % of the points deleted (tombstones only: the reference's deleted-bitset
    # overload hides them from the results, src/search_gpu.cu:716; its topology repair and the insert
    # path are not part of this build, so this is not the reference's "after delete + insert" state).
    rng = np.random.default_rng(77)
    dead = rng.random(w["n"]) < 0.10
    bits = np.packbits(dead, bitorder="little")
    bits = np.concatenate([bits, np.zeros((-len(bits)) % 4, np.uint8)]).view(np.uint32)
    gt_wide = synth.exact_knn(ds.base, ds.test[:n_gt], 4 * k, w["metric"]).cpu().numpy()
    gt_alive = np.stack([row[~dead[row]][:k] for row in gt_wide])
    ix.set_deleted(bits)
    ids_d, _, _, _ = ix.search(ds.test[:n_gt], L, k, dists=False)
    ids_d = ids_d.cpu().numpy() if hasattr(ids_d, "cpu") else np.asarray(ids_d)
    assert not dead[ids_d[ids_d >= 0]].any(), "a deleted id was returned"
    recall_deleted = float(np.mean([len(set(a) & set(b)) / k for a, b in zip(ids_d, gt_alive)]))
    table_deleted = measure()
    ix.set_deleted(None)
    if rank == 0:
        b1 = table[w["latency"][0]]
        out = {"metric": "p50 latency of one query batch, 10Mx512 IP, L=%d" % L, "value": b1["p50_us"], "unit": "us",
               "n_gpus": 1, "steps": b1["batches"], "warmup": args.warmup, "ms_per_step": b1["p50_us"] * 1e-3,
               "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
               "config": {"workload": args.workload, "n": w["n"], "dim": dim, "metric": w["metric"], "max_degree": w["deg"],
                          "k": k, "L": L, "recall": recall, "batch_sizes": w["latency"], "latency": table,
                          "latency_with_10pct_deleted": table_deleted, "recall_with_10pct_deleted": recall_deleted,
                          "l2_policy": "inputs larger than L2; every batch uses different queries"},
               "e2e": {"value": b1["e2e_p50_us"], "unit": "us", "h2d_bytes_per_step": dim * 4 * w["latency"][0],
                       "d2h_bytes_per_step": k * 4 * w["latency"][0] + 32},
               "gpu_launches": int(ix.launch_count - launches0)}
        print(json.dumps(out), flush=True)


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
    ap.add_argument("--cpu-queries", type=int, default=10000, help="query sample of the CPU baseline")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--option", action="append", default=[], help="kernel tuning knob name=value")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)

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
    from coral_b200 import capi, sharded

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the search path has no CPU fallback")
    torch.cuda.set_device(local)
    device = f"cuda:{local}"
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
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

    ds, g = build_inputs(w, device, rank)     # replicated: same seed on every rank; sharded: own shard
    Q, k, dim = w["q"], w["k"], w["dim"]
    if sharded_mode:
        lo, hi = 0, Q                          # every shard searches every query
        id_map = torch.from_numpy(sharded.interleaved_ids(w["n"], world, rank)).to(device)
    else:
        lo, hi = sharded.query_slice(Q, world, rank)
        id_map = None
    my_q = ds.test[lo:hi].contiguous()
    nq = hi - lo
    n_gt = min(2000, Q)

    ix = capi.Index(w["n"], dim, w["deg"], w["metric"], device=local)
    for kv in args.option:
        name, val = kv.split("=")
        ix.set_option(name, int(val))
    ix.attach_vectors(ds.base)
    ix.set_adjacency(g.adj)
    ix.set_start_ids(g.start_ids)
    ix.prepare(max(nq, n_gt), max(w["Ls"] + [args.L]), k)
    torch.cuda.synchronize()
    sh = sharded.ShardedIndex(ix, id_map) if sharded_mode else None

    if w.get("latency"):
        run_latency(args, w, ix, ds, g, device, rank)
        ix.close()
        return

    # ---- ground truth (exact, fp32) for the first n_gt queries; global across shards when sharded
    gt_ids, gt_d = exact_topk(ds.base, ds.test[:n_gt], k, w["metric"])
    if sharded_mode:
        ix.map_ids(gt_ids, id_map)
        torch.cuda.synchronize()
        a_ids, a_d = sharded.all_gather_results(gt_ids, gt_d)
        torch.cuda.synchronize()               # gathered on torch's streams, merged on the handle's
        gt_ids, _ = ix.merge_shards(a_ids, a_d)
        torch.cuda.synchronize()

    # ---- beam capacity: smallest configured L whose recall@k on the ground-truth sample reaches 0.95
    recalls, L = {}, args.L
    for cand in ([args.L] if args.L else w["Ls"]):
        if sharded_mode:
            ids, _ = sh.search(ds.test[:n_gt], cand, k)
        else:
            ids, _, _, _ = ix.search(ds.test[:n_gt], cand, k, dists=False)
        recalls[cand] = ix.count_hits(ids, gt_ids, k) / float(k * n_gt)
        L = cand
        if recalls[cand] >= 0.95:
            break
    log(f"[bench] rank {rank}: recall by L {recalls}, using L={L}")

    d_ids = torch.empty((nq, k), dtype=torch.int32, device=device)
    d_dists = torch.empty((nq, k), dtype=torch.float32, device=device) if sharded_mode else None
    d_stats = torch.empty((nq, capi.STATS_W), dtype=torch.int32, device=device)
    stream = torch.cuda.Stream(device=device)
    h_q = my_q.cpu().pin_memory()
    h_ids = torch.empty((nq, k), dtype=torch.int32).pin_memory()
    h_q_np, h_ids_np = h_q.numpy(), h_ids.numpy()
    lib, handle = capi.load(), ix._h
    merged = {}

    def exchange_and_merge():
        """Sharded tail of a step on `stream`: local->global ids, one all-gather, merge."""
        ix.map_ids(d_ids, id_map, stream.cuda_stream)
        with torch.cuda.stream(stream):        # buffers are allocated for, and used on, this stream
            a_ids, a_d = sharded.all_gather_results(d_ids, d_dists)
            merged["ids"], merged["dists"] = ix.merge_shards(a_ids, a_d, stream.cuda_stream)

    def device_step():
        ix.search_async(my_q, L, k, d_ids, d_dists, None, stream.cuda_stream)
        if sharded_mode:
            exchange_and_merge()

    # ---- algorithmic bytes of one step (deterministic for the query set): untimed pass with counters
    ix.search_async(my_q, L, k, d_ids, d_dists, d_stats, stream.cuda_stream)
    stream.synchronize()
    ix.check()
    st = d_stats.cpu().numpy().astype(np.int64)
    row_bytes, deg_pad = dim * 4, g.adj.shape[1]
    alg_bytes = float((st[:, 1] * row_bytes + st[:, 2] * deg_pad * 4 + row_bytes + k * 8).sum())

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
    dev_ms = reduce_ranks(ev0.elapsed_time(ev1), dist.ReduceOp.MAX) / args.steps
    ref_ids = (merged["ids"] if sharded_mode else d_ids).cpu().numpy()

    # ---- end to end: pinned host queries in, host ids out, through coral_search
    hops = C.c_int64(0)

    def e2e_step():
        out_ptr = C.c_void_p(d_ids.data_ptr()) if sharded_mode else C.c_void_p(h_ids_np.ctypes.data)
        rc = lib.coral_search(handle, C.c_void_p(h_q_np.ctypes.data), nq, L, k, out_ptr,
                              C.c_void_p(d_dists.data_ptr()) if sharded_mode else None, None, C.byref(hops))
        if rc != 0:
            raise RuntimeError(lib.coral_last_error(handle).decode())
        if sharded_mode:
            exchange_and_merge()
            with torch.cuda.stream(stream):
                h_ids.copy_(merged["ids"], non_blocking=True)
            stream.synchronize()

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
    achieved = reduce_ranks(alg_bytes / (dev_ms * 1e-3) / 1e9, dist.ReduceOp.MIN)   # per GPU, against one GPU's peak

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            from oracle import oracle
            base_h, adj_h = ds.base.cpu().numpy(), g.adj.cpu().numpy()
            sample = min(args.cpu_queries, Q)
            cids, _, chops, secs, kind, used = oracle.cpu_search(base_h, adj_h, g.start_ids.cpu().numpy(),
                                                                  ds.test[:sample].cpu().numpy(), L, k)
            m = min(sample, n_gt)
            crec = oracle.recall(cids[:m], gt_ids[:m].cpu().numpy(), k)
            cpu = {"value": sample / secs, "unit": "queries/s", "cores": used, "kind": kind,
                   "sample": f"first {sample} of {Q} queries, L={L}, k={k}, recall@{k}={crec:.4f}, one pass of "
                             f"{secs:.2f}s; search_in_cpu loop (always squared L2; best-first, so its recall on a "
                             f"graph routed for full expansion differs)"}
            del base_h, adj_h
        except Exception as e:  # the baseline is a report, never a reason to lose the measurement
            cpu = {"value": None, "unit": "queries/s", "cores": 0, "kind": "port", "sample": f"failed: {e}"}

    if rank == 0:
        index_gb = w["n"] * (row_bytes + deg_pad * 4) / 1e9
        out = {
            "metric": METRIC, "value": Q / (dev_ms * 1e-3), "unit": "queries/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dev_ms, "higher_is_better": True,
            "scaling": "weak" if sharded_mode else "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "n": w["n"] * (world if sharded_mode else 1), "dim": dim,
                       "metric": w["metric"], "max_degree": w["deg"], "queries_per_step": Q, "k": k, "L": L,
                       "recall": recalls[L], "recall_by_L": recalls, "entry_points": int(g.start_ids.numel()),
                       "parallelism": (f"{world} shards of {w['n']} points, all queries on every shard, one NCCL "
                                       f"all-gather + merge" if sharded_mode else
                                       f"replicated index, queries split x{world}"),
                       "l2_policy": "inputs larger than L2 (index %.1f GB per GPU)" % index_gb,
                       "plan": {n_: ix.get_option(n_) for n_ in ("plan_stages", "plan_chunk_bytes", "plan_smem_bytes",
                                                                  "plan_hash_bits", "plan_ctas_per_sm", "plan_warps")}},
            "e2e": {"value": Q / (e2e_ms * 1e-3), "unit": "queries/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": nq * dim * 4 * world, "d2h_bytes_per_step": (nq * k * 4 + 32) * world},
            "gpu_launches": int(launches * world),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": peak_kind, "traffic": (MEASURED_TRAFFIC.get((args.workload, L))
                                     if world == 1 and not args.queries and not args.n else None),
                         "algorithmic_bytes_per_step": total_alg, "kernel": "beam_search_kernel",
                         "note": "per GPU (slowest rank); algorithmic bytes = n_dist*dim*4 + n_exp*deg_pad*4 + dim*4 + k*8 per query"},
            "cpu_baseline": cpu,
            "clocks": clocks,
        }
        print(json.dumps(out), flush=True)
    ix.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

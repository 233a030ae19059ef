#!/usr/bin/env python
"""Benchmark of the batched graph beam search (one JSON line on rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3|c2|c1|small]
    python bench.py --impl reference ...      # the reference's CPU best-first search, host cores

A step is one pass of the search over the workload's whole query batch.  With N
GPUs the index is replicated and the batch is split into N contiguous slices
(no collective on the data path), so total work is fixed: strong scaling.

value : queries/s with index and queries resident in HBM, device pointers in and
        out (coral_search_async), CUDA events on the launching stream.
e2e   : queries/s through coral_search with pinned HOST queries in and HOST ids
        out, copies inside the timed region.
Inputs are seeded synthetic data of the named shapes (coral_b200/synth.py); the
index (vectors + adjacency) is far larger than L2, so no cache flush is needed
between iterations.
"""
from __future__ import annotations

import argparse
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
    # name: n, dim, metric, max_degree, clusters/centers, queries, k, L candidates, train queries
    "c1": dict(n=1_000_000, dim=200, metric="l2", deg=32, groups=1000, q=10_000, k=10, Ls=[64, 128, 256, 512], train=100_000),
    "c2": dict(n=1_000_000, dim=512, metric="ip", deg=32, groups=410, q=10_000, k=10, Ls=[64, 128, 256], train=100_000),
    "c3": dict(n=10_000_000, dim=512, metric="ip", deg=64, groups=4096, q=100_000, k=10, Ls=[64, 128, 256], train=100_000),
    "small": dict(n=1_000_000, dim=512, metric="ip", deg=64, groups=410, q=8_192, k=10, Ls=[64], train=50_000),
}
METRIC = "QPS @ recall@10>=0.95, 10Mx512 IP"
PEAK_FALLBACK_GBS = 6650.0


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


def build_inputs(w, device, seed=20260001):
    """Seeded synthetic vectors, queries, graph, entry points and ground truth."""
    import torch
    from coral_b200 import synth
    t0 = time.time()
    if w["metric"] == "ip":
        ds = synth.make_ip_cones(w["n"], w["train"], w["q"], dim=w["dim"], clusters=w["groups"], seed=seed, device=device)
    else:
        ds = synth.make_l2_mixture(w["n"], w["train"], w["q"], dim=w["dim"], centers=w["groups"], seed=seed, device=device)
    g = synth.build_graph(ds.base, ds.train, ds.metric, max_degree=w["deg"], k_b=100, cell_size=512)
    n_gt = min(2000, w["q"])
    gt = synth.exact_knn(ds.base, ds.test[:n_gt], w["k"], ds.metric)
    if device != "cpu":
        torch.cuda.synchronize()
    log(f"[bench] inputs ready in {time.time() - t0:.1f}s")
    ds.train = None
    if device != "cpu":
        torch.cuda.empty_cache()      # the builder's workspace is not part of the benchmark's footprint
    return ds, g, gt


def run_reference(args, w, rank, world):
    """The reference's CPU best-first search (src/search_in_cpu.cpp) on the host cores."""
    if rank != 0:
        return
    import torch
    from oracle import oracle
    device = "cuda" if torch.cuda.is_available() else "cpu"   # inputs are synthesised wherever it is fastest
    ds, g, gt = build_inputs(w, device)
    base, adj = ds.base.cpu().numpy(), g.adj.cpu().numpy()
    start, test = g.start_ids.cpu().numpy(), ds.test.cpu().numpy()
    gt = gt.cpu().numpy()
    L = args.L or w["Ls"][0]
    sample = min(args.cpu_queries, w["q"])
    threads = os.cpu_count() or 1
    times, rec = [], None
    for it in range(args.warmup + args.steps):
        ids, _, hops, secs, kind, used = oracle.cpu_search(base, adj, start, test[:sample], L, w["k"], threads=threads)
        if it >= args.warmup:
            times.append(secs)
        n_gt = min(sample, gt.shape[0])
        rec = oracle.recall(ids[:n_gt], gt[:n_gt], w["k"])
    secs = sum(times) / len(times)
    qps = sample / secs
    desc = (f"first {sample} of {w['q']} queries per step, L={L}, k={w['k']}, recall@{w['k']}={rec:.4f}; "
            + ("reference NeighborPriorityQueue + AVX-512 DistanceL2 with the search_in_cpu loop restated"
               if kind == "reference" else "self-contained port of search_in_cpu"))
    out = {
        "impl": "reference", "metric": METRIC, "value": qps, "unit": "queries/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": secs * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "n": w["n"], "dim": w["dim"], "metric": w["metric"], "max_degree": w["deg"],
                   "queries_per_step": sample, "k": w["k"], "L": L, "recall": rec},
        "cpu_baseline": {"value": qps, "unit": "queries/s", "cores": used, "kind": kind, "sample": desc},
        "e2e": {"value": qps, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
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

    if args.impl == "reference":
        run_reference(args, w, rank, world)
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    from coral_b200 import capi

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the search path has no CPU fallback")
    torch.cuda.set_device(local)
    device = f"cuda:{local}"
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(device))

    ds, g, gt = build_inputs(w, device)       # same seed on every rank: the index is replicated
    Q, k, dim = w["q"], w["k"], w["dim"]
    lo, hi = rank * Q // world, (rank + 1) * Q // world
    my_q = ds.test[lo:hi].contiguous()
    nq = hi - lo

    ix = capi.Index(w["n"], dim, w["deg"], w["metric"], device=local)
    for kv in args.option:
        name, val = kv.split("=")
        ix.set_option(name, int(val))
    ix.attach_vectors(ds.base)
    ix.set_adjacency(g.adj)
    ix.set_start_ids(g.start_ids)
    ix.prepare(max(nq, gt.shape[0]), max(w["Ls"] + [args.L]), k)
    torch.cuda.synchronize()

    # beam capacity: smallest configured L whose recall@k on the ground-truth sample reaches 0.95
    recalls = {}
    L = args.L
    for cand in ([args.L] if args.L else w["Ls"]):
        ids, _, _, _ = ix.search(ds.test[:gt.shape[0]], cand, k, dists=False)
        recalls[cand] = ix.count_hits(ids, gt, k) / float(k * gt.shape[0])
        L = cand
        if recalls[cand] >= 0.95:
            break
    log(f"[bench] rank {rank}: recall by L {recalls}, using L={L}")

    d_ids = torch.empty((nq, k), dtype=torch.int32, device=device)
    d_stats = torch.empty((nq, capi.STATS_W), dtype=torch.int32, device=device)
    stream = torch.cuda.Stream(device=device)
    h_q = my_q.cpu().pin_memory()
    h_ids = torch.empty((nq, k), dtype=torch.int32).pin_memory()
    h_q_np, h_ids_np = h_q.numpy(), h_ids.numpy()
    lib, handle = capi.load(), ix._h
    import ctypes as C

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    # ---- algorithmic bytes of one step (deterministic for the query set): untimed pass with counters
    ix.search_async(my_q, L, k, d_ids, None, d_stats, stream.cuda_stream)
    stream.synchronize()
    ix.check()
    st = d_stats.cpu().numpy().astype(np.int64)
    row_bytes, deg_pad = dim * 4, g.adj.shape[1]
    alg_bytes = float((st[:, 1] * row_bytes + st[:, 2] * deg_pad * 4 + row_bytes + k * 8).sum())

    # ---- device-resident timing
    for _ in range(args.warmup):
        ix.search_async(my_q, L, k, d_ids, None, None, stream.cuda_stream)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = ix.launch_count
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for _ in range(args.steps):
        ix.search_async(my_q, L, k, d_ids, None, None, stream.cuda_stream)
    ev1.record(stream)
    barrier()
    ix.check()
    launches = ix.launch_count - launches0
    clocks = sampler.stop() if rank == 0 else None
    dev_ms = max_over_ranks(ev0.elapsed_time(ev1)) / args.steps

    # ---- end to end: pinned host queries in, host ids out, through coral_search
    hops = C.c_int64(0)

    def e2e_step():
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
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3) / args.steps
    same = bool(np.array_equal(h_ids_np, d_ids.cpu().numpy()))
    if not same:
        raise SystemExit("host-pointer and device-pointer searches disagree")

    total_alg = sum_over_ranks(alg_bytes)
    peak, peak_kind = measured_peak()
    achieved = alg_bytes / (dev_ms * 1e-3) / 1e9          # this rank's kernel against this GPU's peak
    achieved = max_over_ranks(achieved) if world > 1 else achieved

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            from oracle import oracle
            base_h, adj_h = ds.base.cpu().numpy(), g.adj.cpu().numpy()
            sample = min(args.cpu_queries, Q)
            cids, _, chops, secs, kind, used = oracle.cpu_search(base_h, adj_h, g.start_ids.cpu().numpy(),
                                                                  ds.test[:sample].cpu().numpy(), L, k)
            n_gt = min(sample, gt.shape[0])
            crec = oracle.recall(cids[:n_gt], gt[:n_gt].cpu().numpy(), k)
            cpu = {"value": sample / secs, "unit": "queries/s", "cores": used, "kind": kind,
                   "sample": f"first {sample} of {Q} queries, L={L}, k={k}, recall@{k}={crec:.4f}, one pass of "
                             f"{secs:.2f}s; search_in_cpu loop (always squared L2 on unit vectors)"}
            del base_h, adj_h
        except Exception as e:  # the baseline is a report, never a reason to lose the measurement
            cpu = {"value": None, "unit": "queries/s", "cores": 0, "kind": "port", "sample": f"failed: {e}"}

    if rank == 0:
        out = {
            "metric": METRIC, "value": Q / (dev_ms * 1e-3), "unit": "queries/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dev_ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "n": w["n"], "dim": dim, "metric": w["metric"], "max_degree": w["deg"],
                       "queries_per_step": Q, "k": k, "L": L, "recall": recalls[L], "recall_by_L": recalls,
                       "entry_points": int(g.start_ids.numel()), "parallelism": f"replicated index, queries split x{world}",
                       "l2_policy": "inputs larger than L2 (index %.1f GB)" % ((w["n"] * (row_bytes + deg_pad * 4)) / 1e9),
                       "plan": {n_: ix.get_option(n_) for n_ in ("plan_stages", "plan_chunk_bytes", "plan_smem_bytes",
                                                                  "plan_hash_bits", "plan_ctas_per_sm", "warps")}},
            "e2e": {"value": Q / (e2e_ms * 1e-3), "unit": "queries/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": Q * dim * 4, "d2h_bytes_per_step": Q * k * 4 + 32 * world},
            "gpu_launches": int(launches * world),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": peak_kind, "traffic": None,
                         "algorithmic_bytes_per_step": total_alg, "kernel": "beam_search_kernel"},
            "cpu_baseline": cpu,
            "clocks": clocks,
        }
        print(json.dumps(out), flush=True)
    ix.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""Benchmark of the hot path: build seconds and search QPS at recall@10 >= 0.95.

    python bench.py --gpus N --steps K --warmup W [--config cfg1] [--impl reference]

A step is one pass of the search call (routing pre-pass + search kernel) over one batch of Q
queries (10,000 for cfg1) at the smallest beam (a fixed ladder, then bisection between its steps)
that reaches recall@10 >= 0.95 against exact kNN; the index is built once before the timed region
and its stage times are reported under "build". `value` is queries/s with queries resident in HBM
(sum over ranks / max time over ranks, CUDA events around the kernels); `e2e` is the same through
the host-buffer entry point with the H2D and D2H copies inside the timed region. Under torchrun
the index build is sharded over the ranks, every rank ends with the full index (a checksum of it is
compared across ranks and with rank 0's own single-GPU build) and searches its own query batch
(weak scaling of the timed step, no collective inside it).

`--impl reference`: the reference has no CPU implementation and its programs cannot be built
without RAFT/cuVS, so this arm times the CPU restatement of its search (the oracle: same
algorithm, same index, same beam, hence the same results and recall as the GPU arm) on all host
threads over a bounded sample of the query batch per step. With `--config cfg1c32`, a
configuration inside the reference's own size ladders, it times the reference's own search kernel
on the GPU instead (compiled from the reference tree into oracle/_ref when that tree was present at
build time), on an index built by this library.

Data are seeded synthetic stand-ins with the shapes and value ranges of the named config.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BEAM_LADDER = [10, 15, 20, 25, 30, 35, 40, 45, 50, 60, 70, 80, 100, 120, 150, 200, 256, 384, 512]
TARGET_RECALL = 0.95
TOP_K = 10
METRIC_NAME = "search QPS @ recall@10>=0.95"

# DRAM bytes of one search_kernel launch, measured with ncu (dram__bytes_read.sum +
# dram__bytes_write.sum, one pass, --clock-control none) on the workload named by the key
# (config, rows, queries, partitions, rounded beam, max_iterations); the summaries under
# profiles/ give the commands. A bench run on another workload reports traffic null.
NCU_TRAFFIC = {
    ("cfg1", 1000000, 10000, 1024, 32, 31): 1_944_421_148,   # profiles/search_kernel_cfg1_full_dram.md (mean of 9 launches)
    ("cfg1_n400000", 400000, 10000, 1024, 32, 15): 396_663_268,     # same file, the small case captured first
}
# issue-slot utilisation of the same kernel from the kept ncu capture (profiles/search_kernel_cfg1_400k.md)
NCU_ISSUE = {"issue_slots_busy_pct": 60.0, "top_stall": "long_scoreboard", "source": "profiles/search_kernel_cfg1_400k.md"}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="cfg1")
    ap.add_argument("--rows", type=int, default=0, help="use only the first ROWS base rows (debugging; marks the run reduced)")
    ap.add_argument("--queries", type=int, default=0)
    ap.add_argument("--partitions", type=int, default=0, help="override the partition count")
    ap.add_argument("--merged", action="store_true", help="large path, one GPU: also build and search the merged index")
    ap.add_argument("--loader-dir", default="/dev/shm", help="--config loader: where the synthetic matrix file is written")
    ap.add_argument("--rows-u8", action="store_true", help="large path: keep integer-valued rows as uint8 in host memory")
    ap.add_argument("--route-min", type=int, default=4, help="large path: partitions every query visits at least")
    ap.add_argument("--route-factor", type=float, default=1.2, help="large path: visit partitions within this factor of the nearest")
    ap.add_argument("--max-beam", type=int, default=256, help="large path: last beam of the ladder that is tried")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="target CPU time of the host baseline sample")
    ap.add_argument("--clock-seconds", type=float, default=1.5,
                    help="the timed step is repeated for this long after the timed region so that the clock sampler sees it")
    return ap.parse_args()


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 200 ms during the timed region."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.device_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            # nvidia-smi takes a moment to initialise and holds driver locks while it does: wait for its
            # first sample so that the start-up does not land inside the timed region
            deadline = time.time() + 5.0
            while not self.lines and time.time() < deadline and self.proc.poll() is None:
                time.sleep(0.02)
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def load_peaks() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def make_data(args):
    from glide_b200 import datasets
    spec = datasets.CONFIGS[args.config]
    reduced = False
    if args.rows and args.rows < spec.n:
        spec = datasets.scaled(spec, args.rows, args.queries or spec.n_queries)
        reduced = True
    elif args.queries:
        spec = datasets.scaled(spec, spec.n, args.queries)
    return spec, reduced


def partition_count(spec, override: int = 0) -> int:
    """One partition per mixture component: the synthetic sets are unions of well separated
    clusters, their kNN graphs have one connected component per cluster, and a beam search that
    enters at a partition's start point only reaches that component. (The reference's default of
    10 partitions suits data whose kNN graph is connected.)"""
    if override:
        return override
    return 1 if spec.n <= 20000 else max(1, min(spec.centres, spec.n // 64))


def workload_string(spec, Q, partitions) -> str:
    return (f"{spec.name}: {spec.n}x{spec.dim} fp32 {spec.metric}, {Q} queries per rank, k={TOP_K}, "
            f"graph degree {spec.graph_degree}, {partitions} partitions")


def build_config(spec, centroid_num):
    from glide_b200 import pipeline
    from glide_b200.params import Metric
    return pipeline.BuildConfig(metric=Metric.parse(spec.metric), graph_degree=spec.graph_degree,
                                knn_degree=max(32, spec.graph_degree), centroid_num=centroid_num,
                                sample_factor=0.1 if centroid_num > 32 else 0.01, seed=spec.seed)


def choose_beam(search, gt, degree, Q):
    """Smallest beam reaching the target recall: a fixed ladder, then bisection between its steps
    (recall grows with the beam). search(sp) -> (ids, seconds)."""
    from glide_b200 import api, pipeline
    chosen, curve = None, []
    for beam in BEAM_LADDER:
        sp = pipeline.derive_search_params(beam, degree, TOP_K)
        ids, sec = search(sp)
        rec = api.calculate_recall(ids, gt, TOP_K)
        curve.append({"beam": beam, "recall": round(rec, 4), "qps": round(Q / sec, 1)})
        if rec >= TARGET_RECALL:
            chosen = (beam, sp, rec)
            break
    if chosen is not None and len(curve) >= 2:
        lo, hi = curve[-2]["beam"], chosen[0]
        while hi - lo > 1:
            mid = (lo + hi) // 2
            sp_mid = pipeline.derive_search_params(mid, degree, TOP_K)
            ids, sec = search(sp_mid)
            rec = api.calculate_recall(ids, gt, TOP_K)
            curve.append({"beam": mid, "recall": round(rec, 4), "qps": round(Q / sec, 1)})
            if rec >= TARGET_RECALL:
                hi, chosen = mid, (mid, sp_mid, rec)
            else:
                lo = mid
        curve.sort(key=lambda c: c["beam"])
    if chosen is None:
        beam = BEAM_LADDER[-1]
        chosen = (beam, pipeline.derive_search_params(beam, degree, TOP_K), curve[-1]["recall"])
    return chosen, curve


def cpu_bruteforce_qps(base, queries, seconds_target, metric):
    """Exact kNN on all host cores over a bounded sample of the queries."""
    import oracle
    # all host threads this process may run on (torchrun sets OMP_NUM_THREADS=1, which would leave one)
    cores = max(oracle.max_threads(), len(os.sched_getaffinity(0)))
    probe = min(len(queries), max(4 * cores, 32))
    oracle.bruteforce_knn(base, queries[:probe], TOP_K, metric, threads=cores, want_dists=False)  # warm (page faults)
    t0 = time.perf_counter()
    oracle.bruteforce_knn(base, queries[:probe], TOP_K, metric, threads=cores, want_dists=False)
    per_query = (time.perf_counter() - t0) / probe
    sample = int(min(len(queries), max(probe, seconds_target / max(per_query, 1e-9))))
    t0 = time.perf_counter()
    oracle.bruteforce_knn(base, queries[:sample], TOP_K, metric, threads=cores, want_dists=False)
    dt = time.perf_counter() - t0
    if dt < 0.66 * seconds_target and sample < len(queries):
        # the small probe underestimates a large batch's throughput: size the sample once more from this run
        sample = int(min(len(queries), sample * seconds_target / dt))
        t0 = time.perf_counter()
        oracle.bruteforce_knn(base, queries[:sample], TOP_K, metric, threads=cores, want_dists=False)
        dt = time.perf_counter() - t0
    return sample / dt, cores, sample, dt


# --------------------------------------------------------------------------------------------
# reference arm
# --------------------------------------------------------------------------------------------
def reference_line(args, spec, reduced, partitions, qps, ms_per_step, cpu_baseline, extra_config, extra):
    line = {
        "impl": "reference", "metric": METRIC_NAME, "value": qps, "unit": "queries/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": dict({"workload": workload_string(spec, spec.n_queries, partitions), "reduced": reduced}, **extra_config),
        "cpu_baseline": cpu_baseline,
        "e2e": {"value": qps, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    line.update(extra)
    return line


def run_reference_bruteforce(args, spec, reduced, base, queries, ometric):
    """No GPU to build an index on: exact brute-force kNN on the host cores."""
    import oracle
    cores = max(oracle.max_threads(), len(os.sched_getaffinity(0)))
    probe = min(len(queries), max(4 * cores, 32))
    oracle.bruteforce_knn(base, queries[:probe], TOP_K, ometric, threads=cores, want_dists=False)
    t0 = time.perf_counter()
    oracle.bruteforce_knn(base, queries[:probe], TOP_K, ometric, threads=cores, want_dists=False)
    per_query = (time.perf_counter() - t0) / probe
    budget = max(args.cpu_seconds * 4, 20.0) / max(args.steps + args.warmup, 1)
    sample = int(min(len(queries), max(probe, budget / max(per_query, 1e-9))))
    for _ in range(args.warmup):
        oracle.bruteforce_knn(base, queries[:sample], TOP_K, ometric, threads=cores, want_dists=False)
    t0 = time.perf_counter()
    for s in range(args.steps):
        lo = (s * sample) % max(len(queries) - sample + 1, 1)
        oracle.bruteforce_knn(base, queries[lo:lo + sample], TOP_K, ometric, threads=cores, want_dists=False)
    dt = time.perf_counter() - t0
    qps = args.steps * sample / dt
    cpu = {"value": qps, "unit": "queries/s", "cores": cores, "kind": "port",
           "sample": f"exact brute-force kNN (recall 1.0), {sample} queries per step on {cores} host threads"}
    return reference_line(args, spec, reduced, partition_count(spec, args.partitions), qps, dt / args.steps * 1e3, cpu,
                          {"note": "no CUDA device to build an index on: exact brute-force kNN instead of the graph search"},
                          {"recall_at_10": 1.0})


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    from oracle import ref
    from glide_b200 import datasets
    oracle.build()
    spec, reduced = make_data(args)
    cent = datasets.centres(spec)
    base = datasets.base_rows(spec, cent=cent)
    queries = datasets.queries(spec, cent=cent)
    ometric = oracle.EUCLIDEAN if spec.metric == "Euclidean" else oracle.COSINE
    import torch
    if not torch.cuda.is_available():
        print(json.dumps(run_reference_bruteforce(args, spec, reduced, base, queries, ometric)), flush=True)
        return
    from glide_b200 import api, pipeline
    ctx = api.Context(int(os.environ.get("LOCAL_RANK", "0")))
    dev = ctx.torch_device
    d_base, d_queries = torch.from_numpy(base).to(dev), torch.from_numpy(queries).to(dev)
    Q = queries.shape[0]
    partitions = partition_count(spec, args.partitions)
    cfg = build_config(spec, partitions)
    # the index both arms search: built by this library outside the timed region (the reference's own
    # kNN and k-means stages are cuVS calls that are not in its tree)
    res = pipeline.build_small(ctx, d_base, cfg)
    index = res.index
    gt = api.to_u32(api.bruteforce_knn(ctx, d_base, d_queries, TOP_K, cfg.metric)[0])
    C = index.centroid_num()
    graph = api.to_u32(index.graph_view())
    centroids = index.centroid_view().cpu().numpy()
    start_points = api.to_u32(index.start_point_view())
    cores = max(oracle.max_threads(), len(os.sched_getaffinity(0)))

    use_kernels = ref.available() and C <= 32 and spec.graph_degree <= 64
    if use_kernels:
        # ---- the reference's own search kernel on the GPU (inside its size ladders) ----
        d_ids = api._u32_tensor(ctx, (Q, TOP_K))
        d_d = ctx.empty((Q, TOP_K), torch.float32)

        def ref_search(sp, d_q=d_queries):
            torch.cuda.synchronize(dev)
            rc = ref.search(d_base.data_ptr(), spec.dim, index.d_graph.data_ptr(), spec.graph_degree,
                            index.d_centroids.data_ptr(), C, index.d_start_points.data_ptr(), d_q.data_ptr(), Q, sp,
                            int(cfg.metric), d_ids.data_ptr(), d_d.data_ptr())
            if rc != 0:
                raise RuntimeError(f"reference search kernel refused the shape (rc {rc})")
            return api.to_u32(d_ids), ref.last_seconds()

        (beam, sp, recall), curve = choose_beam(ref_search, gt, spec.graph_degree, Q)
        flush = torch.empty(512 * 1024 * 1024 // 4, dtype=torch.float32, device=dev)
        h_q = torch.from_numpy(queries).pin_memory()
        h_ids = torch.empty((Q, TOP_K), dtype=torch.int32).pin_memory()
        h_d = torch.empty((Q, TOP_K), dtype=torch.float32).pin_memory()
        d_q2 = torch.empty_like(d_queries)
        for _ in range(args.warmup):
            flush.add_(1.0)
            ref_search(sp)
        kernel_s = e2e_s = 0.0
        for _ in range(args.steps):
            flush.add_(1.0)
            kernel_s += ref_search(sp)[1]       # CUDA events around the reference's kernel
        for _ in range(args.steps):
            flush.add_(1.0)
            torch.cuda.synchronize(dev)
            t0 = time.perf_counter()
            d_q2.copy_(h_q, non_blocking=True)
            ref_search(sp, d_q2)
            h_ids.copy_(d_ids, non_blocking=True)
            h_d.copy_(d_d, non_blocking=True)
            torch.cuda.synchronize(dev)
            e2e_s += time.perf_counter() - t0
        qps = args.steps * Q / kernel_s
        line = reference_line(args, spec, reduced, partitions, qps, kernel_s / args.steps * 1e3, None,
                              {"beam": beam, "beam_rounded": sp.beam, "max_iterations": sp.max_iterations,
                               "l2": "512 MB buffer rewritten between timed iterations",
                               "note": "the reference's search_kernel (one 64-thread CTA per query) on the GPU, on an index "
                                       "built by this library"},
                              {"recall_at_10": round(recall, 4), "recall_curve": curve})
        line["e2e"] = {"value": args.steps * Q / e2e_s, "unit": "queries/s", "h2d_bytes_per_step": Q * spec.dim * 4,
                       "d2h_bytes_per_step": Q * TOP_K * 8}
        if not args.no_cpu_baseline:
            cqps, ccores, sample, dt = cpu_bruteforce_qps(base, queries, args.cpu_seconds, ometric)
            line["cpu_baseline"] = {"value": cqps, "unit": "queries/s", "cores": ccores, "kind": "port",
                                    "sample": f"exact brute-force kNN (recall 1.0) of {sample} queries in {dt:.1f} s"}
        print(json.dumps(line), flush=True)
        ctx.close()
        return

    # ---- the CPU restatement of the reference's search on the same index, all host threads ----
    def gpu_search(sp):
        ids, _, sec = index.search(sp, d_queries)
        return ids, sec
    # the beam is found with the GPU arm's kernels (their results equal the oracle's bit for bit, which
    # the timed sample below re-checks); only the oracle runs inside the timed region
    (beam, sp, recall), curve = choose_beam(gpu_search, gt, spec.graph_degree, Q)
    o = oracle.SearchParams(sp.beam, sp.max_iterations, sp.min_iterations, sp.hash_bit, sp.hash_reset_interval, TOP_K)

    def cpu_search(q):
        return oracle.search(base, graph, centroids, start_points, q, o, ometric, threads=cores)

    probe = min(Q, max(8 * cores, 64))
    cpu_search(queries[:probe])
    t0 = time.perf_counter()
    cpu_search(queries[:probe])
    per_query = (time.perf_counter() - t0) / probe
    budget = max(args.cpu_seconds * 4, 20.0) / max(args.steps + args.warmup, 1)
    sample = int(min(Q, max(probe, budget / max(per_query, 1e-9))))
    for _ in range(args.warmup):
        cpu_search(queries[:sample])
    got = []
    t0 = time.perf_counter()
    for s in range(args.steps):
        lo = (s * sample) % max(Q - sample + 1, 1)
        ids, _ = cpu_search(queries[lo:lo + sample])
        got.append((lo, ids))
    dt = time.perf_counter() - t0
    qps = args.steps * sample / dt
    hits = sum(float(api.calculate_recall(ids, gt[lo:lo + sample], TOP_K)) * len(ids) for lo, ids in got)
    cpu_recall = hits / (args.steps * sample)
    gpu_ids, _ = gpu_search(sp)
    same = float(np.mean([(ids == gpu_ids[lo:lo + sample]).all(axis=1).mean() for lo, ids in got]))
    cpu = {"value": qps, "unit": "queries/s", "cores": cores, "kind": "port",
           "sample": f"graph search (the oracle's restatement of the reference's search_kernel) of {sample} queries per step "
                     f"on {cores} host threads, beam {beam}"}
    line = reference_line(args, spec, reduced, partitions, qps, dt / args.steps * 1e3, cpu,
                          {"beam": beam, "beam_rounded": sp.beam, "max_iterations": sp.max_iterations,
                           "l2": "index and base set (larger than L2 and than the host caches) walked at random",
                           "note": "host cores: the CPU restatement of the reference's search on the index the GPU arm "
                                   "searches (the reference itself has no CPU path and cannot run 1,024 partitions)"},
                          {"recall_at_10": round(cpu_recall, 4), "queries_equal_to_gpu_arm": same})
    print(json.dumps(line), flush=True)
    ctx.close()


# --------------------------------------------------------------------------------------------
# this repository's arm
# --------------------------------------------------------------------------------------------
def graph_checksum(torch, graph_i32):
    """Position-dependent checksum of the graph: sum over slots of ((id + 1) * weight(slot)) mod 2^31-1."""
    g = graph_i32.to(torch.int64).reshape(-1) + 1
    w = (torch.arange(g.numel(), device=g.device, dtype=torch.int64) % 1000003) + 1
    return int(((g * w) % 2147483647).sum().item())


def run_ours(args):
    import torch
    import torch.distributed as dist

    from glide_b200 import api, datasets, pipeline

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = api.Context(local_rank)
    dev = ctx.torch_device

    spec, reduced = make_data(args)
    cent = datasets.centres(spec)
    base = datasets.base_rows(spec, cent=cent)
    # every rank searches its own batch from the same distribution (weak scaling)
    qspec = datasets.DatasetSpec(spec.name, spec.n, spec.dim, spec.n_queries, spec.kind, spec.centres, spec.metric,
                                 spec.graph_degree, spec.seed + 1000 * rank)
    queries = datasets.queries(spec, cent=cent) if rank == 0 else datasets._rows(qspec, cent, 2 + rank, 0, spec.n_queries)
    d_base = torch.from_numpy(base).to(dev)
    d_queries = torch.from_numpy(queries).to(dev)
    Q = queries.shape[0]

    # ---- build (untimed region of the step loop, reported on its own) ----
    centroid_num = partition_count(spec, args.partitions)
    cfg = build_config(spec, centroid_num)
    metric = cfg.metric
    if world > 1:
        # communicator set-up is not part of the build: the library's own NCCL communicator is created
        # (and one small collective run on it) before the clock starts
        from glide_b200 import sharded
        ctx.init_comm(dist, world, rank)
        coll = sharded.GlideCollectives(ctx)
        dist.barrier()
    t0 = time.perf_counter()
    if world > 1:   # kNN by partition owner, build and refine rows split evenly, rows exchanged with all-gathers
        res = pipeline.build_small_sharded(ctx, d_base, cfg, coll)
    else:
        res = pipeline.build_small(ctx, d_base, cfg)
    torch.cuda.synchronize(dev)
    build_wall = time.perf_counter() - t0
    index = res.index
    sharded_check = None
    if world > 1:
        mine = graph_checksum(torch, index.graph_view())
        hi = ctx.all_reduce_u64(torch.tensor([mine], dtype=torch.int64, device=dev), "max")
        lo = ctx.all_reduce_u64(torch.tensor([mine], dtype=torch.int64, device=dev), "min")
        same_on_all = int(hi[0]) == mine and int(lo[0]) == mine
        single = None
        if rank == 0:   # rank 0's own single-GPU build of the same seed
            plain = pipeline.build_small(ctx, d_base, cfg)
            single = graph_checksum(torch, plain.index.graph_view())
            del plain
        sharded_check = {"checksum": mine, "equal_on_all_ranks": bool(same_on_all),
                         "equal_to_single_gpu_build": (single == mine) if single is not None else None}

    # ---- ground truth: exact kNN on the GPU, checked against the host on a few queries ----
    gt_ids, _ = api.bruteforce_knn(ctx, d_base, d_queries, TOP_K, metric)
    gt = api.to_u32(gt_ids)
    gt_seconds = ctx.last_kernel_seconds

    def gpu_search(sp):
        ids, _, sec = index.search(sp, d_queries)
        return ids, sec
    (beam, sp, recall), curve = choose_beam(gpu_search, gt, spec.graph_degree, Q)

    # ---- traffic counters of one search pass (untimed) ----
    ctx.enable_counters(True)
    index.search(sp, d_queries)
    rows_read, expansions, _, _ = ctx.read_counters()
    ctx.enable_counters(False)
    C = index.centroid_num()
    # algorithmic bytes of the search kernel: every data row it scores, one adjacency row per
    # expansion (+ the seed row), the query vector and the results
    algo_bytes = (rows_read * spec.dim * 4 + expansions * spec.graph_degree * 4 +
                  Q * (spec.dim * 4 + spec.graph_degree * 4 + TOP_K * 8))

    flush = torch.empty(512 * 1024 * 1024 // 4, dtype=torch.float32, device=dev)  # 512 MB > 126 MB L2

    def flush_l2():
        flush.add_(1.0)
        torch.cuda.synchronize(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    d_ids = api._u32_tensor(ctx, (Q, TOP_K))
    d_dists = ctx.empty((Q, TOP_K), torch.float32)
    pc = api._params_c(sp)
    import ctypes as C_

    def search_once():
        ctx.check(ctx.lib.glide_search(ctx.handle, d_base.data_ptr(), index.num(), index.dim(), index.d_graph.data_ptr(),
                                       index.graph_degree(), index.d_centroids.data_ptr(), C,
                                       index.d_start_points.data_ptr(), d_queries.data_ptr(), Q, C_.byref(pc),
                                       int(metric), d_ids.data_ptr(), d_dists.data_ptr()))
        ctx.lib.glide_last_search_split_ms(ctx.handle, split)
        return ctx.lib.glide_last_kernel_ms(ctx.handle), split[0], split[1]

    split = (C_.c_float * 2)()
    for _ in range(args.warmup):
        flush_l2()
        search_once()
    sampler = ClockSampler(local_rank)
    barrier()
    if rank == 0:
        sampler.start()
    barrier()
    kernel_ms = route_ms = search_ms = 0.0
    for _ in range(args.steps):
        flush_l2()
        total, r_ms, s_ms = search_once()   # CUDA events on the launching stream, around the kernels
        kernel_ms += total
        route_ms += r_ms
        search_ms += s_ms
    barrier()
    # ---- end to end through the host-buffer entry point (pinned host memory) ----
    h_q = torch.from_numpy(queries).pin_memory()
    h_ids = torch.empty((Q, TOP_K), dtype=torch.int32).pin_memory()
    h_d = torch.empty((Q, TOP_K), dtype=torch.float32).pin_memory()

    def search_host_once():
        ctx.check(ctx.lib.glide_search_host(ctx.handle, d_base.data_ptr(), index.num(), index.dim(),
                                            index.d_graph.data_ptr(), index.graph_degree(),
                                            index.d_centroids.data_ptr(), C, index.d_start_points.data_ptr(),
                                            h_q.data_ptr(), Q, C_.byref(pc), int(metric), h_ids.data_ptr(),
                                            h_d.data_ptr()))

    for _ in range(args.warmup):
        flush_l2()
        search_host_once()
    e2e_s = 0.0
    barrier()
    for _ in range(args.steps):
        flush_l2()
        t0 = time.perf_counter()
        search_host_once()   # returns after the results are in host memory
        e2e_s += time.perf_counter() - t0
    barrier()
    # ---- the same with three batches in flight (glide_search_pipe_*): every step still uploads its own
    # queries from pinned host memory and downloads its own results; uploads, kernels and downloads of
    # consecutive steps overlap. No flush between the steps here (it would drain the pipe): one step reads
    # ~0.6 GB of distinct rows and adjacency lists, five times the L2.
    depth = 3
    pipe = index.search_pipe(Q, TOP_K, depth)
    sets = [(torch.from_numpy(queries).pin_memory(), torch.empty((Q, TOP_K), dtype=torch.int32).pin_memory(),
             torch.empty((Q, TOP_K), dtype=torch.float32).pin_memory()) for _ in range(depth)]

    def pipe_steps(n):
        slot = C_.c_uint32()
        for i in range(n):
            hq, hi, hd = sets[i % depth]
            ctx.check(ctx.lib.glide_search_pipe_submit(pipe._h, d_base.data_ptr(), index.num(), index.dim(),
                                                       index.d_graph.data_ptr(), index.graph_degree(),
                                                       index.d_centroids.data_ptr(), C, index.d_start_points.data_ptr(),
                                                       hq.data_ptr(), Q, C_.byref(pc), int(metric), hi.data_ptr(),
                                                       hd.data_ptr(), C_.byref(slot)))
        pipe.drain()

    pipe_steps(max(args.warmup, depth))
    flush_l2()
    barrier()
    t0 = time.perf_counter()
    pipe_steps(args.steps)
    pipe_s = time.perf_counter() - t0
    barrier()
    pipe_ok = all(np.array_equal(s_[1].numpy(), h_ids.numpy()) for s_ in sets[:min(depth, args.steps)])
    pipe.close()
    # the timed regions last a few tens of milliseconds, less than the sampler's period: repeat the
    # same step (untimed) under the sampler so that the clock record shows the kernel under load
    extra_steps = 0
    t_end = time.perf_counter() + max(args.clock_seconds, 0.0)
    while time.perf_counter() < t_end:
        flush_l2()
        search_once()
        extra_steps += 1
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks["sampled_over"] = (f"the timed regions ({args.steps} + {args.steps} steps) and {extra_steps} further untimed "
                                  f"repeats of the same step ({args.clock_seconds} s)")
    e2e_recall = api.calculate_recall(h_ids.numpy().view(np.uint32), gt, TOP_K)

    t = torch.tensor([kernel_ms, e2e_s * 1e3, pipe_s * 1e3], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    max_kernel_ms, max_e2e_ms, max_pipe_ms = float(t[0]), float(t[1]), float(t[2])
    qps = world * Q * args.steps / (max_kernel_ms / 1e3)
    e2e_qps = world * Q * args.steps / (max_e2e_ms / 1e3)
    pipe_qps = world * Q * args.steps / (max_pipe_ms / 1e3)

    if rank == 0:
        peak, peak_kind = load_peaks()
        search_s = search_ms / args.steps / 1e3
        algo_gbs = algo_bytes / search_s / 1e9
        key = (spec.name, spec.n, Q, cfg.centroid_num, sp.beam, sp.max_iterations)
        traffic = NCU_TRAFFIC.get(key)
        roofline = {"bound": "hbm", "peak": peak, "unit": "GB/s", "peak_kind": peak_kind, "kernel": "search_kernel",
                    "kernel_ms": round(search_s * 1e3, 4), "traffic": traffic,
                    "algorithmic": {"bytes_per_launch": int(algo_bytes), "gbs": round(algo_gbs, 1),
                                    "of_peak": round(algo_gbs / peak, 4), "rows_read_per_launch": int(rows_read),
                                    "expansions_per_launch": int(expansions),
                                    "note": "every scored row counted once per scoring; queries of one partition run "
                                            "together, so most of these bytes are served by L2, not by DRAM"},
                    "issue": NCU_ISSUE}
        if traffic is not None:
            dram_gbs = traffic / search_s / 1e9
            roofline.update({"achieved": round(dram_gbs, 1), "frac": round(dram_gbs / peak, 4),
                             "note": "achieved = DRAM bytes of one launch (ncu, see NCU_TRAFFIC) / the kernel's CUDA-event "
                                     "time in this run. The data set is read about three times per launch (the partitions "
                                     "in flight exceed L2); the rest of the time is the dependent chain of a query"})
        else:
            roofline.update({"achieved": round(algo_gbs, 1), "frac": round(algo_gbs / peak, 4),
                             "note": "no ncu DRAM figure for this workload: achieved is the algorithmic figure, which "
                                     "counts bytes served by L2 and can exceed the DRAM peak"})
        line = {
            "metric": METRIC_NAME, "value": qps, "unit": "queries/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": max_kernel_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_string(spec, Q, cfg.centroid_num),
                       "beam": beam, "beam_rounded": sp.beam, "max_iterations": sp.max_iterations, "reduced": reduced,
                       "l2": "512 MB buffer rewritten between timed iterations",
                       "multi_gpu": ("build sharded: kNN graph by partition owner, subgraph build and refine rows split evenly, "
                                     "rows exchanged with NCCL all-gathers; then one full index and one query batch per "
                                     "rank") if world > 1 else "single GPU"},
            "recall_at_10": round(recall, 4),
            "build": {"seconds": round(res.total_seconds, 4), "wall_seconds": round(build_wall, 3),
                      "stages": {k: round(v, 4) for k, v in res.seconds.items()}, "nnd_rounds": res.nnd_rounds,
                      "tc_knn_fallbacks": ctx.tc_knn_fallbacks,
                      "ground_truth_seconds": round(gt_seconds, 4), "sharded_graph": sharded_check},
            "recall_curve": curve,
            "e2e": {"value": pipe_qps, "unit": "queries/s", "h2d_bytes_per_step": Q * spec.dim * 4,
                    "d2h_bytes_per_step": Q * TOP_K * 8, "recall_at_10": round(e2e_recall, 4),
                    "mode": f"glide_search_pipe_submit/wait, {depth} batches in flight, pinned host buffers, wall clock "
                            f"over the {args.steps} steps; results equal the blocking call's: {bool(pipe_ok)}",
                    "blocking_value": e2e_qps,
                    "blocking_mode": "glide_search_host, one batch at a time, wall clock around each call"},
            "gpu_launches": int(ctx.lib.glide_last_search_launches(ctx.handle)) * args.steps,
            "kernels_ms_per_step": {"route(assign_kernel)": round(route_ms / args.steps, 4),
                                    "search_kernel": round(search_ms / args.steps, 4)},
            "roofline": roofline,
            "clocks": clocks,
        }
        if not args.no_cpu_baseline:
            import oracle
            ometric = oracle.EUCLIDEAN if spec.metric == "Euclidean" else oracle.COSINE
            cqps, cores, sample, dt = cpu_bruteforce_qps(base, queries, args.cpu_seconds, ometric)
            # the same sample validates the GPU ground truth
            ref_gt = oracle.bruteforce_knn(base, queries[:min(sample, 64)], TOP_K, ometric, want_dists=False)
            line["cpu_baseline"] = {"value": cqps, "unit": "queries/s", "cores": cores, "kind": "port",
                                    "sample": f"exact brute-force kNN (recall 1.0) of {sample} queries in {dt:.1f} s",
                                    "gt_agreement": float((ref_gt == gt[:ref_gt.shape[0]]).mean())}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    ctx.close()


# --------------------------------------------------------------------------------------------
# large path (cfg3: 10M x 96 cosine in 64 partitions; cfg4: 100M x 128 in 512 partitions)
# --------------------------------------------------------------------------------------------
LARGE = {"cfg3": dict(partitions=64, sample_rows=1 << 18), "cfg4": dict(partitions=512, sample_rows=1 << 19),
         "cfg3c64": dict(partitions=64, sample_rows=1 << 18), "cfg4c512": dict(partitions=512, sample_rows=1 << 19)}
LARGE_BLOCK = 1 << 22   # rows generated and assigned at a time


def run_large(args):
    """Partitions owned by ranks (consecutive partitions to consecutive ranks, balanced by kNN cost); a
    rank keeps the rows of its own partitions in pinned host memory and streams them through its GPU
    (kNN graph, subgraph build, reverse edges, refine per partition). Search: every rank searches its
    own partitions (kept in HBM) for the whole query batch, the per-rank top-k lists are gathered with
    one NCCL all-gather and folded with the reference's merge network."""
    import torch
    import torch.distributed as dist
    from glide_b200 import api, datasets, large, pipeline, sharded
    from glide_b200.params import IndexParameter, Metric, NNDescentParameter

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = api.Context(local_rank)
    dev = ctx.torch_device
    if world > 1:
        ctx.init_comm(dist, world, rank)
    spec, reduced = make_data(args)
    metric = Metric.parse(spec.metric)
    n, dim, S = spec.n, spec.dim, args.partitions or LARGE[args.config]["partitions"]
    cent = torch.from_numpy(datasets.centres(spec)).to(dev)
    d_queries = datasets.device_queries(spec, dev, cent)
    Q = d_queries.shape[0]

    # ---- untimed: centroids, assignment of every row, exact ground truth, this rank's rows to host ----
    d_sample = datasets.device_rows(spec, 0, min(n, LARGE[args.config]["sample_rows"]), dev, cent)
    d_centroids, _, _ = api.kmeans_fit(ctx, d_sample, S, 0, metric, 1)
    del d_sample
    labels = torch.empty(n, dtype=torch.int32, device=dev)
    gt_d = torch.full((Q, TOP_K), float("inf"), device=dev)
    gt_i = torch.full((Q, TOP_K), -1, dtype=torch.int64, device=dev)
    assign_s = gt_s = 0.0
    for lo in range(0, n, LARGE_BLOCK):
        rows = datasets.device_rows(spec, lo, min(LARGE_BLOCK, n - lo), dev, cent)
        d_seg, _, _ = api.define_partition(ctx, rows, d_centroids, -1.0, metric)
        assign_s += ctx.last_kernel_seconds
        labels[lo:lo + rows.shape[0]] = d_seg[:, 0]
        if rank == 0 or world == 1:
            ids, dd = api.bruteforce_knn(ctx, rows, d_queries, TOP_K, metric)
            gt_s += ctx.last_kernel_seconds
            cat_d = torch.cat([gt_d, dd], dim=1)
            cat_i = torch.cat([gt_i, ids.to(torch.int64) + lo], dim=1)
            gt_d, pick = torch.topk(cat_d, TOP_K, dim=1, largest=False)
            gt_i = torch.gather(cat_i, 1, pick)
        del rows, d_seg
    order = torch.sort(labels.to(torch.int64), stable=True)[1]          # reorder id -> original id
    seg_len = torch.bincount(labels.to(torch.int64), minlength=S).cpu().numpy().astype(np.uint32)
    seg_start = np.concatenate([[0], np.cumsum(seg_len.astype(np.int64))[:-1]]).astype(np.uint32)
    owners = sharded.owner_ranges(seg_len, world, 1 << 20)
    p_lo, p_hi = owners[rank]
    r_lo = int(seg_start[p_lo]) if p_hi > p_lo else 0
    r_hi = int(seg_start[p_hi - 1]) + int(seg_len[p_hi - 1]) if p_hi > p_lo else 0
    mine = r_hi - r_lo
    pos = torch.empty(n, dtype=torch.int64, device=dev)
    pos[order] = torch.arange(n, device=dev)
    h_map = order[r_lo:r_hi].to(torch.int32).cpu().numpy().view(np.uint32)
    del order, labels
    d_mine = torch.empty((mine, dim), dtype=torch.float32, device=dev)
    for lo in range(0, n, LARGE_BLOCK):
        rows = datasets.device_rows(spec, lo, min(LARGE_BLOCK, n - lo), dev, cent)
        p = pos[lo:lo + rows.shape[0]]
        keep = (p >= r_lo) & (p < r_hi)
        d_mine[p[keep] - r_lo] = rows[keep]
        del rows
    del pos
    use_u8 = args.rows_u8 and spec.kind in ("int_mixture", "int_lowrank_mixture")
    h_rows = large.pinned_empty((mine, dim), np.uint8 if use_u8 else np.float32)
    t_rows = large._PINNED[id(h_rows)]
    t_rows.copy_(d_mine.to(torch.uint8) if use_u8 else d_mine)
    del d_mine
    torch.cuda.synchronize(dev)
    torch.cuda.empty_cache()

    # ---- build (timed: wall clock around the streamed pass; kernel seconds per stage beside it) ----
    degree = spec.graph_degree
    index = large.GLIDE_large(ctx, degree, metric, h_rows, h_map, d_centroids.cpu().numpy(), seg_start, seg_len, row_offset=r_lo)
    cfg = pipeline.BuildConfig(metric=metric, graph_degree=degree, knn_degree=32)
    p_knn, p_refine = pipeline.derive_build_search_params(cfg)
    my_parts = np.arange(p_lo, p_hi, dtype=np.uint32)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(dev)
    t0 = time.perf_counter()
    index.build(IndexParameter(degree, 32, 1.05, metric), p_knn, p_refine, seed=spec.seed, partitions=my_parts)
    torch.cuda.synchronize(dev)
    build_wall = time.perf_counter() - t0
    stage = dict(index.stage_seconds)
    bstats = dict(index.stats)
    tb = torch.tensor([build_wall] + [stage[k] for k in ("knn", "subgraph_build", "reverse_graph", "refine")],
                      dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tb, op=dist.ReduceOp.MAX)
    build_wall_max = float(tb[0])

    # ---- search ----
    resident = index.make_resident(int(150e9), partitions=my_parts)
    set_ids = torch.empty((world, Q, TOP_K), dtype=torch.int32, device=dev)
    set_d = torch.empty((world, Q, TOP_K), dtype=torch.float32, device=dev)
    out_ids = api._u32_tensor(ctx, (Q, TOP_K))
    out_d = ctx.empty((Q, TOP_K), torch.float32)
    offs = [r * Q for r in range(world)]
    cnts = [Q] * world
    coll = sharded.GlideCollectives(ctx) if world > 1 else None

    def search(sp):
        """(ids on the host, seconds of this rank's kernels, wall seconds including the gather and the merge)"""
        torch.cuda.synchronize(dev)
        t1 = time.perf_counter()
        d_i, d_dd, ksec = index.search_device(sp, args.route_min, args.route_factor, d_queries, partitions=my_parts)
        if world == 1:
            torch.cuda.synchronize(dev)
            return api.to_u32(d_i), ksec, time.perf_counter() - t1
        set_ids[rank].copy_(d_i)
        set_d[rank].copy_(d_dd)
        coll.all_gather_v(set_ids.view(world * Q, TOP_K), offs, cnts)
        coll.all_gather_v(set_d.view(world * Q, TOP_K), offs, cnts)
        coll.sync()
        ctx.check(ctx.lib.glide_merge_results(ctx.handle, set_ids.data_ptr(), set_d.data_ptr(), world, Q, TOP_K,
                                              out_ids.data_ptr(), out_d.data_ptr()))
        torch.cuda.synchronize(dev)
        return api.to_u32(out_ids), ksec, time.perf_counter() - t1

    gt = gt_i.to(torch.int32).cpu().numpy().view(np.uint32)
    if world > 1:   # every rank measures recall against rank 0's ground truth
        g = torch.from_numpy(gt.view(np.int32).copy()).to(dev)
        dist.broadcast(g, src=0)
        gt = g.cpu().numpy().view(np.uint32)
    chosen, curve = None, []
    for beam in [b for b in BEAM_LADDER if b <= args.max_beam]:
        sp = pipeline.derive_search_params(beam, degree, TOP_K)
        ids, ksec, wall = search(sp)
        rec = api.calculate_recall(ids, gt, TOP_K)
        curve.append({"beam": beam, "recall": round(rec, 4), "qps_wall": round(Q / wall, 1)})
        chosen = (beam, sp, rec)
        if rec >= TARGET_RECALL:
            break
    beam, sp, recall = chosen
    for _ in range(args.warmup):
        search(sp)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    if world > 1:
        dist.barrier()   # after the sampler has started: a late rank 0 would make the others wait inside the first gather
    torch.cuda.synchronize(dev)
    ksum = wsum = 0.0
    for _ in range(args.steps):
        _, ksec, wall = search(sp)
        ksum += ksec
        wsum += wall
    sstats = dict(index.stats)
    clocks = sampler.stop() if rank == 0 else None
    ts = torch.tensor([ksum, wsum], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ts, op=dist.ReduceOp.MAX)
    kmax, wmax = float(ts[0]), float(ts[1])
    # ---- more than one rank: the same search with the QUERIES split over the ranks instead of the
    # partitions. Every rank receives the partitions the others built (rows as fp32, graph rows, id
    # maps: NCCL broadcasts into resident buffers), searches all partitions for its slice of the
    # queries, and the slices are gathered; no merge is needed. ----
    by_query = None
    if world > 1 and (n * dim * 4 + n * degree * 4 + n * 4) < 150e9 and resident == len(my_parts):
        owner_of = np.empty(S, np.int64)
        for r, (lo_p, hi_p) in enumerate(owners):
            owner_of[lo_p:hi_p] = r
        sp_all = torch.from_numpy(index.start_point_view().astype(np.int64)).to(dev)
        sp_all[torch.from_numpy(owner_of != rank).to(dev)] = 0
        dist.all_reduce(sp_all)
        index.set_start_points(sp_all.cpu().numpy().astype(np.uint32))
        torch.cuda.synchronize(dev)
        t_r = time.perf_counter()
        received = index.replicate_partitions(owner_of.tolist(), rank)
        replicate_wall = time.perf_counter() - t_r
        q_lo, q_hi = sharded.split_range(Q, world, rank)
        my_q = d_queries[q_lo:q_hi].contiguous()
        full_ids = torch.zeros((Q, TOP_K), dtype=torch.int32, device=dev)
        q_offs = [sharded.split_range(Q, world, r)[0] for r in range(world)]
        q_cnts = [sharded.split_range(Q, world, r)[1] - sharded.split_range(Q, world, r)[0] for r in range(world)]

        def search_by_query():
            torch.cuda.synchronize(dev)
            t1 = time.perf_counter()
            d_i, _, ksec = index.search_device(sp, args.route_min, args.route_factor, my_q)
            full_ids[q_lo:q_hi].copy_(d_i)
            coll.all_gather_v(full_ids, q_offs, q_cnts)
            coll.sync()
            torch.cuda.synchronize(dev)
            return ksec, time.perf_counter() - t1

        for _ in range(max(args.warmup, 1)):
            search_by_query()
        rec_q = api.calculate_recall(api.to_u32(full_ids), gt, TOP_K)
        dist.barrier()
        kq = wq = 0.0
        for _ in range(args.steps):
            ksec, wall = search_by_query()
            kq += ksec
            wq += wall
        tq = torch.tensor([kq, wq, replicate_wall], dtype=torch.float64, device=dev)
        dist.all_reduce(tq, op=dist.ReduceOp.MAX)
        by_query = {"recall_at_10": round(rec_q, 4), "kernel_qps": Q * args.steps / float(tq[0]),
                    "wall_qps_with_gather": Q * args.steps / float(tq[1]),
                    "replication": {"bytes_received_rank0": received, "wall_seconds": round(float(tq[2]), 3)},
                    "note": "every rank holds every partition (rows, graph, id map received over NCCL) and searches its "
                            "slice of the queries; beam as above"}
    # ---- the merged index on the same build (one GPU, sets whose two copies fit): links across partition
    # borders, then ONE beam search per query instead of one per routed partition ----
    merged = None
    if world == 1 and args.merged and resident == len(my_parts) and (n * dim * 4 * 2 + n * degree * 4 * 3) < 150e9:
        torch.cuda.empty_cache()   # the arena is allocated by the library, outside torch's pool
        t_m = time.perf_counter()
        mstats = index.build_with_merge(args.route_factor, link_count=8, link_beam=32)
        torch.cuda.synchronize(dev)
        merge_wall = time.perf_counter() - t_m
        mchosen, mcurve = None, []
        for mbeam in [b for b in BEAM_LADDER if b <= args.max_beam]:
            msp = pipeline.derive_search_params(mbeam, degree, TOP_K)
            d_i, _, ksec = index.search_merged_device(msp, d_queries)
            rec = api.calculate_recall(api.to_u32(d_i), gt, TOP_K)
            mcurve.append({"beam": mbeam, "recall": round(rec, 4), "qps": round(Q / ksec, 1)})
            mchosen = (mbeam, msp, rec)
            if rec >= TARGET_RECALL:
                break
        mbeam, msp, mrec = mchosen
        for _ in range(args.warmup):
            index.search_merged_device(msp, d_queries)
        msum = 0.0
        for _ in range(args.steps):
            msum += index.search_merged_device(msp, d_queries)[2]
        merged = {"merge_wall_seconds": round(merge_wall, 3), "link_seconds": round(mstats["link_seconds"], 4),
                  "reverse_seconds": round(mstats["reverse_seconds"], 4), "rows_with_links": mstats["rows_with_links"],
                  "link_rule": f"partitions within {args.route_factor} of the nearest centroid, 8 links per point, beam 32",
                  "beam": mbeam, "recall_at_10": round(mrec, 4), "qps": Q * args.steps / msum, "recall_curve": mcurve}
    if rank == 0:
        line = {
            "metric": METRIC_NAME, "value": Q * args.steps / kmax, "unit": "queries/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": kmax / args.steps * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic (drawn on the device, seeded per block of 2^20 rows)",
            "config": {"workload": f"{spec.name}: {n}x{dim} {'uint8' if use_u8 else 'fp32'} {spec.metric}, large path, {S} partitions, "
                                   f"{Q} queries, k={TOP_K}, graph degree {degree}",
                       "beam": beam, "reduced": reduced, "route_min_partitions": args.route_min, "route_factor": args.route_factor,
                       "l2": "partitions larger than L2 walked per query batch",
                       "multi_gpu": "partitions owned by ranks; per-rank top-k gathered (NCCL) and merged" if world > 1 else "single GPU"},
            "recall_at_10": round(recall, 4), "recall_target_reached": bool(recall >= TARGET_RECALL), "recall_curve": curve,
            "build": {"wall_seconds": round(build_wall_max, 3),
                      "kernel_seconds_max_over_ranks": {k: round(float(v), 4) for k, v in
                                                        zip(("knn", "subgraph_build", "reverse_graph", "refine"), tb[1:].tolist())},
                      "rank0": {"rows": mine, "partitions": int(p_hi - p_lo), "h2d_gbs": round(bstats["h2d_bytes"] / max(bstats["h2d_seconds"], 1e-9) / 1e9, 2),
                                "h2d_bytes": bstats["h2d_bytes"], "upload_stream_seconds": round(bstats["h2d_seconds"], 3)},
                      "untimed": {"assignment_kernel_seconds": round(assign_s, 3), "ground_truth_kernel_seconds": round(gt_s, 3)}},
            "search": {"resident_partitions_rank0": resident, "partitions_searched_rank0": sstats.get("partitions_searched"),
                       "partitions_uploaded_rank0": sstats.get("partitions_uploaded"),
                       "kernel_qps": Q * args.steps / kmax, "wall_qps_with_gather_and_merge": Q * args.steps / wmax},
            "e2e": {"value": Q * args.steps / wmax, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": Q * TOP_K * 4,
                    "note": "wall clock of the public call on device-resident queries, result ids read back to the host"},
            "gpu_launches": None, "clocks": clocks,
        }
        if merged is not None:
            line["merged_index"] = merged
        if by_query is not None:
            line["search_with_queries_split_over_ranks"] = by_query
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    index.close()
    ctx.close()


# --------------------------------------------------------------------------------------------
# loader (row f4: matrix file -> pinned host memory, overlapped with partition assignment)
# --------------------------------------------------------------------------------------------
def run_loader(args):
    """Not a bench line of the contract: one JSON line with the loader's throughput on a synthetic
    matrix file (cfg4's row shape: 128 uint8 or fp32 values per row, `--rows` of them, written to
    `--loader-dir`), beside the reference's row-by-row reader timed on the same file."""
    import tempfile
    import torch
    from glide_b200 import api, large
    from glide_b200.params import Metric
    ctx = api.Context(0)
    dtype = np.uint8 if args.rows_u8 else np.float32
    rows, dim, C = args.rows or 8_000_000, 128, args.partitions or 512
    rng = np.random.default_rng(5)
    folder = tempfile.mkdtemp(dir=args.loader_dir)
    path = os.path.join(folder, "rows.bin")
    block = rng.integers(0, 256, (1 << 20, dim)).astype(dtype)
    with open(path, "wb") as f:
        np.array([rows, dim], np.uint32).tofile(f)
        left = rows
        while left > 0:
            block[:min(left, block.shape[0])].tofile(f)
            left -= block.shape[0]
    file_gb = (8 + rows * dim * np.dtype(dtype).itemsize) / 1e9
    d_centroids = torch.from_numpy(rng.integers(0, 256, (C, dim)).astype(np.float32)).to(ctx.torch_device)
    out = {"loader": "glide_load_rows", "file": f"{rows}x{dim} {np.dtype(dtype).name}, {file_gb:.2f} GB in {args.loader_dir}",
           "partitions": C, "host_cores": os.cpu_count()}
    try:
        for name, kw in (("read_only_4_threads", dict(threads=4)), ("read_only_8_threads", dict(threads=8)),
                         ("read_and_assign_4_threads", dict(threads=4, d_centroids=d_centroids)),
                         ("read_and_assign_8_threads", dict(threads=8, d_centroids=d_centroids))):
            best = None
            for _ in range(3):
                h_rows, nearest, st = large.load_rows(ctx, path, dtype, metric=Metric.Euclidean, **kw)
                if best is None or st["total_seconds"] < best["total_seconds"]:
                    best = st
                keep = (h_rows, nearest)
            out[name] = {"GB/s": round(file_gb / best["total_seconds"], 2), "seconds": round(best["total_seconds"], 4),
                         "read_seconds": round(best["read_seconds"], 4),
                         "device_waited_for_file_seconds": round(best["device_waited_seconds"], 4)}
        # assignment alone on rows already in pinned memory: what the overlap hides
        t0 = time.perf_counter()
        pre_rows = keep[0]
        step = 1 << 19
        for lo in range(0, rows, step):
            d_rows = torch.from_numpy(pre_rows[lo:lo + step]).to(ctx.torch_device).to(torch.float32)
            api.define_partition(ctx, d_rows, d_centroids, -1.0, Metric.Euclidean)
        torch.cuda.synchronize()
        out["upload_and_assign_after_the_read"] = {"seconds": round(time.perf_counter() - t0, 4)}
        if not args.no_cpu_baseline:
            import oracle
            t0 = time.perf_counter()
            ref_rows = oracle.load_matrix_rowwise(path, dtype)
            dt = time.perf_counter() - t0
            out["reference_row_by_row_reader"] = {"GB/s": round(file_gb / dt, 2), "seconds": round(dt, 4),
                                                  "kind": "port of load.cuh:10-30 (one ifstream read per row, pageable memory), 1 thread",
                                                  "rows_equal": bool(np.array_equal(ref_rows, keep[0]))}
    finally:
        os.remove(path)
        os.rmdir(folder)
    print(json.dumps(out), flush=True)
    ctx.close()


def main():
    args = parse_args()
    if args.config == "loader":
        if int(os.environ.get("RANK", "0")) == 0:
            run_loader(args)
        return
    if args.config in LARGE:
        if args.impl == "reference":
            if int(os.environ.get("RANK", "0")) == 0:
                print(json.dumps({"impl": "reference", "unavailable": "the reference's large path does not compile as shipped "
                                  "(glide_large.cuh:182 against glide_large_impl.cuh:79) and has no CPU implementation"}), flush=True)
            return
        run_large(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

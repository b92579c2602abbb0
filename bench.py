"""Benchmark of the ANN graph build / beam search hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c2]

One "step" is one complete graph build (`ANN(vectors=...)`: circulant start graph, up to
`optimization_loops` rounds of fused beam search + prune + self-recall check) over the
workload's synthetic vectors.  The JSON line reports build vectors/s (`value`, inputs already
in HBM; `e2e` with host buffers), the search QPS and recall@10 of the built graph, the
roofline of the dominant kernel (per launch class: the first build round, the later rounds, the
search), and a CPU baseline (the C oracle on a bounded sample).
`--impl reference` times the reference's algorithm on the host cores only (the C oracle, all
threads) on a bounded sample of the same workload.  The reference's own Numba kernels are not run
on the GPU: below 1024 dimensions they read shared memory past what was written or allocated
(kernels.py:50-69,217,231) and after a prune they index vectors[MAXINT] (kernels.py:245-247).
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
for _p in (ROOT, os.path.join(ROOT, "vectorlink-gpu_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import numpy as np
import torch

# workload shapes follow BASELINE.json's configs; all data is synthetic with seed 0.
WORKLOADS = {
    # config 1: 2,000 x 64 unit vectors, cosine, degree 16, beam 32
    "c1": dict(n=2_000, dim=64, metric="cosine", degree=16, beam=32, queries=100, kind="gauss_unit"),
    # config 2: 1,000,000 x 128 SIFT-like integer mixture, L2, degree 32, beam 64, 10,000 queries
    "c2": dict(n=1_000_000, dim=128, metric="l2", degree=32, beam=64, queries=10_000, kind="sift_like", centres=256),
    # config 3: 1,000,000 x 768 unit-norm embedding-like mixture, cosine, degree 64, beam 128
    "c3": dict(n=1_000_000, dim=768, metric="cosine", degree=64, beam=128, queries=10_000, kind="embed_like",
               centres=1000, noise=0.1, unit_centres=True),
    # config 4 (per-GPU shard of it at N GPUs): 10,000,000 x 96 Deep-like, cosine, degree 32
    # (centres are plain N(0,1) draws, norm ~ 9.8, not normalised; only the rows are)
    "c4": dict(n=10_000_000, dim=96, metric="cosine", degree=32, beam=64, queries=10_000, kind="embed_like",
               centres=4096, noise=0.3, unit_centres=False),
    # config 5 (20,000,000 x 1024 over 8 GPUs): cosine, degree 64, beam 128, 100,000 queries
    "c5": dict(n=20_000_000, dim=1024, metric="cosine", degree=64, beam=128, queries=100_000, kind="embed_like",
               centres=16384, noise=0.05, unit_centres=True),
}


def ann_kwargs(w):
    """Parameter mapping: beam_size = degree; recall_search_queue_factor = visit_queue_factor =
    beam / degree; every other ANN keyword at its default.  search_seed_factor widens the
    seed scan so that a seed lands in the query's cluster (the data has separated clusters)."""
    f = max(1, w["beam"] // w["degree"])
    kw = dict(beam_size=w["degree"], visit_queue_factor=f, recall_search_queue_factor=f, metric=w["metric"])
    if w["kind"] != "gauss_unit":
        kw["search_seed_factor"] = 30
    return kw


def make_data(w, n, device, seed=0, queries=None):
    """Generator order: centres -> assignments -> noise -> queries (one torch generator)."""
    g = torch.Generator(device=device).manual_seed(seed)
    dim = w["dim"]
    nq = w["queries"] if queries is None else queries

    def draw(count):
        if w["kind"] == "gauss_unit":
            x = torch.randn((count, dim), device=device, generator=g)
            return torch.nn.functional.normalize(x, dim=1)
        out = torch.empty((count, dim), device=device)
        for lo in range(0, count, 1_000_000):
            hi = min(count, lo + 1_000_000)
            assign = torch.randint(0, centres.size(0), (hi - lo,), device=device, generator=g)
            noise = torch.randn((hi - lo, dim), device=device, generator=g)
            if w["kind"] == "sift_like":
                out[lo:hi] = (centres[assign] + 20.0 * noise).round().clamp(0, 255)
            else:
                out[lo:hi] = torch.nn.functional.normalize(centres[assign] + w["noise"] * noise, dim=1)
        return out

    centres = None
    if w["kind"] == "sift_like":
        centres = torch.rand((w["centres"], dim), device=device, generator=g) * 255.0
    elif w["kind"] == "embed_like":
        centres = torch.randn((w["centres"], dim), device=device, generator=g)
        if w.get("unit_centres", True):
            centres = torch.nn.functional.normalize(centres, dim=1)
    vectors = draw(n)
    q = draw(nq)
    return vectors.contiguous(), q.contiguous()


def brute_force_topk(vectors, queries, k, metric, query_chunk=8192):
    """Exact top-k on the GPU in fp32 (ground truth for recall; measurement harness only)."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.set_float32_matmul_precision("highest")
    out = []
    for q0 in range(0, queries.size(0), query_chunk):
        qs = queries[q0:q0 + query_chunk]
        best_d = torch.full((qs.size(0), k), float("inf"), device=vectors.device)
        best_i = torch.zeros((qs.size(0), k), dtype=torch.int64, device=vectors.device)
        qn = (qs * qs).sum(1, keepdim=True)
        for lo in range(0, vectors.size(0), 262_144):
            blk = vectors[lo:lo + 262_144]
            dots = qs @ blk.t()
            d = (qn - 2 * dots + (blk * blk).sum(1).unsqueeze(0)) if metric == "l2" else (1 - dots) / 2
            cd, ci = torch.topk(d, min(k, blk.size(0)), dim=1, largest=False)
            alld = torch.cat([best_d, cd], 1)
            alli = torch.cat([best_i, ci + lo], 1)
            best_d, sel = torch.topk(alld, k, dim=1, largest=False)
            best_i = torch.gather(alli, 1, sel)
        out.append(best_i)
    torch.backends.cuda.matmul.allow_tf32 = prev
    return torch.cat(out, 0) if out else torch.zeros((0, k), dtype=torch.int64, device=vectors.device)


def recall_at_k(found_ids, truth, k):
    f = found_ids[:, :k].long()
    hits = (f.unsqueeze(2) == truth[:, :k].unsqueeze(1)).any(2).sum().item()
    return hits / (truth.size(0) * k)


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 9 for i in range(4) if r[5 + i] == "Active"})
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def oracle_build_rate(w, sample_n, seed=0):
    """The C oracle (all host threads) building the graph of a `sample_n`-vector draw of the
    workload with the same ANN parameters; returns (vectors/s, seconds, loops, threads)."""
    import oracle
    # a launcher that starts several workers per node exports OMP_NUM_THREADS=1 to each of them;
    # this leg runs on one rank only and is meant to use the host's cores
    oracle.set_num_threads(os.cpu_count() or 1)
    vec, _ = make_data(w, sample_n, "cpu", seed, queries=1)
    kw = ann_kwargs(w)
    metric = kw.pop("metric")
    kw.pop("search_seed_factor", None)
    cfg = oracle.make_config(**kw)
    t0 = time.time()
    _, _, loops, _ = oracle.generate_ann(vec.numpy(), cfg, metric=metric)
    dt = time.time() - t0
    return sample_n / dt, dt, loops, oracle.num_threads()


def default_sample(w):
    """Vectors in the CPU sample: about 10-30 s of oracle work on 16-32 host cores."""
    return max(500, min(w["n"], int(2_000_000 / (w["dim"] * (w["degree"] / 16)))))


def run_reference(args, w, name):
    """The reference's CPU implementation of the path on the host cores: the C restatement of its
    algorithm (oracle/), OpenMP over all cores, building the graph of a bounded sample of the
    workload.  (The reference's own kernels exist only as Numba CUDA kernels: the Numba simulator
    runs them at about one CUDA block per second, and on the GPU they read out of range below 1024
    dimensions, see the module docstring - neither is a usable timing arm.)"""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample = args.sample or default_sample(w)
    budget_s = 240.0                       # the whole arm ends within a few minutes
    t_begin = time.time()
    for _ in range(min(args.warmup, 1)):
        oracle_build_rate(w, min(sample, 500))
    rates, secs = [], []
    for i in range(args.steps):
        rate, dt, loops, threads = oracle_build_rate(w, sample)
        rates.append(rate)
        secs.append(dt)
        if time.time() - t_begin + dt > budget_s:      # no room for another step of this length
            break
    ms = float(np.mean(secs)) * 1e3
    value = float(np.mean(rates))
    line = {"impl": "reference", "metric": "graph_build_vectors_per_s", "value": value, "unit": "vectors/s",
            "n_gpus": args.gpus, "steps": len(rates), "warmup": min(args.warmup, 1), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": name, "sample_vectors": sample, **{k: v for k, v in ann_kwargs(w).items()}},
            "cpu_baseline": {"value": value, "unit": "vectors/s", "cores": threads, "kind": "port",
                             "sample": f"full build of a {sample}-vector draw of {name} ({loops} loops), C oracle with OpenMP"},
            "e2e": {"value": value, "unit": "vectors/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
            "numba_on_gpu": "not run: the reference's kernels read shared memory out of range for dim < 1024 "
                            "(kernels.py:217,231) and index vectors[MAXINT] after a prune (kernels.py:245-247)"}
    print(json.dumps(line), flush=True)


def launch_classes(profile, reps, dim):
    """Fused-kernel launches of a timed region grouped by phase (first build round / later build
    rounds / self-recall check / search), each with its mean duration (CUDA events recorded around
    the launch on the launching stream), the distance evaluations the reference's schedule
    prescribes and the candidate rows the kernel actually loaded (its own counter)."""
    bytes_per_row = 4 * dim + 12          # candidate row + neighbour id + (id, distance) result
    groups = {}
    for p in profile:
        tag = p.get("tag", "search")
        cls = "build_round0" if tag == "round0" else ("build_later_rounds" if tag.startswith("round") else tag)
        groups.setdefault(cls, []).append(p)
    out = {}
    for cls, ps in groups.items():
        ms = sum(p["start"].elapsed_time(p["end"]) for p in ps)
        evals = sum(p["evals"] for p in ps)
        gathered = sum(int(p["stats"][1].item()) for p in ps if p.get("stats") is not None)
        out[cls] = {"launches_per_step": len(ps) / reps, "ms_per_launch": ms / len(ps),
                    "evals_per_launch": evals / len(ps), "gathered_rows_per_launch": gathered / len(ps),
                    "gathered_fraction": gathered / evals if evals else None,
                    "memo": all(p["memo"] for p in ps),
                    "schedule_gbs": evals * bytes_per_row / (ms * 1e-3) / 1e9 if ms else None,
                    "gathered_gbs": gathered * bytes_per_row / (ms * 1e-3) / 1e9 if ms else None}
    return out


def dram_captures(workload):
    """ncu DRAM counters of earlier captures of this workload, kept as data beside the summaries."""
    try:
        doc = json.load(open(os.path.join(ROOT, "profiles", "dram_traffic.json")))
        return [c for c in doc["captures"] if c["workload"] == workload]
    except Exception:
        return []


def roofline_of(build_classes, search_classes, peak, peak_kind, workload, dim, kernel_share):
    """Three figures per launch class, all against the measured HBM copy bandwidth:
    `vs_reference_schedule` - bytes the reference's schedule would move (every evaluation gathers
        its row), per second: can exceed 1 because the kernel memoises distances per query row;
    `gathered` - bytes of the candidate rows the kernel really loaded, per second: the achieved
        bandwidth of the gather, whichever level of the memory system served it;
    `dram` - DRAM bytes of an ncu capture of the same launch class (scaled by gathered rows).
    The headline `achieved`/`frac` is `gathered` of the build's later rounds, whose rows come from
    DRAM; the first round's candidates lie in a band of rows that stays in L2, so its `gathered`
    figure is an L2 rate and is reported but not used as the HBM fraction."""
    classes = {}
    caps = dram_captures(workload)
    for cls, c in list(build_classes.items()) + [("search", search_classes.get("search"))]:
        if not c:
            continue
        entry = dict(c)
        entry["vs_reference_schedule"] = c["schedule_gbs"] / peak if c["schedule_gbs"] else None
        entry["gathered_frac"] = c["gathered_gbs"] / peak if c["gathered_gbs"] else None
        for cap in caps:
            if cap["class"] == cls and bool(cap["memo"]) == bool(c["memo"]):
                traffic = cap["dram_bytes_per_gathered_row"] * c["gathered_rows_per_launch"]
                entry["dram_traffic_bytes"] = traffic
                entry["dram_gbs"] = traffic / (c["ms_per_launch"] * 1e-3) / 1e9
                entry["dram_frac"] = entry["dram_gbs"] / peak
                entry["dram_capture"] = {k: cap[k] for k in ("commit", "summary") if k in cap}
        classes[cls] = entry
    head = classes.get("build_later_rounds") or classes.get("build_round0") or {}
    served = "DRAM" if "build_later_rounds" in classes else "mostly L2 (single-round build: circulant band)"
    return {"bound": "hbm", "kernel": "beam_search_kernel", "class": "build_later_rounds" if "build_later_rounds" in classes else "build_round0",
            "achieved": head.get("gathered_gbs"), "peak": peak, "unit": "GB/s",
            "frac": (head.get("gathered_gbs") or 0.0) / peak, "peak_source": peak_kind,
            "frac_of_8TBs_nominal": (head.get("gathered_gbs") or 0.0) / 8000.0,
            "achieved_counts": "bytes of candidate rows actually loaded (kernel counter) x (4*dim+12) / CUDA-event time",
            "rows_served_from": served, "bytes_per_row": 4 * dim + 12,
            "traffic": head.get("dram_traffic_bytes"), "kernel_share_of_step": kernel_share, "classes": classes}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--workload", default="c2")
    ap.add_argument("--vectors", dest="n", type=int, default=0, help="override the vector count (per GPU)")
    ap.add_argument("--sample", type=int, default=0, help="vectors in the CPU baseline sample")
    ap.add_argument("--queries", type=int, default=0, help="override the number of search queries")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--loops", type=int, default=0, help="override optimization_loops")
    ap.add_argument("--quick", action="store_true", help="skip the host-buffer pass and the recall evaluation")
    ap.add_argument("--entry-sample", type=int, default=0,
                    help="start searches from tensor-core entry points (best 64 of this many evenly spaced rows) "
                         "instead of the widened circulant seed scan")
    ap.add_argument("--no-tile-start", action="store_true", help="skip the extra builds with the tensor-core start graph")
    ap.add_argument("--skip-e2e", action="store_true", help="skip only the host-buffer pass (long single builds)")
    ap.add_argument("--init", default="circulant", choices=["circulant", "knn_tile"],
                    help="start graph of the build: the reference's circulant graph (default) or the tensor-core tile pass")
    ap.add_argument("--mode", default="rows", choices=["rows", "shards"], help="multi-GPU build mode (see sharded.py)")
    ap.add_argument("--merge", default="tile", choices=["tile", "search"], help="how mode shards finds cross-shard neighbours")
    args = ap.parse_args()
    name = args.workload
    w = dict(WORKLOADS[name])
    if args.n:
        w["n"] = args.n
    if args.queries:
        w["queries"] = args.queries
    if args.impl == "reference":
        run_reference(args, w, name)
        return

    import torch.distributed as dist
    from vectorlink_gpu import ANN, _lib
    from vectorlink_gpu import ann as vl_ann

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    kw = ann_kwargs(w)
    if args.loops:
        kw["optimization_loops"] = args.loops
    if args.entry_sample:
        kw.pop("search_seed_factor", None)
        kw["search_entry_sample"] = args.entry_sample
    if args.init != "circulant":
        kw["init"] = args.init
        if not args.loops:
            # the lists of the tile pass are already near neighbours: one round (search + prune) ends in the same
            # graph as three (measured on config 2), so that is how this start graph is meant to be used
            kw["optimization_loops"] = 1
    # strong scaling: the job is always the workload's w["n"] vectors; rank r starts with rows
    # [lo_r, hi_r) of them in its HBM.  A step all-gathers the shards and runs the build with every
    # round's rows split across the ranks (ShardedANN mode "rows"): the graph is bit-identical to
    # the one a single GPU builds, whatever the number of ranks.
    total = w["n"]
    full, queries = make_data(w, total, dev, seed=0)
    if world > 1:
        from vectorlink_gpu.sharded import partition_rows
        lo, hi = partition_rows(total, world)[rank]
        vectors = full[lo:hi].clone()
        del full
        torch.cuda.empty_cache()
    else:
        vectors = full
    n = vectors.size(0)
    dim = vectors.size(1)
    do_e2e = not (args.quick or args.skip_e2e)
    if do_e2e:
        host_vectors = torch.empty((n, dim), dtype=torch.float32, pin_memory=True)
        host_vectors.copy_(vectors)
        host_beams = torch.empty((n, kw["beam_size"]), dtype=torch.int32, pin_memory=True)
        host_dist = torch.empty((n, kw["beam_size"]), dtype=torch.float32, pin_memory=True)

    if world > 1:
        from vectorlink_gpu.sharded import ShardedANN

    def build(v):
        if world > 1:
            return ShardedANN(v, group=dist.group.WORLD, mode=args.mode, merge=args.merge, **kw)
        return ANN(vectors=v, **kw)

    def step_device():
        return build(vectors)

    def step_e2e():
        v = host_vectors.to(dev, non_blocking=True)
        a = build(v)
        host_beams.copy_(a.beams, non_blocking=True)
        host_dist.copy_(a.distances, non_blocking=True)
        torch.cuda.synchronize(dev)
        return a

    for _ in range(args.warmup):
        ann = step_device()
    barrier()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    vl_ann.PROFILE = []
    launches0 = _lib.LAUNCHES
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        ann = step_device()
    ev1.record()
    barrier()
    launches = _lib.LAUNCHES - launches0
    loops_run = vl_ann.generate_ann.last_loops
    profile = vl_ann.PROFILE
    vl_ann.PROFILE = None
    ms_total = ev0.elapsed_time(ev1)
    clocks = sampler.stop() if rank == 0 else None

    build_classes = launch_classes(profile, args.steps, dim)
    kernel_share = sum(p["start"].elapsed_time(p["end"]) for p in profile) / ms_total if profile else 0.0

    # end to end with host buffers
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if do_e2e:
        step_e2e()
        barrier()
    e0.record()
    if do_e2e:
        for _ in range(args.steps):
            step_e2e()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) if do_e2e else float("nan")

    # search over the built graph (data-parallel over the ranks when there are several)
    def do_search():
        if world > 1:
            return ann.search(queries)[0]
        return ann.search(queries).indices

    found = do_search()
    barrier()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = max(3, args.steps)
    vl_ann.PROFILE = []
    s0.record()
    for _ in range(reps):
        found = do_search()
    s1.record()
    barrier()
    sprof = vl_ann.PROFILE
    vl_ann.PROFILE = None
    search_ms = s0.elapsed_time(s1) / reps
    search_classes = launch_classes(sprof, reps, dim)
    recall = graph_recall = None
    want_recall = not args.quick and rank == 0          # the ground truth is brute force: one rank computes it
    if want_recall:
        index = ann.index if world > 1 else ann
        n_eval = min(queries.size(0), 10_000)           # recall is evaluated on the first 10,000 queries at most
        truth = brute_force_topk(index.vectors, queries[:n_eval], 10, w["metric"])
        recall = recall_at_k(found[:n_eval], truth, 10)
        gsample = min(index.vectors.size(0), 10_000)
        gtruth = brute_force_topk(index.vectors, index.vectors[:gsample], 11, w["metric"])[:, 1:]
        graph_recall = recall_at_k(index.beams[:gsample], gtruth, 10)

    # the opt-in tensor-core start graph, beside the headline (which is the reference's algorithm): same
    # data, same queries, one round
    tile_start = None
    if not args.quick and args.init == "circulant" and not args.no_tile_start:
        kw_tile = dict(kw, init="knn_tile", optimization_loops=1)
        # its searches start from tensor-core entry points (best 64 of 65,536 evenly spaced rows) instead of
        # the widened circulant seed scan
        kw_tile.pop("search_seed_factor", None)
        kw_tile["search_entry_sample"] = min(total, 65_536)

        def build_tile():
            if world > 1:
                return ShardedANN(vectors, group=dist.group.WORLD, mode=args.mode, merge=args.merge, **kw_tile)
            return ANN(vectors=vectors, **kw_tile)

        ann = None                      # frees the first index before the second is built
        alt = build_tile()
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        alt_steps = min(args.steps, 3)            # a side measurement: a few builds are enough
        t0.record()
        for _ in range(alt_steps):
            alt = build_tile()
        t1.record()
        barrier()
        alt_ms = torch.tensor([t0.elapsed_time(t1) / alt_steps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(alt_ms, op=dist.ReduceOp.MAX)
        alt_index = alt.index if world > 1 else alt
        def alt_search():
            return alt.search(queries)[0] if world > 1 else alt.search(queries).indices

        alt_found = alt_search()
        barrier()
        q0, q1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        q0.record()
        for _ in range(reps):
            alt_found = alt_search()
        q1.record()
        barrier()
        alt_q = torch.tensor([q0.elapsed_time(q1) / reps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(alt_q, op=dist.ReduceOp.MAX)
        # the tile pass alone, timed live (CUDA events, all pairs of this GPU's rows): its roofline is the tensor one
        tile_pass = None
        if world == 1 and total <= 2_000_000:          # all pairs: the cost grows with the square of the rows
            from vectorlink_gpu import knn_tile
            rows_bf16, norms = knn_tile.prepare(vectors, want_norms=w["metric"] == "l2")
            knn_tile.proposals(rows_bf16, norms, (0, total), (0, total), 1)
            p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            p0.record()
            for _ in range(3):
                knn_tile.proposals(rows_bf16, norms, (0, total), (0, total), 1)
            p1.record()
            torch.cuda.synchronize()
            pass_ms = p0.elapsed_time(p1) / 3
            tflops = 2.0 * total * total * rows_bf16.size(1) / (pass_ms * 1e-3) / 1e12
            tile_pass = {"kernel": "knn_tile_kernel", "ms_per_launch": pass_ms, "pairs": float(total) * total,
                         "dim_padded": rows_bf16.size(1), "bound": "tensor", "achieved": tflops, "unit": "TFLOP/s"}
            del rows_bf16, norms
        tile_start = {"init": "knn_tile", "optimization_loops": 1, "search_entry_sample": kw_tile["search_entry_sample"],
                      "steps": alt_steps, "ms_per_step": float(alt_ms.item()),
                      "value": total / (float(alt_ms.item()) * 1e-3), "unit": "vectors/s",
                      "graph_recall_at_10": recall_at_k(alt_index.beams[:gsample], gtruth, 10) if want_recall else None,
                      "search_qps": queries.size(0) / (float(alt_q.item()) * 1e-3),
                      "search_recall_at_10": recall_at_k(alt_found[:n_eval], truth, 10) if want_recall else None,
                      "tile_pass": tile_pass}
    status = _lib.read_status(dev)

    times = torch.tensor([ms_total, e2e_ms, search_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms, search_ms = [float(x) for x in times.tolist()]

    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        peak_kind = "measured (MEASURED_PEAKS.json hbm_gbs)" if "hbm_gbs" in peaks else "fallback 6650"
        ms_per_step = ms_total / args.steps
        if tile_start and tile_start.get("tile_pass"):
            tp = tile_start["tile_pass"]
            tp["peak"] = float(peaks.get("bf16_tflops", 1590.0))
            tp["peak_sustained"] = float(peaks.get("bf16_tflops_sustained", 1400.0))
            tp["peak_source"] = ("measured (MEASURED_PEAKS.json bf16_tflops, a burst cuBLAS GEMM)" if "bf16_tflops" in peaks
                                 else "fallback 1590")
            tp["frac"] = tp["achieved"] / tp["peak"]
            tp["frac_of_sustained"] = tp["achieved"] / tp["peak_sustained"]
        line = {
            "metric": "graph_build_vectors_per_s", "value": total / (ms_per_step * 1e-3), "unit": "vectors/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": name, "vectors": total, "vectors_per_gpu": n, "dim": dim, **kw, "loops_run": loops_run,
                       "l2_policy": "inputs (vectors %d MB + graph) exceed the 126 MB L2" % (total * dim * 4 // 2**20),
                       "sharding": ("none" if world == 1 else
                                    ("vectors all-gathered; each round's rows split evenly across ranks, searched and pruned "
                                     "by their rank, lists all-gathered (NCCL): the single-GPU graph") if args.mode == "rows" else
                                    ("each rank builds the graph of its own shard, then a merge pass: rows all-gathered "
                                     "chunk by chunk, every shard scanned for the foreign rows (%s), candidate lists "
                                     "all-gathered and merged by the owner (NCCL)" % args.merge))},
            "e2e": {"value": (total / (e2e_ms / args.steps * 1e-3)) if e2e_ms == e2e_ms else None, "unit": "vectors/s",
                    "h2d_bytes_per_step": total * dim * 4, "d2h_bytes_per_step": total * kw["beam_size"] * 8},
            "gpu_launches": launches,
            "search": {"qps": queries.size(0) / (search_ms * 1e-3), "queries": queries.size(0), "k": 10,
                       "recall_at_10": recall, "ms": search_ms},
            "graph_recall_at_10": graph_recall,
            "tile_start": tile_start,
            "roofline": roofline_of(build_classes, search_classes, peak, peak_kind, name, dim, kernel_share),
            "clocks": clocks, "status_word": status,
        }
        if not args.no_cpu_baseline and world == 1:
            sample = args.sample or default_sample(w)
            rate, dt, loops, threads = oracle_build_rate(w, sample)
            line["cpu_baseline"] = {"value": rate, "unit": "vectors/s", "cores": threads, "kind": "port",
                                    "sample": f"full build of a {sample}-vector draw of {name} ({loops} loops, {dt:.1f} s), "
                                              "C oracle with OpenMP"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

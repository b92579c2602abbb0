"""ANN graph build and beam search with the reference's driver API (vectorlink_gpu/ann.py).

`closest_vectors` runs the whole budgeted search of a batch as one fused kernel
(csrc/vl_beam.cu) whenever the queue shapes allow it, and otherwise steps through the
reference's loop with the operator-level kernels.  Both produce the reference's queues.
"""
from __future__ import annotations

import ctypes
import json
import os
import subprocess
import time
from typing import Dict, List, Optional, Tuple

import torch
from torch import Tensor

from . import _lib
from ._lib import BeamParams, check, lib, ptr, stream_of
from .constants import MAXFLOAT, MAXINT, PRIMES_HOST
from .kernels import calculate_distances, connected_components, metric_code, prune_, search_from_seeds, sort_pairs_
from .log import log_time, nvtx_range
from . import log as _log
from .queue import Queue
from .utils import add_new_to_seen_, generate_circulant_beams, generate_queue_circulants, primes

FUSED_MAX_SMEM_PER_ROW = 200 * 1024
# When set to a list, every fused-kernel launch appends its CUDA events (recorded on the
# launching stream) and its count of distance evaluations: the benchmark's roofline figures.
PROFILE = None
PROFILE_TAG = "search"     # which phase the launches being profiled belong to (generate_ann sets it per round)
# When set to an int64 CUDA tensor of 16 zeros, the fused kernel adds its work counters and
# per-phase warp cycles to it (layout: `stats` in include/vlgpu.h).
STATS = None
STATS_TIMERS = False


def _metric_of(config: Dict):
    return config.get("metric", "cosine")


def _fused_shape_ok(vectors: Tensor, beam_w: int, sq_len: int, sq_cap: int, config: Dict) -> bool:
    """The fused kernel models a queue as "the `length` best of head + candidates", which is
    what Queue.insert computes when capacity == length + candidates per iteration."""
    pvc = config["parallel_visit_count"]
    vq_len = config["visit_queue_factor"] * config["beam_size"]
    m = pvc * beam_w
    e = config["exclude_factor"] * vq_len
    smem = 10 * m + 16 * sq_len + 16 * vq_len + 4 * 6 * max(e, 16) + 4 * vectors.size(1) + 512
    return (vectors.size(1) % 4 == 0 and vectors.data_ptr() % 16 == 0 and 1 <= pvc <= 32 and pvc <= vq_len
            and sq_cap == sq_len + m and sq_len <= 4096 and smem <= FUSED_MAX_SMEM_PER_ROW
            and config["speculative_readahead"] >= 1)


def loop_bounds(config: Dict) -> Tuple[int, int, int]:
    """(k_none, n_checks, n_max) of the reference loop (ann.py:66-91, utils.py:61-82) for a
    batch in which some row always pops real ids: `seen` takes pvc ids per iteration and is
    found full at iteration k_none = ceil(E/pvc)+1; from then on nothing changes, so the loop
    leaves at the first multiple of speculative_readahead after k_none (n_max) unless an
    earlier check saw no change; n_checks = checks at or before k_none."""
    pvc = config["parallel_visit_count"]
    e = config["exclude_factor"] * config["visit_queue_factor"] * config["beam_size"]
    ra = config["speculative_readahead"]
    k_none = (e + pvc - 1) // pvc + 1
    n_checks = k_none // ra
    n_max = (k_none // ra + 1) * ra
    return k_none, n_checks, n_max


def _launch_beam(vectors, graph, queries, seed_ids, seed_dist, seed_cols, sq_len, out_ids, out_dist, out_cols,
                 config, n_iters, dump_last, exclude, self_base, group_rows, flags, full, stats=None, group_row0=0):
    pvc = config["parallel_visit_count"]
    if stats is None:
        stats = STATS
    if stats is None and PROFILE is not None:
        # a profiled launch reports its own counters (gathered candidates, rows, iterations)
        stats = torch.zeros(24, dtype=torch.int64, device=vectors.device)
    vq_len = config["visit_queue_factor"] * config["beam_size"]
    p = BeamParams()
    p.vectors = vectors.data_ptr()
    p.n = vectors.size(0)
    p.dim = vectors.size(1)
    p.metric = metric_code(_metric_of(config))
    p.graph = graph.data_ptr()
    p.graph_w = graph.size(1)
    p.pvc = pvc
    p.queries = queries.data_ptr()
    p.rows = queries.size(0)
    p.seed_ids = seed_ids.data_ptr()
    p.seed_dist = seed_dist.data_ptr()
    p.seed_ld = seed_ids.stride(0)
    p.seed_cols = seed_cols
    p.sq_len = sq_len
    p.vq_len = vq_len
    p.seen_cap = config["exclude_factor"] * vq_len
    p.out_ids = out_ids.data_ptr()
    p.out_dist = out_dist.data_ptr()
    p.out_ld = out_ids.stride(0)
    p.out_cols = out_cols
    p.n_iters = n_iters
    p.readahead = config["speculative_readahead"]
    p.dump_last = 1 if dump_last else 0
    p.exclude_w = exclude.size(1) if exclude is not None else 0
    p.exclude = exclude.data_ptr() if exclude is not None else 0
    p.self_base = self_base
    p.group_rows = group_rows
    p.group_row0 = group_row0
    p.changed_flags = flags.data_ptr()
    p.n_checks = flags.size(1)
    p.group_full = full.data_ptr()
    p.status = _lib.status_word(vectors.device).data_ptr()
    p.memo = 0
    p.memo_entries = 0
    p.memo_slots = 0
    p.stats = stats.data_ptr() if stats is not None else 0
    p.flags = 1 if (stats is not None and stats is STATS and STATS_TIMERS) else 0
    # rows differ in the work they take: warps draw their next row from a counter instead of a fixed stride
    ticket = torch.zeros(1, dtype=torch.int64, device=vectors.device) if config.get("row_ticket", True) else None
    p.row_ticket = ticket.data_ptr() if ticket is not None else 0
    if config.get("memo", True):
        # id -> distance memo of each row in flight (scratch; the kernel clears a row's slice)
        smem, warps, blocks = ctypes.c_int(0), ctypes.c_int(0), ctypes.c_int(0)
        check(lib().vl_beam_search_plan(ctypes.byref(p), ctypes.byref(smem), ctypes.byref(warps), ctypes.byref(blocks)),
              "vl_beam_search_plan")
        entries = int(config.get("memo_entries", 0))
        if entries <= 0:
            entries = 1024        # measured on 1M x 128: 8192 entries per row at E=320 (24*E) is the knee
            while entries < 24 * p.seen_cap and entries < 16384:
                entries *= 2
        slots = max(1, warps.value * blocks.value)
        memo = _memo_buffer(vectors.device, slots * entries)
        p.memo = memo.data_ptr()
        p.memo_entries = entries
        p.memo_slots = slots
    if PROFILE is not None:
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        start.record()
    check(lib().vl_beam_search(ctypes.byref(p), stream_of(vectors)), "vl_beam_search")
    if PROFILE is not None:
        end.record()
        k_none = (p.seen_cap + pvc - 1) // pvc + 1
        PROFILE.append({"start": start, "end": end, "rows": int(p.rows), "graph_w": int(p.graph_w),
                        "iterations": int(min(n_iters, k_none)), "evals": int(p.rows) * min(n_iters, k_none) * pvc * int(p.graph_w),
                        "memo": bool(p.memo), "stats": stats if stats is not STATS else None, "tag": PROFILE_TAG})


_memo_cache = {}


def _memo_buffer(device, words: int) -> Tensor:
    """A reusable int64 scratch tensor of at least `words` entries on `device`."""
    key = _lib._device_key(device)
    buf = _memo_cache.get(key)
    if buf is None or buf.numel() < words:
        buf = torch.empty(words, dtype=torch.int64, device=key)
        _memo_cache[key] = buf
    return buf


def _natural_end(flag_row: List[int], config: Dict) -> int:
    """Iteration at which the reference loop leaves, given the per-check "any head changed"."""
    k_none, n_checks, n_max = loop_bounds(config)
    ra = config["speculative_readahead"]
    for c in range(n_checks):
        if not flag_row[c]:
            return (c + 1) * ra
    return n_max


def _fused_batches(vectors, graph, queries, seed_ids, seed_dist, seed_cols, sq_len, sq_cap, config, exclude,
                   self_base, group_rows, out_ids, out_dist, out_cols, stepwise, group_row0=0, total_groups=None,
                   reduce_group=None):
    """Runs the fused search over `queries` split in batches of `group_rows` (the reference's
    host loop, ann.py:132-166) in one launch, then repairs the batches for which the
    reference's batch-wide decisions differ from the budgeted schedule: a batch whose heads
    stopped changing at an earlier check is re-run up to that iteration, a batch in which
    every row popped a MAXINT at some point goes through `stepwise(lo, hi)` (rows of this
    launch).  Returns the iteration count of every batch this launch touched.

    `group_row0`: position of query row 0 in the host loop (a launch may start inside a batch);
    `total_groups`: batches of the whole loop; `reduce_group`: a torch.distributed group whose
    ranks each run a slice of the same loop - the two batch-wide flags are then OR-ed across the
    ranks (one small all-reduce) before any decision is taken, because a batch can straddle ranks."""
    rows = queries.size(0)
    k_none, n_checks, n_max = loop_bounds(config)
    if total_groups is None:
        total_groups = (group_row0 + rows + group_rows - 1) // group_rows if rows else 0
    dev = vectors.device
    nc = max(n_checks, 1)
    ng = max(total_groups, 1)
    # one buffer for both flag arrays: one all-reduce, one read-back
    flag_buf = torch.zeros(ng * nc + ng, dtype=torch.int32, device=dev)
    flags = flag_buf[: ng * nc].view(ng, nc)
    full = flag_buf[ng * nc:]
    if rows == 0 and reduce_group is None:
        return []
    # a caller that wants to know how useful the distance memo is on this graph (generate_ann's
    # self-recall check) gets the share of candidates that had to be gathered
    counters = None
    if config.get("measure_gathered") and config.get("memo", True):
        counters = torch.zeros(24, dtype=torch.int64, device=dev)
    if rows:
        _launch_beam(vectors, graph, queries, seed_ids, seed_dist, seed_cols, sq_len, out_ids, out_dist, out_cols,
                     config, n_max, False, exclude, self_base, group_rows, flags, full, counters, group_row0)
    if reduce_group is not None:
        import torch.distributed as dist
        with nvtx_range("vl.flags_allreduce"):
            dist.all_reduce(flag_buf, op=dist.ReduceOp.MAX, group=reduce_group)
    if rows == 0:
        return []
    host = flag_buf.cpu()
    flags_h = host[: ng * nc].view(ng, nc).tolist()
    full_h = host[ng * nc:].tolist()
    if counters is not None:
        if STATS is not None:
            shared = min(STATS.numel(), counters.numel())
            STATS[:shared].add_(counters[:shared])
        c = counters.cpu().tolist()
        offered = c[7] * config["parallel_visit_count"] * graph.size(1)
        _fused_batches.last_gathered = c[1] / offered if offered else None
    counts = []
    for gi in range(group_row0 // group_rows, (group_row0 + rows - 1) // group_rows + 1):
        lo, hi = max(0, gi * group_rows - group_row0), min(rows, (gi + 1) * group_rows - group_row0)
        end = _natural_end(flags_h[gi][:n_checks], config) if n_checks else n_max
        if not full_h[gi]:
            counts.append(stepwise(lo, hi))
            continue
        counts.append(end)
        if end > k_none:
            continue
        # the reference left at check iteration `end`: redo the batch up to it; the last insert
        # is a whole-row sort so that the columns behind `length` match too
        tmp_i = torch.empty((hi - lo, sq_cap), dtype=torch.int32, device=dev)
        tmp_d = torch.empty((hi - lo, sq_cap), dtype=torch.float32, device=dev)
        f2 = torch.zeros((1, nc), dtype=torch.int32, device=dev)
        u2 = torch.zeros((1,), dtype=torch.int32, device=dev)
        _launch_beam(vectors, graph, queries[lo:hi], seed_ids[lo:hi], seed_dist[lo:hi], seed_cols, sq_len, tmp_i, tmp_d,
                     sq_cap, config, end, True, exclude[lo:hi] if exclude is not None else None,
                     self_base + lo if self_base >= 0 else -1, hi - lo, f2, u2)
        sort_pairs_(tmp_i, tmp_d, dedup=True)
        out_ids[lo:hi, :out_cols].copy_(tmp_i[:, :out_cols])
        out_dist[lo:hi, :out_cols].copy_(tmp_d[:, :out_cols])
    return counts


_fused_batches.last_gathered = None

# Above this share of gathered candidates the distance memo costs more than it saves (measured on
# 1M x 96 with 98 % gathered: build round 28 % and search 9 % faster without it; on 1M x 128 with
# 5-25 % gathered the memo is what makes the round 2.5 x faster).
MEMO_USELESS_ABOVE = 0.75


def closest_vectors_stepwise(query_vecs: Tensor, search_queue: Queue, vectors: Tensor, beams: Tensor, config: Dict,
                             exclude: Optional[Tensor] = None) -> int:
    """ann.py:37-93 step by step with the operator-level kernels (any queue shape)."""
    metric = _metric_of(config)
    (beam_count, beam_size) = beams.size()
    extra_capacity = beam_size * config["parallel_visit_count"]
    (batch_size, queue_capacity) = search_queue.size()
    visit_queue_len = config["visit_queue_factor"] * config["beam_size"]
    capacity = visit_queue_len + extra_capacity
    visit_queue = Queue(batch_size, visit_queue_len, capacity, device=vectors.device)
    visit_queue.initialize_from_queue(search_queue)
    exclude_len = config["exclude_factor"] * visit_queue_len
    seen = torch.full((batch_size, exclude_len), MAXINT, dtype=torch.int32, device=vectors.device)
    progressing = True
    count = 0
    while progressing:
        count += 1
        checking_output = (count % config["speculative_readahead"]) == 0
        neighbors_to_visit = visit_queue.pop_n_ids(config["parallel_visit_count"])
        (indexes_of_comparisons, distances_of_comparisons) = search_from_seeds(
            query_vecs, neighbors_to_visit, beams, vectors, metric=metric)
        did_something = search_queue.insert(indexes_of_comparisons, distances_of_comparisons, exclude=exclude,
                                            output_update=checking_output)
        if seen is not None:
            seen = add_new_to_seen_(seen, neighbors_to_visit)
        if seen is not None:
            visit_queue.insert(indexes_of_comparisons, distances_of_comparisons, exclude=seen)
        if checking_output:
            progressing = bool(torch.any(did_something))
    return count


@log_time
def closest_vectors(query_vecs: Tensor, search_queue: Queue, vectors: Tensor, beams: Tensor, config: Dict,
                    exclude: Optional[Tensor] = None):
    """ann.py:37-93: beam search of every row of `query_vecs` through the graph `beams`,
    starting from and updating `search_queue`.  Returns True like the reference; the number
    of loop iterations the reference would have run is kept in `closest_vectors.last_count`."""
    _lib.require_cuda(query_vecs, vectors, beams, search_queue.indices)
    assert query_vecs.is_contiguous() and vectors.is_contiguous() and beams.is_contiguous()
    (batch_size, queue_capacity) = search_queue.size()
    sq_len = search_queue.length
    force_stepwise = bool(config.get("stepwise", False))
    if force_stepwise or not _fused_shape_ok(vectors, beams.size(1), sq_len, queue_capacity, config) or batch_size == 0:
        closest_vectors.last_count = closest_vectors_stepwise(query_vecs, search_queue, vectors, beams, config, exclude)
        return True
    if exclude is not None:
        exclude = exclude.contiguous()
        assert exclude.dtype == torch.int32 and exclude.size(0) == batch_size
    in_ids, in_dist = search_queue.indices, search_queue.distances
    out_ids = torch.empty_like(in_ids)
    out_dist = torch.empty_like(in_dist)

    def stepwise(lo, hi):
        assert lo == 0 and hi == batch_size
        q = Queue(batch_size, sq_len, queue_capacity, device=vectors.device)
        q.indices.copy_(in_ids)
        q.distances.copy_(in_dist)
        n = closest_vectors_stepwise(query_vecs, q, vectors, beams, config, exclude)
        out_ids.copy_(q.indices)
        out_dist.copy_(q.distances)
        return n

    counts = _fused_batches(vectors, beams, query_vecs, in_ids, in_dist, sq_len, sq_len, queue_capacity, config,
                            exclude, -1, batch_size, out_ids, out_dist, queue_capacity, stepwise)
    search_queue.indices = out_ids
    search_queue.distances = out_dist
    closest_vectors.last_count = counts[0]
    return True


closest_vectors.last_count = 0


def search_layers(layers: List[Tensor], query_vecs: Tensor, search_queue: Queue, vectors: Tensor, config: Dict):
    """ann.py:96-106."""
    for layer in layers:
        closest_vectors(query_vecs, search_queue, vectors, layer, config, None)


def excluding_self(start, end, queue_length, device="cuda"):
    """ann.py:315-320: one exclusion list per row holding the row's own id."""
    return torch.arange(start, end, dtype=torch.int32, device=device).unsqueeze(1).contiguous()


def _gather_row_blocks(buf: Tensor, per: int, group) -> None:
    """`buf` [world * per, ...] holds rank r's rows in block r; afterwards every rank holds every
    block (one in-place all-gather)."""
    import torch.distributed as dist
    rank = dist.get_rank(group)
    mine = buf[rank * per:(rank + 1) * per]
    if buf.is_cuda:
        dist.all_gather_into_tensor(buf.view(-1), mine.reshape(-1), group=group)
    else:
        world = dist.get_world_size(group)
        dist.all_gather([buf[r * per:(r + 1) * per] for r in range(world)], mine.clone(), group=group)


def generate_ann(vectors: Tensor, config: Dict, group=None) -> Tuple[Tensor, Tensor]:
    """ann.py:109-193: circulant start graph of width W = beam_size * beam_queue_factor, then up
    to `optimization_loops` rounds of: beam-search every node from its current neighbours
    (batch by batch in the reference; all batches in one launch here, since a batch only
    reads the previous round's graph), detour prune, self-recall check.
    Departures from the reference, both where its own result is accidental: the distances
    carried into the next round and returned are those of the neighbour lists (the reference
    keeps the initial circulant distances, ann.py:172 assigns to an unused name), and a
    MAXINT neighbour yields sentinels instead of an out-of-range read.

    With `group` (a torch.distributed group whose ranks all hold the same `vectors`) the rows of
    each round are split evenly across the ranks (a batch of the host loop may straddle two
    ranks: its batch-wide flags are OR-ed across them), each rank searches and prunes its own
    rows, and the new lists are all-gathered, so every rank ends with the same graph as a
    single-GPU build.

    config["init"] == "knn_tile" (added; default "circulant" = the reference) starts from the
    lists of the tensor-core tile pass instead of the circulant graph (see knn_tile.py)."""
    _lib.require_cuda(vectors)
    (num_vecs, vec_dim) = vectors.size()
    beam_size = config["beam_size"]
    queue_length = beam_size * config["beam_queue_factor"]
    dev = vectors.device
    metric = _metric_of(config)
    remaining_capacity = queue_length * config["parallel_visit_count"]
    capacity = queue_length + remaining_capacity
    batch_size = config["batch_size"]
    fused = not config.get("stepwise", False) and _fused_shape_ok(vectors, queue_length, queue_length, capacity, config)
    world, rank = 1, 0
    if group is not None:
        import torch.distributed as dist
        world, rank = dist.get_world_size(group), dist.get_rank(group)
    per = (num_vecs + world - 1) // world              # rows per rank; the last ranks may hold fewer
    row_lo, row_hi = min(num_vecs, rank * per), min(num_vecs, (rank + 1) * per)
    n_batches = (num_vecs + batch_size - 1) // batch_size

    with nvtx_range("vl.start_graph"):
        if config.get("init", "circulant") == "knn_tile":
            from .knn_tile import knn_start_graph
            (beams, beam_distances) = knn_start_graph(vectors, queue_length, config, group=group)
        else:
            neighbor_primes = primes(queue_length, dev)
            beams = generate_circulant_beams(num_vecs, neighbor_primes)
            assert beams.dtype == torch.int32
            beam_distances = calculate_distances(vectors, beams, metric=metric)

    loops_run = 0
    memo_useful = True
    for i in range(0, config["optimization_loops"]):
        print_timestamp(f"start of cagra loop {i}")
        # padded to world * per rows so that the exchange is one equal-sized all-gather
        next_pad = torch.empty((world * per, queue_length), dtype=torch.int32, device=dev)
        next_dist_pad = torch.empty((world * per, queue_length), dtype=torch.float32, device=dev)
        next_beams = next_pad[:num_vecs]
        next_beam_distances = next_dist_pad[:num_vecs]

        def whole_batch_stepwise(glo, ghi):
            """One batch of the reference's host loop (global rows), operator by operator."""
            exclude = excluding_self(glo, ghi, queue_length, dev)
            queue = Queue(ghi - glo, queue_length, capacity, device=dev)
            queue.insert(beams.narrow(0, glo, ghi - glo), beam_distances.narrow(0, glo, ghi - glo))
            n = closest_vectors_stepwise(vectors[glo:ghi], queue, vectors, beams, config, exclude)
            next_beams.narrow(0, glo, ghi - glo).copy_(queue.indices.narrow(1, 0, queue_length))
            next_beam_distances.narrow(0, glo, ghi - glo).copy_(queue.distances.narrow(1, 0, queue_length))
            return n

        def batch_stepwise(lo, hi):
            # rows [lo, hi) of this rank's launch lie in one batch; the operator path couples the rows of
            # a batch, so the whole batch is run (a rank that holds the rest of it computes the same rows)
            g = (row_lo + lo) // batch_size
            return whole_batch_stepwise(g * batch_size, min(num_vecs, (g + 1) * batch_size))

        round_config = config
        circulant_round = i == 0 and config.get("init", "circulant") == "circulant"
        if (circulant_round or not memo_useful) and "memo" not in config and "memo_entries" not in config:
            # the circulant start graph makes candidates that hardly ever repeat within a row
            # (6 % memo hits measured): the first round runs faster without the memo; so do later
            # rounds on data where the last self-recall check gathered nearly every candidate
            round_config = dict(config, memo=False)
        global PROFILE_TAG
        with nvtx_range(f"vl.round{i}.search"):
            PROFILE_TAG = f"round{i}"
            if fused:
                _fused_batches(vectors, beams, vectors[row_lo:row_hi], beams[row_lo:row_hi],
                               beam_distances[row_lo:row_hi], queue_length, queue_length, capacity, round_config, None,
                               row_lo, batch_size, next_beams[row_lo:row_hi], next_beam_distances[row_lo:row_hi],
                               queue_length, batch_stepwise, group_row0=row_lo, total_groups=n_batches,
                               reduce_group=group if world > 1 else None)
            elif row_hi > row_lo:
                for g in range(row_lo // batch_size, (row_hi - 1) // batch_size + 1):
                    whole_batch_stepwise(g * batch_size, min(num_vecs, (g + 1) * batch_size))
        if world > 1:
            with nvtx_range(f"vl.round{i}.exchange"):
                _gather_row_blocks(next_pad, per, group)
                _gather_row_blocks(next_dist_pad, per, group)

        with nvtx_range(f"vl.round{i}.prune"):
            if config["prune"]:
                full_scan = config.get("prune_mode") == "full"
                if world > 1:
                    # a row's detour witnesses are read from the other rows as they came out of the search,
                    # so each rank prunes its own rows from the gathered lists and the results are gathered
                    out_pad = torch.empty_like(next_pad)
                    out_dist_pad = torch.empty_like(next_dist_pad)
                    prune_(next_beams, next_beam_distances, full=full_scan, rows=(row_lo, row_hi),
                           out=(out_pad[:num_vecs], out_dist_pad[:num_vecs]))
                    _gather_row_blocks(out_pad, per, group)
                    _gather_row_blocks(out_dist_pad, per, group)
                    (beams, beam_distances) = (out_pad[:num_vecs], out_dist_pad[:num_vecs])
                else:
                    (beams, beam_distances) = prune_(next_beams, next_beam_distances, full=full_scan)
            else:
                (beams, beam_distances) = (next_beams, next_beam_distances)
        loops_run += 1
        prefix = min(num_vecs, 1000)
        _fused_batches.last_gathered = None
        with nvtx_range(f"vl.round{i}.recall"):
            PROFILE_TAG = "self_recall"
            (found, recall) = ann_calculate_recall(vectors, beams.narrow_copy(1, 0, beam_size),
                                                   dict(config, measure_gathered=True), sample=vectors[:prefix])
        PROFILE_TAG = "search"
        if _fused_batches.last_gathered is not None:
            memo_useful = _fused_batches.last_gathered <= MEMO_USELESS_ABOVE
        if recall == 1.0:
            break
        print_timestamp(f"end of cagra loop {i}")
    generate_ann.last_loops = loops_run
    generate_ann.memo_useful = memo_useful
    return (beams.narrow_copy(1, 0, beam_size), beam_distances.narrow_copy(1, 0, beam_size))


generate_ann.last_loops = 0
generate_ann.memo_useful = True


def initial_queue(vectors: Tensor, config: Dict):
    """ann.py:196-208: circulant seeds among the sample itself."""
    queue_size = config["recall_search_queue_factor"] * config["beam_size"]
    (batch_size, _) = vectors.size()
    extra_capacity = max(queue_size, config["parallel_visit_count"] * config["beam_size"])
    queue = Queue(batch_size, queue_size, queue_size + extra_capacity, device=vectors.device)
    p = primes(queue_size, vectors.device)
    initial_queue_indices = generate_circulant_beams(batch_size, p)
    d = calculate_distances(vectors, initial_queue_indices, metric=_metric_of(config))
    queue.insert(initial_queue_indices, d)
    return queue


def query_distances(query_vectors: Tensor, vectors: Tensor, ids: Tensor, metric="cosine") -> Tensor:
    """Distances of query b to vectors[ids[b, j]] (the role of query_cosine_distances,
    ann.py:211-214, whose broadcast only works for one query row).  Taken with the same
    summation order and clamp as every other distance, so a seed that comes back as a
    candidate carries the same bits; the reference's torch-order sum differs from this by
    at most an ulp or two."""
    return calculate_distances(vectors, ids, metric=metric, queries=query_vectors)


def initial_search_queue(vectors: Tensor, query_vectors: Tensor, config: Dict, first_row: int = 0):
    """ann.py:217-232: circulant seeds (b + p_j) mod N for query row b; the queue starts as the
    Q = recall_search_queue_factor * beam_size seeds ordered by distance.
    config["search_seed_factor"] (added, default 1 = the reference) scans that many times Q
    seeds and keeps the best Q: on data with well separated clusters the graph has no links
    between clusters, so a search only finds a query's neighbourhood if a seed lands in it."""
    queue_size = config["recall_search_queue_factor"] * config["beam_size"]
    (batch_size, _) = query_vectors.size()
    extra_capacity = max(queue_size, config["parallel_visit_count"] * config["beam_size"])
    queue = Queue(batch_size, queue_size, queue_size + extra_capacity, device=vectors.device)
    seed_count = queue_size * max(1, int(config.get("search_seed_factor", 1)))
    p = primes(seed_count, vectors.device)
    (vector_count, _) = vectors.size()
    initial_queue_indices = generate_queue_circulants(batch_size, vector_count, p, first_row)
    d = query_distances(query_vectors, vectors, initial_queue_indices, _metric_of(config))
    if seed_count <= extra_capacity:
        queue.insert(initial_queue_indices, d)
    else:
        # same result as inserting the seeds piecewise: the best Q distinct (distance, id) pairs
        sort_pairs_(initial_queue_indices, d, dedup=True)
        queue.indices.narrow(1, 0, queue_size).copy_(initial_queue_indices.narrow(1, 0, queue_size))
        queue.distances.narrow(1, 0, queue_size).copy_(d.narrow(1, 0, queue_size))
    return queue


def ann_calculate_recall(vectors: Tensor, beams: Tensor, config: Dict, sample: Optional[Tensor] = None):
    """ann.py:235-259: self-recall - rows of the sample whose best hit is themselves."""
    if sample is None:
        sample = vectors
    (sample_size, _) = sample.size()
    queue = initial_queue(sample.contiguous(), config)
    closest_vectors(sample.contiguous(), queue, vectors, beams.contiguous(), config)
    expected = torch.arange(sample_size, device=vectors.device)
    actual = queue.indices.t()[0]
    found = (expected == actual).sum().item()
    print_timestamp(f"found: {found} / {sample_size}")
    print_timestamp(f"recall: {found / sample_size}")
    return (found, found / sample_size)


def hnsw_calculate_recall(vectors: Tensor, hnsw: List[Tensor], config: Dict, sample: Optional[Tensor] = None):
    """ann.py:262-284: self-recall through a list of layer graphs, coarsest first."""
    if sample is None:
        sample = vectors
    (sample_size, _) = sample.size()
    queue = initial_queue(sample.contiguous(), config)
    search_layers([layer.contiguous() for layer in hnsw], sample.contiguous(), queue, vectors, config)
    expected = torch.arange(sample_size, device=vectors.device)
    actual = queue.indices.t()[0]
    found = (expected == actual).sum().item()
    print_timestamp(f"found: {found} / {sample_size}")
    print_timestamp(f"recall: {found / sample_size}")
    return (found, found / sample_size)


def ann_recall_test(vectors: Tensor, config: Dict):
    """ann.py:287-293."""
    (beams, _) = generate_ann(vectors, config)
    prefix = min(vectors.size()[0], 10_000)
    return ann_calculate_recall(vectors, beams, config, sample=vectors[:prefix])


def grid_search(vectors: Optional[Tensor] = None, grid: Optional[Dict[str, list]] = None, base: Optional[Dict] = None,
                log_dir: str = "./grid-log") -> List[Dict]:
    """ann.py:323-353: one build + self-recall per point of a parameter grid, one JSON log per
    point in `log_dir`.  Defaults are the reference's experiment: 1,000,000 random unit vectors of
    1536 dimensions; prune x beam_size {24, 32, 46} x parallel_visit_count {1, 4} x
    optimization_loops {1, 2} x visit_queue_factor {3, 4}.  (The reference's version calls an
    undefined `main`; this one runs.)"""
    import itertools
    from .utils import generate_random_vectors
    config = {"exclude_factor": 5, "batch_size": 10_000, "beam_queue_factor": 3, "recall_search_queue_factor": 6}
    config.update(base or {})
    if vectors is None:
        vectors = generate_random_vectors(number_of_vectors=1_000_000, dimensions=1536)
    if grid is None:
        grid = {"prune": [True, False], "beam_size": [24, 32, 46], "parallel_visit_count": [1, 4],
                "optimization_loops": [1, 2], "visit_queue_factor": [3, 4]}
    os.makedirs(log_dir, exist_ok=True)
    results = []
    names = list(grid)
    for point in itertools.product(*(grid[k] for k in names)):
        kwargs = dict(config, **dict(zip(names, point)))
        ann = ANN(vectors=vectors, **kwargs)
        log = ann.dump_logs()
        log["type"] = "cagra"
        with open(os.path.join(log_dir, f"experiment-{time.time()}.log"), "w") as out:
            json.dump(log, out)
        results.append(log)
    return results


VERBOSE = bool(os.getenv("VECTORLINK_VERBOSE"))


def print_timestamp(msg):
    """ann.py:297-298 prints unconditionally; here only when VECTORLINK_VERBOSE is set."""
    if VERBOSE:
        print(msg)


class ANN:
    """ann.py:356-489.  `ANN(vectors=...)` builds the graph; `.beams` int32 [N, beam_size],
    `.distances` fp32 [N, beam_size], `.search(query)` returns the search `Queue`.
    Added keywords: metric ("cosine" - the reference's distance on unit vectors - or "l2") and
    search_seed_factor (how many times Q seeds `.search` scans for its starting queue; 1 = the
    reference), prune_mode ("first" = the reference's detour test against y's first neighbour only,
    "full" = against all of them), symmetrize (add reverse edges after the build; off = the reference),
    init ("circulant" = the reference's start graph; "knn_tile" = exact-reranked proposals of a tensor-core
    tile pass, see knn_tile.py), search_entry_sample (0 = the reference's circulant seeds; S > 0: `.search` starts
    every query from its best 64 of S evenly spaced rows, scored on the tensor cores, see `_entry_seeds`) and group (a torch.distributed group whose ranks all pass the same vectors: the
    build's rows are split across them, see generate_ann)."""

    def __init__(self, vectors: Tensor, prune: bool = True, beam_size: int = 24, parallel_visit_count: int = 4,
                 beam_queue_factor: int = 3, visit_queue_factor: int = 3, exclude_factor: int = 5,
                 optimization_loops: int = 3, batch_size: int = 10_000, recall_search_queue_factor: int = 3,
                 speculative_readahead: int = 5, beams: Optional[Tensor] = None, distances: Optional[Tensor] = None,
                 metric: str = "cosine", search_seed_factor: int = 1, group=None, symmetrize: bool = False,
                 prune_mode: str = "first", init: str = "circulant", search_entry_sample: int = 0):
        (count, dim) = vectors.size()
        assert vectors.dtype == torch.float32
        _lib.require_cuda(vectors)
        metric_code(metric)
        self.configuration: Dict = {
            "prune": prune,
            "beam_size": beam_size,
            "parallel_visit_count": parallel_visit_count,
            "beam_queue_factor": beam_queue_factor,
            "visit_queue_factor": visit_queue_factor,
            "exclude_factor": exclude_factor,
            "optimization_loops": optimization_loops,
            "batch_size": batch_size,
            "recall_search_queue_factor": recall_search_queue_factor,
            "speculative_readahead": speculative_readahead,
        }
        if metric != "cosine":
            self.configuration["metric"] = metric
        if search_seed_factor != 1:
            self.configuration["search_seed_factor"] = search_seed_factor
        assert prune_mode in ("first", "full")
        if prune_mode != "first":
            self.configuration["prune_mode"] = prune_mode
        assert init in ("circulant", "knn_tile")
        if init != "circulant":
            self.configuration["init"] = init
        if search_entry_sample:
            self.configuration["search_entry_sample"] = int(search_entry_sample)
        self._entry = None
        self.vectors = vectors.contiguous()
        wall_start = time.time()
        if beams is not None:
            self.beams = beams
            if distances is None:
                self.distances = calculate_distances(self.vectors, self.beams, metric=metric)
            else:
                self.distances = distances
        else:
            (self.beams, self.distances) = generate_ann(self.vectors, self.configuration, group=group)
            if not generate_ann.memo_useful and "memo" not in self.configuration:
                # the last self-recall check over this graph gathered nearly every candidate:
                # searches run faster without the distance memo (same results either way)
                self.configuration["memo"] = False
        if symmetrize:
            from .kernels import symmetrize as _symmetrize
            (self.beams, self.distances) = _symmetrize(self.vectors, self.beams.contiguous(), self.distances.contiguous(),
                                                       metric=metric)
        torch.cuda.synchronize(self.vectors.device)
        wall_end = time.time()
        total_time: float = wall_end - wall_start
        self.log = self.configuration.copy()
        self.log["total_time"] = total_time
        self.log["vector_count"] = count
        self.log["vector_dimension"] = dim

    @classmethod
    def load_from_dataframe(cls, dataframe, device="cuda", **kwargs) -> "ANN":
        """ann.py:408-454: a saved index back from Arrow data with the columns `vector_id`,
        `embedding`, `beams` and optionally `distances`.  Takes a `pyarrow.Table` (or a DataFusion
        DataFrame where that package is installed); rows are ordered by `vector_id`."""
        import pyarrow as pa
        import pyarrow.compute as pc
        from .datafusion import dataframe_to_tensor
        table = dataframe if isinstance(dataframe, pa.Table) else dataframe.to_arrow_table()
        names = table.schema.names
        assert "embedding" in names and "beams" in names
        if "vector_id" in names:
            table = table.take(pc.sort_indices(table, sort_keys=[("vector_id", "ascending")]))
        count = table.num_rows

        def width(name):
            ty = table.schema.field(name).type
            size = getattr(ty, "list_size", None)
            return size if size is not None else len(table.column(name)[0])

        vectors_tensor = torch.empty((count, width("embedding")), dtype=torch.float32, device=device)
        dataframe_to_tensor(table.column("embedding"), vectors_tensor)
        beam_size = width("beams")
        beams_tensor = torch.empty((count, beam_size), dtype=torch.int32, device=device)
        dataframe_to_tensor(table.column("beams"), beams_tensor)
        distances_tensor = None
        if "distances" in names:
            distances_tensor = torch.empty((count, beam_size), dtype=torch.float32, device=device)
            dataframe_to_tensor(table.column("distances"), distances_tensor)
        return ANN(vectors_tensor, beam_size=beam_size, beams=beams_tensor, distances=distances_tensor, **kwargs)

    def to_arrow(self):
        """The index as a `pyarrow.Table` in the column layout `load_from_dataframe` reads."""
        import pyarrow as pa
        from .datafusion import tensor_to_arrow
        count = self.vectors.size(0)
        return pa.table({"vector_id": pa.array(range(count), type=pa.int32()),
                         "embedding": tensor_to_arrow(self.vectors), "beams": tensor_to_arrow(self.beams),
                         "distances": tensor_to_arrow(self.distances)})

    def recall(self, sample_size: int = 1000) -> Tuple[float, float]:
        """ann.py:456-464."""
        (count, _) = self.vectors.size()
        sample_size = min(sample_size, count)
        sample = self.vectors[0:sample_size]
        return ann_calculate_recall(self.vectors, self.beams, self.configuration, sample)

    def clusters(self) -> Queue:
        """ann.py:466-467 is an empty stub; its README says it "returns all search queues":
        the search queue of every indexed vector, seeded like the recall check
        (initial_queue) and searched through the graph."""
        queue = initial_queue(self.vectors, self.configuration)
        closest_vectors(self.vectors, queue, self.vectors, self.beams, self.configuration)
        return queue

    def cluster_labels(self, threshold: float, queues: Optional[Queue] = None) -> Tensor:
        """Clusters as connected components (added; the reference stops at the `clusters` stub):
        int32 [N] labels, the smallest vector id of each component of the graph whose links are
        the neighbour pairs at distance <= threshold.  Links come from the graph's own rows
        (`.beams` / `.distances`), or from the heads of `queues` as returned by `clusters()`."""
        if queues is None:
            return connected_components(self.beams, self.distances, threshold)
        return connected_components(queues.indices[:, :queues.length], queues.distances[:, :queues.length], threshold)

    def search(self, query: Tensor, first_row: int = 0) -> Queue:
        """ann.py:469-477: `query` fp32 [B, dim] -> Queue with `.indices` int32 and `.distances`
        fp32 of shape [B, Q + max(Q, pvc*beam_size)], Q = recall_search_queue_factor*beam_size
        = `.length`; rows ascending by distance, ids unique, MAXINT/MAXFLOAT padding.
        `first_row` (added): index of query row 0 in the batch it was cut from (the seeds of a
        row depend on its index)."""
        assert query.dtype == torch.float32
        query = query.contiguous()
        config = self.configuration
        queue_size = config["recall_search_queue_factor"] * config["beam_size"]
        extra_capacity = max(queue_size, config["parallel_visit_count"] * config["beam_size"])
        seed_count = queue_size * max(1, int(config.get("search_seed_factor", 1)))
        beams = self.beams.contiguous()
        entry_sample = int(config.get("search_entry_sample", 0))
        fused_ok = (query.size(0) > 0 and not config.get("stepwise", False)
                    and _fused_shape_ok(self.vectors, beams.size(1), queue_size, queue_size + extra_capacity, config))
        if entry_sample > 0 and query.size(0) > 0:
            # entry points from the tensor-core pass instead of circulant seeds
            seeds = self._entry_seeds(query)
            d = query_distances(query, self.vectors, seeds, _metric_of(config))

            def seeded_queue():
                q = Queue(query.size(0), queue_size, queue_size + extra_capacity, device=self.vectors.device)
                if seeds.size(1) <= extra_capacity:
                    q.insert(seeds, d)
                else:       # the best Q distinct (distance, id) pairs of all seeds, as inserting them piecewise would leave
                    (si, sd) = (seeds.clone(), d.clone())
                    sort_pairs_(si, sd, dedup=True)
                    q.indices.narrow(1, 0, queue_size).copy_(si.narrow(1, 0, queue_size))
                    q.distances.narrow(1, 0, queue_size).copy_(sd.narrow(1, 0, queue_size))
                return q

            if not fused_ok:
                search_queue = seeded_queue()
                closest_vectors(query, search_queue, self.vectors, beams, config, None)
                return search_queue
            seed_count = seeds.size(1)
        if (entry_sample > 0 or seed_count > extra_capacity) and fused_ok:
            # many seeds: the fused kernel starts every row from an empty queue and merges the
            # seeds itself, so the best-Q selection needs no separate sort
            _lib.require_cuda(query, self.vectors, beams)
            dev = self.vectors.device
            if entry_sample <= 0:
                seeds = generate_queue_circulants(query.size(0), self.vectors.size(0), primes(seed_count, dev), first_row)
                d = query_distances(query, self.vectors, seeds, _metric_of(config))
            queue = Queue(query.size(0), queue_size, queue_size + extra_capacity, device=dev)

            def stepwise(lo, hi):
                q = seeded_queue() if entry_sample > 0 else initial_search_queue(self.vectors, query, config, first_row)
                n = closest_vectors_stepwise(query, q, self.vectors, beams, config, None)
                queue.indices.copy_(q.indices)
                queue.distances.copy_(q.distances)
                return n

            counts = _fused_batches(self.vectors, beams, query, seeds, d, seed_count, queue_size,
                                    queue_size + extra_capacity, config, None, -1, query.size(0), queue.indices,
                                    queue.distances, queue_size + extra_capacity, stepwise)
            closest_vectors.last_count = counts[0]
            return queue
        search_queue = initial_search_queue(self.vectors, query, config, first_row)
        closest_vectors(query, search_queue, self.vectors, beams, config, None)
        return search_queue

    def _entry_seeds(self, query: Tensor) -> Tensor:
        """int32 [B, 64]: for every query the 64 best-scoring of S = config["search_entry_sample"] evenly
        spaced rows of the index (bf16 inner products on the tensor cores, knn_tile.py), as global ids,
        MAXINT-padded.  Added: the reference seeds a search with Q rows at fixed offsets from the query's
        batch position (utils.py:26-32), which finds the query's neighbourhood only if one of them happens
        to lie near it; on clustered data most queries then never reach their cluster.  The seeds only pick
        where the search starts: their distances are taken exactly afterwards, like any other seed's."""
        from . import knn_tile
        (n, _) = self.vectors.size()
        sample = min(n, int(self.configuration["search_entry_sample"]))
        metric = _metric_of(self.configuration)
        b = query.size(0)
        if self._entry is None or self._entry["sample"] != sample or self._entry["both"].size(0) < sample + b:
            ids = (torch.arange(sample, device=self.vectors.device, dtype=torch.int64) * n // sample).to(torch.int32)
            rows_bf16, norms = knn_tile.prepare(self.vectors[ids.long()].contiguous(), want_norms=metric_code(metric) == 1)
            # one matrix for both sides of the tile pass: the sample's rows, then room for a batch of queries
            room = max(b, 16_384)
            both = torch.zeros((sample + room, rows_bf16.size(1)), dtype=rows_bf16.dtype, device=rows_bf16.device)
            both[:sample] = rows_bf16
            if norms is not None:
                norms = torch.cat([norms, torch.zeros(room, dtype=torch.float32, device=norms.device)])
            self._entry = {"sample": sample, "ids": ids, "both": both, "norms": norms}
        e = self._entry
        knn_tile.prepare(query, want_norms=False, out=e["both"][sample:sample + b])
        # (one segment: more segments would occupy more SMs on a small batch, but their extra picks cost more
        # in exact distances and sorting than the pass gains - measured)
        picks = knn_tile.proposals(e["both"], e["norms"], (sample, sample + b), (0, sample), 1)   # indices into the sample
        valid = picks != MAXINT
        return torch.where(valid, e["ids"][picks.clamp(max=sample - 1).long()], picks).contiguous()

    def dump_logs(self) -> Dict:
        """ann.py:479-489."""
        log = self.log.copy()
        log["closest_vectors_batch_time"] = _log.CLOSEST_VECTORS_BATCH_TIME
        try:
            log["gpu_arch"] = subprocess.check_output(["nvidia-smi", "-L"]).decode("utf-8").strip()
        except Exception:
            log["gpu_arch"] = torch.cuda.get_device_name(self.vectors.device)
        try:
            log["commit"] = subprocess.check_output(["git", "rev-parse", "--verify", "HEAD"]).decode("utf-8").strip()
        except Exception:
            log["commit"] = None
        (_, recall) = self.recall()
        log["recall"] = recall
        return log

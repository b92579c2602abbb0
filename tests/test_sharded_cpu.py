"""The cross-shard exchange of the sharded build on two CPU ranks over gloo.

The GPU kernels are replaced by exact stand-ins (brute-force search inside a shard, a torch
sort for the merge), so the test checks the choreography: what is gathered, which slice each
owner keeps, padding of uneven shards - against a brute-force kNN over the whole set."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, total, dim, degree, chunk, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from vectorlink_gpu.sharded import merge_pass, partition_rows, shard_offsets
    from vectorlink_gpu.constants import MAXINT
    g = torch.Generator().manual_seed(0)
    full = torch.nn.functional.normalize(torch.randn(total, dim, generator=g), dim=1)
    lo, hi = partition_rows(total, world)[rank]
    local = full[lo:hi].contiguous()
    offsets = shard_offsets(local.size(0))
    assert offsets[rank] == lo and offsets[-1] == total

    def knn(rows, base_rows, exclude_base=None):
        d = (1 - rows @ base_rows.t()) / 2
        if exclude_base is not None:
            idx = torch.arange(rows.size(0))
            d[idx, idx + exclude_base] = float("inf")
        dd, ii = torch.topk(d, degree, dim=1, largest=False)
        return ii.int(), dd

    li, ld = knn(local, local, exclude_base=0)            # exact local graph, self excluded
    li = li + lo

    def search_fn(rows):
        ii, dd = knn(rows, local)
        return ii + lo, dd

    def merge_fn(ids, d, keep):
        order = torch.argsort(d, dim=1, stable=True)
        return torch.gather(ids, 1, order)[:, :keep], torch.gather(d, 1, order)[:, :keep]

    mi, md = merge_pass(local, li, ld, offsets, degree, search_fn, merge_fn, chunk_rows=chunk)
    torch.save((mi, md), os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("total,chunk", [(101, 16), (64, 1000)])
def test_merge_pass_yields_the_global_neighbours(tmp_path, total, chunk):
    world, dim, degree = 2, 8, 5
    port = _free_port()
    mp.spawn(_worker, args=(world, port, total, dim, degree, chunk, str(tmp_path)), nprocs=world, join=True)
    g = torch.Generator().manual_seed(0)
    full = torch.nn.functional.normalize(torch.randn(total, dim, generator=g), dim=1)
    d = (1 - full @ full.t()) / 2
    d.fill_diagonal_(float("inf"))
    want_d, want_i = torch.topk(d, degree, dim=1, largest=False)
    got = [torch.load(os.path.join(str(tmp_path), f"r{r}.pt")) for r in range(world)]
    got_i = torch.cat([g[0] for g in got], 0)
    got_d = torch.cat([g[1] for g in got], 0)
    assert got_i.shape == (total, degree)
    assert torch.allclose(got_d, want_d, atol=1e-6)
    assert (got_i.long() == want_i).float().mean() > 0.99     # equal up to exact distance ties


def test_partition_covers_every_row_once():
    from vectorlink_gpu.sharded import partition_rows
    for total in (0, 1, 7, 8, 1000003):
        for world in (1, 2, 3, 8):
            b = partition_rows(total, world)
            assert b[0][0] == 0 and b[-1][1] == total
            assert all(b[i][1] == b[i + 1][0] for i in range(world - 1))
            sizes = [h - l for l, h in b]
            assert max(sizes) - min(sizes) <= 1


def _rows_worker(rank, world, port, total, batch, out_dir):
    """generate_ann's row-split rounds on CPU ranks: the device operators are replaced by
    oracle-backed stand-ins, everything else (row ranges, whole-batch handling of a batch that
    straddles two ranks, padded all-gathers, pruning of the own rows only) is the product's code."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from vectorlink_gpu import _lib, ann
    oracle.set_num_threads(1)

    class HostQueue:
        def __init__(self, num_queues, queue_length, capacity, device=None):
            self.q = oracle.Queue(num_queues, queue_length, capacity)
            self.length = queue_length

        indices = property(lambda self: torch.from_numpy(self.q.indices))
        distances = property(lambda self: torch.from_numpy(self.q.distances))

        def insert(self, ids, dd, exclude=None, output_update=False):
            return self.q.insert(ids.numpy(), dd.numpy(), None if exclude is None else exclude.numpy(), output_update)

    def stepwise(query_vecs, queue, vectors, beams, config, exclude=None):
        return oracle.closest_vectors(query_vecs.numpy(), queue.q, vectors.numpy(), beams.contiguous().numpy(), config,
                                      None if exclude is None else exclude.numpy())

    def prune(beams, distances, full=False, rows=None, out=None):
        pb, pd = oracle.prune_(beams.numpy(), distances.numpy())
        if out is None:
            return torch.from_numpy(pb), torch.from_numpy(pd)
        lo, hi = rows
        out[0][lo:hi] = torch.from_numpy(pb[lo:hi])
        out[1][lo:hi] = torch.from_numpy(pd[lo:hi])
        return out

    def recall(vectors, beams, config, sample=None):
        found = oracle.self_recall(vectors.numpy(), beams.numpy(), config, sample.size(0))
        return found, found / sample.size(0)

    _lib.require_cuda = lambda *a: None
    ann.Queue = HostQueue
    ann.closest_vectors_stepwise = stepwise
    ann.prune_ = prune
    ann.ann_calculate_recall = recall
    ann.calculate_distances = lambda v, b, metric="cosine": torch.from_numpy(oracle.calculate_distances(v.numpy(), b.numpy()))
    ann.excluding_self = lambda start, end, ql, device="cpu": torch.arange(start, end, dtype=torch.int32).unsqueeze(1)
    ann.primes = lambda size, device="cpu": torch.from_numpy(oracle.primes_table()[:size].copy())

    g = torch.Generator().manual_seed(3)
    vectors = torch.nn.functional.normalize(torch.randn(total, 12, generator=g), dim=1).contiguous()
    cfg = oracle.make_config(beam_size=5, batch_size=batch, optimization_loops=2)
    beams, dd = ann.generate_ann(vectors, dict(cfg, stepwise=True), group=dist.group.WORLD)
    want_b, want_d, loops, _ = oracle.generate_ann(vectors.numpy(), cfg)
    assert ann.generate_ann.last_loops == loops
    assert np.array_equal(beams.numpy(), want_b) and np.array_equal(dd.numpy(), want_d)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,total,batch", [(2, 131, 30), (3, 100, 7), (2, 90, 1000)])
def test_row_split_build_rounds_equal_the_single_process_build(tmp_path, world, total, batch):
    """Uneven row ranges, batches that straddle two ranks, a batch larger than the set."""
    mp.spawn(_rows_worker, args=(world, _free_port(), total, batch, str(tmp_path)), nprocs=world, join=True)


def _host_launch_beam(oracle, MAXINT, MAXFLOAT):
    """A CPU stand-in with the fused kernel's contract (include/vlgpu.h, vl_beam_search): every row runs the
    budgeted loop on its own - `seen` takes pvc ids per iteration whatever the other rows do - and reports the
    two batch-wide facts through the flag arrays.  Built from the oracle's operators, one row at a time."""
    def launch(vectors, graph, queries, seed_ids, seed_dist, seed_cols, sq_len, out_ids, out_dist, out_cols, config,
               n_iters, dump_last, exclude, self_base, group_rows, flags, full, stats=None, group_row0=0):
        launch.calls.append((int(queries.size(0)), bool(dump_last), int(group_row0)))
        v, g = vectors.numpy(), graph.contiguous().numpy()
        pvc, ra = config["parallel_visit_count"], config["speculative_readahead"]
        vq_len = config["visit_queue_factor"] * config["beam_size"]
        e_cap = config["exclude_factor"] * vq_len
        w = g.shape[1]
        m = pvc * w
        k_none = (e_cap + pvc - 1) // pvc + 1
        for r in range(queries.size(0)):
            q = queries[r:r + 1].numpy()
            group = (group_row0 + r) // group_rows if group_rows > 0 else 0
            sq = oracle.Queue(1, sq_len, sq_len + max(m, seed_cols))
            sq.insert(seed_ids[r:r + 1, :seed_cols].numpy(), seed_dist[r:r + 1, :seed_cols].numpy())
            vq = oracle.Queue(1, vq_len, vq_len + m)
            vq.initialize_from_queue(sq)
            banned = [int(self_base + r)] if self_base >= 0 else []
            if exclude is not None:
                for x in exclude[r].tolist():
                    if x == MAXINT:
                        break
                    banned.append(x)
            ex = np.array([banned + [MAXINT]], dtype=np.int32)
            seen, always_full, dumped = [], True, False
            for k in range(1, min(n_iters, k_none) + 1):
                first = (k - 1) * pvc
                ncopy = max(0, min(pvc, e_cap - first))
                visit = vq.pop_n_ids(pvc)
                ci, cd = oracle.search_from_seeds(q, visit, g, v)
                if dump_last and k == n_iters:
                    hit = np.isin(ci[0], banned)
                    out_ids[r, :sq_len] = torch.from_numpy(sq.indices[0, :sq_len])
                    out_dist[r, :sq_len] = torch.from_numpy(sq.distances[0, :sq_len])
                    out_ids[r, sq_len:sq_len + m] = torch.from_numpy(np.where(hit, MAXINT, ci[0]).astype(np.int32))
                    out_dist[r, sq_len:sq_len + m] = torch.from_numpy(np.where(hit, np.float32(MAXFLOAT), cd[0]).astype(np.float32))
                    out_ids[r, sq_len + m:out_cols] = MAXINT
                    out_dist[r, sq_len + m:out_cols] = MAXFLOAT
                    dumped = True
                    break
                changed = sq.insert(ci, cd, exclude=ex, output_update=True)
                if changed.any() and k % ra == 0 and k // ra - 1 < flags.size(1):
                    flags[group, k // ra - 1] = 1
                if ncopy > 0:
                    for x in visit[0, :ncopy].tolist():
                        if x == MAXINT:
                            always_full = False
                        else:
                            seen.append(x)
                    vq.insert(ci, cd, exclude=np.array([seen + [MAXINT]], dtype=np.int32))
            if not dumped:
                out_ids[r, :sq_len] = torch.from_numpy(sq.indices[0, :sq_len])
                out_dist[r, :sq_len] = torch.from_numpy(sq.distances[0, :sq_len])
                out_ids[r, sq_len:out_cols] = MAXINT
                out_dist[r, sq_len:out_cols] = MAXFLOAT
            if always_full:
                full[group] = 1
    launch.calls = []
    return launch


def _fused_rows_worker(rank, world, port, total, batch, out_dir):
    """generate_ann's FUSED row-split rounds on CPU ranks: one launch per rank that may start inside a batch
    (group_row0), the batch-wide flags OR-ed across ranks, the repair of batches that stop early, the hand-over
    of dry batches to the operator path - with the kernel replaced by the host stand-in above."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from vectorlink_gpu import _lib, ann
    from vectorlink_gpu.constants import MAXFLOAT, MAXINT
    oracle.set_num_threads(1)          # thousands of one-row calls: thread teams would only get in each other's way

    class HostQueue:
        def __init__(self, num_queues, queue_length, capacity, device=None):
            self.q = oracle.Queue(num_queues, queue_length, capacity)
            self.length = queue_length

        indices = property(lambda self: torch.from_numpy(self.q.indices))
        distances = property(lambda self: torch.from_numpy(self.q.distances))

        def insert(self, ids, dd, exclude=None, output_update=False):
            return self.q.insert(ids.numpy(), dd.numpy(), None if exclude is None else exclude.numpy(), output_update)

    def stepwise(query_vecs, queue, vectors, beams, config, exclude=None):
        return oracle.closest_vectors(query_vecs.numpy(), queue.q, vectors.numpy(), beams.contiguous().numpy(), config,
                                      None if exclude is None else exclude.numpy())

    def prune(beams, distances, full=False, rows=None, out=None):
        pb, pd = oracle.prune_(beams.numpy(), distances.numpy())
        if out is None:
            return torch.from_numpy(pb), torch.from_numpy(pd)
        lo, hi = rows
        out[0][lo:hi] = torch.from_numpy(pb[lo:hi])
        out[1][lo:hi] = torch.from_numpy(pd[lo:hi])
        return out

    def sort_pairs(ids, dd, dedup):
        si, sd = oracle.queue_sort(ids.numpy(), dd.numpy())
        ids.copy_(torch.from_numpy(si))
        dd.copy_(torch.from_numpy(sd))

    def recall(vectors, beams, config, sample=None):
        found = oracle.self_recall(vectors.numpy(), beams.numpy(), config, sample.size(0))
        return found, found / sample.size(0)

    _lib.require_cuda = lambda *a: None
    _lib.status_word = lambda device: torch.zeros(1, dtype=torch.int32)
    ann.Queue = HostQueue
    ann.closest_vectors_stepwise = stepwise
    ann.prune_ = prune
    ann.sort_pairs_ = sort_pairs
    ann.ann_calculate_recall = recall
    ann._launch_beam = _host_launch_beam(oracle, MAXINT, MAXFLOAT)
    ann.calculate_distances = lambda v, b, metric="cosine": torch.from_numpy(oracle.calculate_distances(v.numpy(), b.numpy()))
    ann.excluding_self = lambda start, end, ql, device="cpu": torch.arange(start, end, dtype=torch.int32).unsqueeze(1)
    ann.primes = lambda size, device="cpu": torch.from_numpy(oracle.primes_table()[:size].copy())

    g = torch.Generator().manual_seed(5)
    vectors = torch.nn.functional.normalize(torch.randn(total, 24, generator=g), dim=1).contiguous()
    cfg = oracle.make_config(beam_size=6, batch_size=batch, optimization_loops=2)
    beams, dd = ann.generate_ann(vectors, dict(cfg), group=dist.group.WORLD)
    want_b, want_d, loops, _ = oracle.generate_ann(vectors.numpy(), cfg)
    assert ann.generate_ann.last_loops == loops
    assert np.array_equal(beams.numpy(), want_b), "row-split fused rounds differ from the single-process build"
    assert np.array_equal(dd.numpy(), want_d)
    calls = ann._launch_beam.calls
    with open(os.path.join(out_dir, f"calls{rank}.txt"), "w") as f:
        f.write(f"{sum(1 for c in calls if c[1])} {sum(1 for c in calls if not c[1] and c[2] % batch != 0)}")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,total,batch", [(2, 230, 3), (3, 200, 7)])
def test_row_split_fused_rounds_equal_the_single_process_build(tmp_path, world, total, batch):
    """Small batches stop early (the reference's batch-wide check) and straddle the ranks' row ranges."""
    mp.spawn(_fused_rows_worker, args=(world, _free_port(), total, batch, str(tmp_path)), nprocs=world, join=True)
    repaired = straddling = 0
    for r in range(world):
        a, b = open(os.path.join(str(tmp_path), f"calls{r}.txt")).read().split()
        repaired += int(a)
        straddling += int(b)
    assert repaired > 0, "no batch stopped early: the repair path did not run"
    assert straddling > 0, "no launch started inside a batch"

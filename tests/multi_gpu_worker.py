"""Worker of tests/test_gpu_multi.py: one rank of a 2-GPU run (launched with torchrun)."""
import os
import sys

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
for p in (ROOT, os.path.join(ROOT, "vectorlink-gpu_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import numpy as np
import torch
import torch.distributed as dist


def _lib_status_clear(dev):
    from vectorlink_gpu import _lib
    return _lib.read_status(dev) == 0


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from vectorlink_gpu.sharded import ShardedANN, partition_rows
    g = dict(np.load(os.path.join(ROOT, "tests", "golden", "c1_host.npz")))
    kw = {k[4:]: int(v) for k, v in g.items() if k.startswith("cfg_")}
    kw["batch_size"] = 500                                   # several batches per rank
    vectors = torch.from_numpy(g["vectors"]).to(dev)
    queries = torch.from_numpy(g["queries"]).to(dev)
    lo, hi = partition_rows(vectors.size(0), world)[rank]

    # mode "rows": the graph of the whole set, identical to a single-GPU build (the fixture)
    rows = ShardedANN(vectors[lo:hi].contiguous(), mode="rows", **kw)
    assert np.array_equal(rows.index.beams.cpu().numpy(), g["beams"]), "row-parallel graph differs from the single-GPU graph"
    assert np.array_equal(rows.index.distances.cpu().numpy(), g["distances"])
    ids, dd = rows.search(queries)
    assert np.array_equal(ids.cpu().numpy(), g["search_tree_ids"]), "data-parallel search differs"
    assert np.array_equal(dd.cpu().numpy(), g["search_tree_dist"])

    # three rounds whose batches straddle the two ranks' row ranges (1800 rows, batches of 500):
    # the reference's host code with its two accidental spots repaired (tests/golden/make_golden.py)
    m = dict(np.load(os.path.join(ROOT, "tests", "golden", "multi_host.npz")))
    mkw = {k[4:]: int(v) for k, v in m.items() if k.startswith("cfg_")}
    mv = torch.from_numpy(m["vectors"]).to(dev)
    mlo, mhi = partition_rows(mv.size(0), world)[rank]
    three = ShardedANN(mv[mlo:mhi].contiguous(), mode="rows", **mkw)
    assert np.array_equal(three.index.beams.cpu().numpy(), m["beams"]), "three-round row-parallel graph differs"
    assert np.array_equal(three.index.distances.cpu().numpy(), m["distances"])

    # batches of a few rows stop early inside the build (the reference's batch-wide check); a batch
    # that straddles the ranks must take the same decision on both: against the CPU oracle
    import oracle
    rng = np.random.default_rng(123)
    tv = rng.standard_normal((250, 24)).astype(np.float32)
    tv /= np.linalg.norm(tv, axis=1, keepdims=True)
    for batch in (3, 7, 60):
        tkw = dict(beam_size=6, batch_size=batch, optimization_loops=2)
        wb, wd, _, _ = oracle.generate_ann(tv, oracle.make_config(**tkw))
        tlo, thi = partition_rows(250, world)[rank]
        tiny = ShardedANN(torch.from_numpy(tv[tlo:thi]).to(dev), mode="rows", **tkw)
        assert np.array_equal(tiny.index.beams.cpu().numpy(), wb), f"batch_size {batch}: graph differs from the oracle"
        assert np.array_equal(tiny.index.distances.cpu().numpy(), wd)

    # mode "shards": local graphs + cross-shard merge; quality check against brute force.  The merge finds a
    # foreign row's neighbours in a shard either with the tensor-core tile pass (default) or by searching the
    # shard's graph.
    full = vectors
    d = (1 - queries @ full.t()) / 2
    truth = torch.topk(d, 10, dim=1, largest=False).indices
    own = torch.arange(lo, hi, device=dev, dtype=torch.int32).unsqueeze(1)
    dg = (1 - full[lo:hi] @ full.t()) / 2
    dg[torch.arange(hi - lo, device=dev), torch.arange(lo, hi, device=dev)] = float("inf")
    gtruth = torch.topk(dg, 10, dim=1, largest=False).indices
    report = {}
    for merge in ("tile", "search"):
        shards = ShardedANN(vectors[lo:hi].contiguous(), mode="shards", merge=merge, **kw)
        ids2, _ = shards.search(queries)
        hits = (ids2[:, :10].long().unsqueeze(2) == truth.unsqueeze(1)).any(2).float().mean().item()
        assert hits >= 0.95, (merge, hits)
        b = shards.beams
        assert b.shape == (hi - lo, kw["beam_size"]) and int(b[b != 2147483647].max()) < vectors.size(0)
        assert bool((b != own).all()), "self loop in the merged graph"
        graph_hits = (b[:, :10].long().unsqueeze(2) == gtruth.unsqueeze(1)).any(2).float().mean().item()
        foreign = ((b < lo) | (b >= hi)) & (b != 2147483647)
        assert bool(foreign.any()), "the merge pass brought no neighbour from the other shard"
        report[merge] = (hits, graph_hits)
    assert report["tile"][1] >= 0.9, report           # merged graph recall@10 against the exact neighbours
    assert _lib_status_clear(dev)
    dist.barrier()
    if rank == 0:
        print(f"MULTI_GPU_OK shards(search recall, graph recall) = {report}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

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

    # mode "shards": local graphs + cross-shard merge; quality check against brute force
    shards = ShardedANN(vectors[lo:hi].contiguous(), mode="shards", **kw)
    ids2, _ = shards.search(queries)
    full = vectors
    d = (1 - queries @ full.t()) / 2
    truth = torch.topk(d, 10, dim=1, largest=False).indices
    hits = (ids2[:, :10].long().unsqueeze(2) == truth.unsqueeze(1)).any(2).float().mean().item()
    assert hits >= 0.95, hits
    b = shards.beams
    assert b.shape == (hi - lo, kw["beam_size"]) and int(b[b != 2147483647].max()) < vectors.size(0)
    own = torch.arange(lo, hi, device=dev, dtype=torch.int32).unsqueeze(1)
    assert bool((b != own).all()), "self loop in the merged graph"
    dist.barrier()
    if rank == 0:
        print(f"MULTI_GPU_OK recall_shards={hits:.3f}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

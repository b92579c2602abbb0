"""Sharded graph build and data-parallel search over the GPUs of one box (not in the
reference, which is single-device: `DEVICE = "cuda"`, constants.py:7).

One process per GPU, `torch.distributed` for the plumbing (NCCL on GPUs).  Rank r owns a
contiguous block of rows of the vector set; ids stay global int32.

Two build modes:

mode="shards"
        1. every rank builds the graph of its own shard with the single-GPU path (no
           communication);
        2. merge pass, chunk by chunk: the owners' rows are all-gathered, every rank looks
           for the neighbours of the other shards' rows inside its own shard, the per-shard
           candidate lists [chunk, D] (global ids, distances) are all-gathered, and each owner
           keeps the D best distinct (distance, id) pairs of its own list and the G-1 foreign
           ones.  How a rank finds a foreign row's neighbours in its shard: merge="tile"
           (default) scores the foreign rows against the whole shard on the tensor cores
           (the tile pass of knn_tile.py) and reranks the proposals with exact distances;
           merge="search" beam-searches the shard's graph (`ANN.search` on the local index),
           which only finds them when a seed lands in the right region of the shard.  Work
           per GPU grows with the number of shards (every shard is scanned for every foreign
           row).
mode="rows" (default)
        the shards' vectors are all-gathered first (20M x 1024 fp32 is 82 GB of a B200's
        180 GB), then the single-GPU algorithm runs with the ROWS of every round split across
        the ranks and the new neighbour lists exchanged after each round (generate_ann with
        `group`): the graph is the one a single GPU would build over the whole set, and the
        work per GPU does not depend on the number of ranks.
search  vectors and graph are on every GPU, query batches are split across the ranks,
        searched independently and the queues all-gathered.

Remote rows only ever arrive through collectives into this GPU's own memory before a kernel
reads them.  The choreography is independent of the device: the unit tests run it on CPU
ranks over gloo with stand-in search/merge callables.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor

from .constants import MAXFLOAT, MAXINT


def partition_rows(total: int, world: int) -> List[Tuple[int, int]]:
    """Contiguous row blocks: shard s owns [lo, hi); sizes differ by at most one row."""
    base, extra = divmod(total, world)
    bounds, lo = [], 0
    for s in range(world):
        hi = lo + base + (1 if s < extra else 0)
        bounds.append((lo, hi))
        lo = hi
    return bounds


def shard_offsets(n_local: int, group=None) -> List[int]:
    """Global id of every shard's first row (all-gather of the shard sizes)."""
    world = dist.get_world_size(group)
    sizes = [None] * world
    dist.all_gather_object(sizes, int(n_local), group=group)
    offsets, lo = [], 0
    for s in sizes:
        offsets.append(lo)
        lo += s
    offsets.append(lo)
    return offsets


def _all_gather_rows(t: Tensor, group=None) -> Tensor:
    """[rows, ...] of every rank stacked as [world, rows, ...] (equal shapes on all ranks)."""
    world = dist.get_world_size(group)
    out = torch.empty((world,) + tuple(t.shape), dtype=t.dtype, device=t.device)
    dist.all_gather_into_tensor(out.view(-1), t.contiguous().view(-1), group=group) if t.is_cuda else \
        dist.all_gather(list(out.unbind(0)), t.contiguous(), group=group)
    return out


def merge_pass(local_vectors: Tensor, local_ids: Tensor, local_dist: Tensor, offsets: List[int], degree: int,
               search_fn: Callable[[Tensor], Tuple[Tensor, Tensor]],
               merge_fn: Callable[[Tensor, Tensor, int], Tuple[Tensor, Tensor]], chunk_rows: int = 65536,
               group=None) -> Tuple[Tensor, Tensor]:
    """Cross-shard candidate exchange.

    local_ids/local_dist: this shard's graph [n_loc, degree] with GLOBAL ids.
    search_fn(rows[fp32 b, dim]) -> (ids[b, degree] GLOBAL, dist[b, degree]): the neighbours of
    foreign rows inside this shard.  merge_fn(ids[b, m], dist[b, m], degree) -> the `degree` best
    distinct pairs per row.  Returns the merged (ids, dist) of this shard's rows.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    n_loc, dim = local_vectors.shape
    sizes = [offsets[s + 1] - offsets[s] for s in range(world)]
    out_ids = torch.empty_like(local_ids)
    out_dist = torch.empty_like(local_dist)
    for c0 in range(0, max(sizes), chunk_rows):
        rows = min(chunk_rows, max(sizes) - c0)
        mine = max(0, min(rows, n_loc - c0))
        chunk = torch.zeros((rows, dim), dtype=local_vectors.dtype, device=local_vectors.device)
        if mine:
            chunk[:mine] = local_vectors[c0:c0 + mine]
        gathered = _all_gather_rows(chunk, group)                       # [world, rows, dim]
        part_ids = torch.full((world, rows, degree), MAXINT, dtype=torch.int32, device=local_vectors.device)
        part_dist = torch.full((world, rows, degree), MAXFLOAT, dtype=torch.float32, device=local_vectors.device)
        for src in range(world):
            valid = max(0, min(rows, sizes[src] - c0))
            if valid == 0:
                continue
            if src == rank:
                part_ids[src, :valid] = local_ids[c0:c0 + valid]
                part_dist[src, :valid] = local_dist[c0:c0 + valid]
            elif n_loc > 0:
                ids, d = search_fn(gathered[src, :valid].contiguous())
                part_ids[src, :valid] = ids[:, :degree]
                part_dist[src, :valid] = d[:, :degree]
        all_ids = _all_gather_rows(part_ids, group)                     # [world(by), world(for), rows, degree]
        all_dist = _all_gather_rows(part_dist, group)
        if mine:
            cand_ids = all_ids[:, rank, :mine].permute(1, 0, 2).reshape(mine, world * degree).contiguous()
            cand_dist = all_dist[:, rank, :mine].permute(1, 0, 2).reshape(mine, world * degree).contiguous()
            m_ids, m_dist = merge_fn(cand_ids, cand_dist, degree)
            out_ids[c0:c0 + mine] = m_ids
            out_dist[c0:c0 + mine] = m_dist
    return out_ids, out_dist


def split_queries(count: int, world: int) -> List[Tuple[int, int]]:
    return partition_rows(count, world)


class ShardedANN:
    """Graph over a vector set whose rows are spread over the ranks of `group`.

    `local_vectors` fp32 [n_loc, dim] on this rank's GPU; keyword arguments are those of `ANN`.
    After construction: `.beams/.distances` [n_loc, D] of this shard's rows with global ids, and
    (with `replicate=True`) `.index`, an `ANN` over the whole set on every rank for `.search`.
    """

    def __init__(self, local_vectors: Tensor, group=None, mode: str = "rows", merge=True,
                 replicate: bool = True, chunk_rows: int = 65536, **ann_kwargs):
        from .ann import ANN
        from .kernels import sort_pairs_
        assert mode in ("rows", "shards")
        assert merge in (True, False, "tile", "search")
        merge = "tile" if merge is True else merge
        self.group = group if group is not None else dist.group.WORLD
        group = self.group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.offsets = shard_offsets(local_vectors.size(0), group)
        base = self.offsets[self.rank]
        if mode == "rows":
            self.local = None
            vectors = self._gather_blocks(local_vectors.contiguous())
            self.index = ANN(vectors, group=group if self.world > 1 else None, **ann_kwargs)
            self.beams = self.index.beams[base:self.offsets[self.rank + 1]]
            self.distances = self.index.distances[base:self.offsets[self.rank + 1]]
            return
        self.local = ANN(local_vectors, **ann_kwargs)
        degree = self.local.beams.size(1)
        ids = torch.where(self.local.beams == MAXINT, self.local.beams, self.local.beams + base)
        dist_ = self.local.distances

        def search_fn(rows: Tensor):
            q = self.local.search(rows)
            got = q.indices[:, :degree]
            return torch.where(got == MAXINT, got, got + base), q.distances[:, :degree]

        tile_state = {}

        def tile_fn(rows: Tensor):
            """Neighbours of foreign rows inside this shard: tensor-core proposals over the whole shard,
            exact distances, queue order (knn_tile.py).  The shard's bf16 copy is made once; the foreign
            chunk is appended behind it so that one matrix holds both sides of the tile pass."""
            from . import knn_tile
            from .kernels import calculate_distances, metric_code
            local = self.local.vectors
            metric = self.local.configuration.get("metric", "cosine")
            n_loc = local.size(0)
            if not tile_state:
                head, norms = knn_tile.prepare(local, want_norms=metric_code(metric) == 1)
                both = torch.empty((n_loc + chunk_rows, head.size(1)), dtype=head.dtype, device=head.device)
                both[:n_loc] = head
                tile_state["both"] = both
                if norms is not None:
                    tile_state["norms"] = torch.cat([norms, torch.zeros(chunk_rows, dtype=norms.dtype, device=norms.device)])
            both = tile_state["both"]
            b = rows.size(0)
            knn_tile.prepare(rows.contiguous(), want_norms=False, out=both[n_loc:n_loc + b])
            got = knn_tile.proposals(both, tile_state.get("norms"), (n_loc, n_loc + b), (0, n_loc), 1)
            d = calculate_distances(local, got, metric=metric, queries=rows.contiguous())
            sort_pairs_(got, d, dedup=True)
            got, d = got[:, :degree], d[:, :degree]
            return torch.where(got == MAXINT, got, got + base), d

        def merge_fn(cand_ids: Tensor, cand_dist: Tensor, keep: int):
            sort_pairs_(cand_ids, cand_dist, dedup=True)      # (distance, id) order, repeats out
            return cand_ids[:, :keep], cand_dist[:, :keep]

        if merge and self.world > 1:
            ids, dist_ = merge_pass(self.local.vectors, ids.contiguous(), dist_.contiguous(), self.offsets, degree,
                                    tile_fn if merge == "tile" else search_fn, merge_fn, chunk_rows, group)
            tile_state.clear()
        self.beams, self.distances = ids, dist_
        self.index = None
        if replicate:
            self.index = self._replicate(ann_kwargs)

    def _gather_blocks(self, t: Tensor) -> Tensor:
        """Row blocks of every rank (sizes from self.offsets) concatenated in rank order."""
        sizes = [self.offsets[s + 1] - self.offsets[s] for s in range(self.world)]
        if self.world == 1:
            return t
        pad = max(sizes)
        buf = torch.zeros((pad,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        buf[: t.size(0)] = t
        g = _all_gather_rows(buf, self.group)
        if all(sz == pad for sz in sizes):
            return g.reshape((-1,) + tuple(t.shape[1:]))
        return torch.cat([g[s, : sizes[s]] for s in range(self.world)], 0).contiguous()

    def _replicate(self, ann_kwargs):
        from .ann import ANN
        vectors = self._gather_blocks(self.local.vectors)
        beams = self._gather_blocks(self.beams.contiguous())
        distances = self._gather_blocks(self.distances.contiguous())
        assert vectors.size(0) == self.offsets[-1]
        kw = {k: v for k, v in ann_kwargs.items() if k not in ("beams", "distances")}
        kw["beam_size"] = beams.size(1)
        return ANN(vectors, beams=beams, distances=distances, **kw)

    def search(self, query: Tensor):
        """Data-parallel `.search`: every rank holds all `query` rows, searches its slice of them
        on the replicated index, and the queues are all-gathered; returns (indices, distances)
        [B, capacity] on every rank."""
        assert self.index is not None, "search needs replicate=True"
        bounds = split_queries(query.size(0), self.world)
        lo, hi = bounds[self.rank]
        width = max(h - l for l, h in bounds)
        q = self.index.search(query[lo:hi].contiguous(), first_row=lo) if hi > lo else None
        cap = self.index.search(query[:1].contiguous()).indices.size(1) if q is None else q.indices.size(1)
        ids = torch.full((width, cap), MAXINT, dtype=torch.int32, device=query.device)
        dd = torch.full((width, cap), MAXFLOAT, dtype=torch.float32, device=query.device)
        if q is not None:
            ids[: hi - lo] = q.indices
            dd[: hi - lo] = q.distances
        gi = _all_gather_rows(ids, self.group)
        gd = _all_gather_rows(dd, self.group)
        out_i = torch.cat([gi[s, : bounds[s][1] - bounds[s][0]] for s in range(self.world)], 0)
        out_d = torch.cat([gd[s, : bounds[s][1] - bounds[s][0]] for s in range(self.world)], 0)
        return out_i, out_d

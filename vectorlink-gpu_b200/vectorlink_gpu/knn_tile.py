"""Opt-in start graph from a tensor-core kNN tile pass (`ANN(init="knn_tile")`).

The reference starts every build from a circulant graph (utils.py:35-41, ann.py:116-118):
row i's first neighbours are rows i + p_j, i.e. arbitrary rows, and the first optimisation
round spends its whole budget finding real neighbours.  This module proposes near neighbours
with bf16 inner products on the tensor cores (csrc/vl_knn_tile.cu), then evaluates every proposed
pair with the exact fp32 distance and orders the lists with the queue order, so the start
graph holds exact distances and only real candidates; bf16 never reaches a list.

Default builds do not come here: `init="circulant"` is the reference's behaviour.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Tuple

import torch
from torch import Tensor

from . import _lib
from ._lib import check, lib, ptr, stream_of
from .constants import MAXFLOAT, MAXINT
from .kernels import calculate_distances, metric_code, sort_pairs_
from .log import nvtx_range

TILE_K = 16            # VL_KNN_TILE_K: ids per list
TILE_LISTS = 4         # VL_KNN_TILE_LISTS: lists per row and candidate segment (one per 64-candidate quarter of the tiles)
PER_SEGMENT = TILE_K * TILE_LISTS
BLOCK_K = 64           # the bf16 copy is padded to a multiple of this many columns


def prepare(vectors: Tensor, want_norms: bool, out: Optional[Tensor] = None) -> Tuple[Tensor, Optional[Tensor]]:
    """bf16 copy of the rows, zero-padded to a multiple of 64 columns, and |row|^2 (fp32) when asked.
    `out` (optional): a contiguous bf16 [rows, padded columns] tensor to write the copy into."""
    _lib.require_cuda(vectors)
    assert vectors.dtype == torch.float32 and vectors.is_contiguous()
    (n, dim) = vectors.size()
    dim_pad = (dim + BLOCK_K - 1) // BLOCK_K * BLOCK_K
    if out is None:
        rows_bf16 = torch.empty((n, dim_pad), dtype=torch.bfloat16, device=vectors.device)
    else:
        rows_bf16 = out
        assert rows_bf16.dtype == torch.bfloat16 and rows_bf16.is_contiguous() and tuple(rows_bf16.shape) == (n, dim_pad)
    norms = torch.empty(n, dtype=torch.float32, device=vectors.device) if want_norms else None
    check(lib().vl_knn_prepare(ptr(vectors), ctypes.c_int64(n), dim, ptr(rows_bf16), dim_pad, ptr(norms),
                               stream_of(vectors)), "vl_knn_prepare")
    return rows_bf16, norms


def proposals(rows_bf16: Tensor, norms: Optional[Tensor], rows: Tuple[int, int], candidates: Tuple[int, int],
              segments: int) -> Tensor:
    """int32 [rows, segments * 64]: per row and per part of the candidate range (`segments` equal
    parts) four lists of 16 ids: list k holds the best-scoring candidates among the k-th quarters
    (64 candidates) of the part's 256-candidate tiles (approximate scores; the row itself excluded),
    MAXINT-padded."""
    _lib.require_cuda(rows_bf16, norms)
    assert rows_bf16.dtype == torch.bfloat16 and rows_bf16.is_contiguous()
    (n, dim_pad) = rows_bf16.size()
    (lo, hi) = rows
    out = torch.empty((hi - lo, segments * PER_SEGMENT), dtype=torch.int32, device=rows_bf16.device)
    check(lib().vl_knn_tile(ptr(rows_bf16), ctypes.c_int64(n), dim_pad, ptr(norms), ctypes.c_int64(lo), ctypes.c_int64(hi),
                            ctypes.c_int64(candidates[0]), ctypes.c_int64(candidates[1]), segments, ptr(out),
                            ptr(_lib.status_word(rows_bf16.device)), stream_of(rows_bf16)), "vl_knn_tile")
    return out


def exact_lists(vectors: Tensor, ids: Tensor, row_lo: int, width: int, metric: str) -> Tuple[Tensor, Tensor]:
    """The fp32 rerank: exact distances of the proposed pairs (the same summation tree as every
    other distance), rows put in queue order with repeats removed, cut or MAXINT-padded to `width`."""
    rows = ids.size(0)
    dist = calculate_distances(vectors, ids, metric=metric, queries=vectors[row_lo:row_lo + rows])
    sort_pairs_(ids, dist, dedup=True)
    if ids.size(1) >= width:
        return ids[:, :width].contiguous(), dist[:, :width].contiguous()
    out_i = torch.full((rows, width), MAXINT, dtype=torch.int32, device=ids.device)
    out_d = torch.full((rows, width), MAXFLOAT, dtype=torch.float32, device=ids.device)
    out_i[:, : ids.size(1)] = ids
    out_d[:, : ids.size(1)] = dist
    return out_i, out_d


def knn_start_graph(vectors: Tensor, width: int, config: Dict, group=None) -> Tuple[Tensor, Tensor]:
    """Start graph [N, width] (ids, exact distances) for generate_ann: per row the exact-reranked
    proposals of the tile pass, at most 64 per candidate segment, MAXINT-padded to `width`.
    config["knn_segments"] (default 1) cuts the row range into that many candidate segments; more
    segments give more proposals per row and cost more (measured on 1M x 128: 1, 2 and 3 segments end
    in the same graph after one round, and one segment is the fastest build by 40-70 %).  With `group`, each rank
    computes the lists of its share of the rows and the lists are all-gathered (every rank holds all
    vectors)."""
    (n, dim) = vectors.size()
    metric = config.get("metric", "cosine")
    segments = max(1, int(config.get("knn_segments", 1)))
    world, rank = 1, 0
    if group is not None:
        import torch.distributed as dist
        world, rank = dist.get_world_size(group), dist.get_rank(group)
    per = (n + world - 1) // world
    lo, hi = min(n, rank * per), min(n, (rank + 1) * per)
    with nvtx_range("vl.knn_tile.prepare"):
        rows_bf16, norms = prepare(vectors, want_norms=metric_code(metric) == 1)
    beams = torch.empty((world * per, width), dtype=torch.int32, device=vectors.device)
    dists = torch.empty((world * per, width), dtype=torch.float32, device=vectors.device)
    if hi > lo:
        with nvtx_range("vl.knn_tile.proposals"):
            ids = proposals(rows_bf16, norms, (lo, hi), (0, n), segments)
        with nvtx_range("vl.knn_tile.rerank"):
            (b, d) = exact_lists(vectors, ids, lo, width, metric)
        beams[lo:hi] = b
        dists[lo:hi] = d
    if world > 1:
        from .ann import _gather_row_blocks
        _gather_row_blocks(beams, per, group)
        _gather_row_blocks(dists, per, group)
    return beams[:n], dists[:n]

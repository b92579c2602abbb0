"""Launch wrappers with the reference's operator signatures (vectorlink_gpu/kernels.py).

Each function keeps the name, argument meaning and asserted contracts of the reference
operator it replaces and calls one entry point of libvlgpu.so on torch's current stream.
`metric` is the only added argument ("cosine", the reference's distance, or "l2" = squared
Euclidean).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch
from torch import Tensor

from . import _lib
from ._lib import check, lib, ptr, stream_of
from .constants import MAXFLOAT, MAXINT
from .log import log_time

METRICS = {"cosine": 0, 0: 0, "l2": 1, "sqeuclidean": 1, 1: 1}


def metric_code(metric) -> int:
    try:
        return METRICS[metric]
    except KeyError:
        raise ValueError(f"unknown metric {metric!r}; use 'cosine' or 'l2'") from None


@log_time
def calculate_distances(vectors: Tensor, beams: Tensor, distances_out=None, metric="cosine",
                        queries: Optional[Tensor] = None) -> Tensor:
    """kernels.py:174-201: out[i, j] = distance(vectors[i], vectors[beams[i, j]]), MAXFLOAT
    where beams[i, j] == MAXINT.  `queries` (added) takes the left-hand rows from another
    matrix: out[i, j] = distance(queries[i], vectors[beams[i, j]])."""
    assert vectors.dtype == torch.float32
    assert vectors.is_contiguous()
    assert beams.dtype == torch.int32
    assert beams.is_contiguous()
    q = vectors if queries is None else queries
    assert q.dtype == torch.float32 and q.is_contiguous()
    _lib.require_cuda(vectors, beams, q)
    (vector_count, vector_dimension) = vectors.size()
    (batches, beam_size) = beams.size()
    assert batches == q.size(0)
    assert q.size(1) == vector_dimension
    if distances_out is None:
        distances_out = torch.empty((batches, beam_size), dtype=torch.float32, device=vectors.device)
    else:
        assert distances_out.is_contiguous() and distances_out.dtype == torch.float32
    check(lib().vl_calculate_distances(ptr(vectors), ctypes.c_int64(vector_count), vector_dimension, ptr(q),
                                       ctypes.c_int64(batches), ptr(beams), beam_size, ptr(distances_out),
                                       metric_code(metric), ptr(_lib.status_word(vectors.device)),
                                       stream_of(vectors)), "vl_calculate_distances")
    return distances_out


def search_from_seeds(query_vecs: Tensor, neighbors_to_visit: Tensor, beams: Tensor, vectors: Tensor,
                      metric="cosine") -> Tuple[Tensor, Tensor]:
    """kernels.py:260-311: ids and distances of the neighbours of the visited nodes, slot
    v*W + j for visited column v and neighbour slot j; sentinels for a MAXINT visit."""
    assert query_vecs.dtype == torch.float32
    assert query_vecs.is_contiguous()
    assert neighbors_to_visit.dtype == torch.int32
    assert neighbors_to_visit.is_contiguous()
    assert beams.dtype == torch.int32
    assert beams.is_contiguous()
    assert vectors.is_contiguous()
    assert vectors.dtype == torch.float32
    _lib.require_cuda(query_vecs, neighbors_to_visit, beams, vectors)
    (batch_size, visit_length) = neighbors_to_visit.size()
    (_, beam_size) = beams.size()
    (vector_count, vector_dimension) = vectors.size()
    index_out = torch.empty((batch_size, visit_length * beam_size), dtype=torch.int32, device=vectors.device)
    distance_out = torch.empty((batch_size, visit_length * beam_size), dtype=torch.float32, device=vectors.device)
    check(lib().vl_search_from_seeds(ptr(query_vecs), ctypes.c_int64(batch_size), ptr(neighbors_to_visit),
                                     visit_length, ptr(beams), beam_size, ptr(vectors),
                                     ctypes.c_int64(vector_count), vector_dimension, ptr(index_out),
                                     ptr(distance_out), metric_code(metric),
                                     ptr(_lib.status_word(vectors.device)), stream_of(vectors)),
          "vl_search_from_seeds")
    return (index_out, distance_out)


def dedup_tensor_(ids: Tensor):
    """kernels.py:370-380: in place, an id equal to the one before it becomes MAXINT."""
    assert ids.is_contiguous()
    assert ids.dtype == torch.int32
    _lib.require_cuda(ids)
    (batch_size, queue_size) = ids.size()
    check(lib().vl_dedup_adjacent(ptr(ids), None, ctypes.c_int64(batch_size), queue_size, stream_of(ids)),
          "vl_dedup_adjacent")


def dedup_tensor_pair_(ids: Tensor, distances: Tensor):
    """kernels.py:383-397.  Assumes sorted tensors!"""
    (batch_size, queue_size) = ids.size()
    (batch_size2, queue_size2) = distances.size()
    assert batch_size == batch_size2
    assert queue_size == queue_size2
    assert ids.is_contiguous()
    assert distances.is_contiguous()
    _lib.require_cuda(ids, distances)
    check(lib().vl_dedup_adjacent(ptr(ids), ptr(distances), ctypes.c_int64(batch_size), queue_size,
                                  stream_of(ids)), "vl_dedup_adjacent")


def punchout_duplicates_(ids: Tensor, distances: Tensor):
    """kernels.py:400-406: dedup the sorted pair in place, then move the punched entries last;
    returns the re-sorted (ids, distances)."""
    dedup_tensor_pair_(ids, distances)
    ids = ids.clone()
    distances = distances.clone()
    (batch_size, queue_size) = ids.size()
    check(lib().vl_sort_pairs(ptr(ids), ptr(distances), ctypes.c_int64(batch_size), queue_size, 0,
                              stream_of(ids)), "vl_sort_pairs")
    assert ids.dtype == torch.int32
    assert distances.dtype == torch.float32
    return (ids, distances)


def prune_(beams: Tensor, distances: Tensor, out_cols: Optional[int] = None, punch: bool = True, full: bool = False,
           rows: Optional[Tuple[int, int]] = None, out: Optional[Tuple[Tensor, Tensor]] = None):
    """kernels.py:441-468: remove detourable links (x->z when d_xz > d_xy and d_xz > d_yz, z the
    first neighbour of y), then order every row by distance.  Returns new (beams, distances);
    `out_cols` (added) keeps only the first columns; `full` (added) tests every neighbour of y as the
    detour witness, which is what the reference's docstring describes (its launch only ever
    looks at y's first neighbour); `rows` = (lo, hi) (added) prunes only those rows - the others
    are read, their output rows are left untouched - and `out` (added) gives the output tensors."""
    assert beams.dtype == torch.int32
    assert distances.dtype == torch.float32
    assert beams.is_contiguous() and distances.is_contiguous()
    _lib.require_cuda(beams, distances)
    (batch_size, beam_size) = beams.size()
    cols = beam_size if out_cols is None else out_cols
    if out is None:
        out_b = torch.empty((batch_size, cols), dtype=torch.int32, device=beams.device)
        out_d = torch.empty((batch_size, cols), dtype=torch.float32, device=beams.device)
    else:
        (out_b, out_d) = out
        assert out_b.dtype == torch.int32 and out_d.dtype == torch.float32
        assert out_b.is_contiguous() and out_d.is_contiguous()
        assert tuple(out_b.shape) == (batch_size, cols) and tuple(out_d.shape) == (batch_size, cols)
    (lo, hi) = (0, batch_size) if rows is None else rows
    check(lib().vl_prune_rows(ptr(beams), ptr(distances), ctypes.c_int64(batch_size), beam_size, ctypes.c_int64(lo),
                              ctypes.c_int64(hi), (2 if full else 1) if punch else 0, ptr(out_b), ptr(out_d), cols,
                              ptr(_lib.status_word(beams.device)), stream_of(beams)), "vl_prune_rows")
    return (out_b, out_d)


def punchout_excluded_(indices: Tensor, distances: Tensor, exclusions: Tensor):
    """kernels.py:491-501: in place on (possibly column-sliced) views."""
    (batch_size, queue_size) = indices.size()
    (batch_size2, exclusion_size) = exclusions.size()
    assert batch_size == batch_size2
    assert indices.dtype == torch.int32 and distances.dtype == torch.float32
    assert exclusions.dtype == torch.int32 and exclusions.is_contiguous()
    assert indices.stride(1) == 1 and distances.stride(1) == 1
    _lib.require_cuda(indices, distances, exclusions)
    check(lib().vl_punchout_excluded(ptr(indices), ptr(distances), ctypes.c_int64(indices.stride(0)),
                                     ctypes.c_int64(distances.stride(0)), ctypes.c_int64(batch_size), queue_size,
                                     ptr(exclusions), exclusion_size, stream_of(indices)), "vl_punchout_excluded")


def sort_pairs_(ids: Tensor, distances: Tensor, dedup: bool):
    """Rows ordered by (distance, id) in place; with `dedup` also queue_sort's punch-and-compact."""
    assert ids.is_contiguous() and distances.is_contiguous()
    assert ids.dtype == torch.int32 and distances.dtype == torch.float32
    _lib.require_cuda(ids, distances)
    (batch_size, queue_size) = ids.size()
    check(lib().vl_sort_pairs(ptr(ids), ptr(distances), ctypes.c_int64(batch_size), queue_size, 1 if dedup else 0,
                              stream_of(ids)), "vl_sort_pairs")


def index_by_tensor(a: Tensor, b: Tensor):
    """kernels.py:554-559: row-wise gather a[i, b[i, j]]."""
    return torch.gather(a, 1, b.long())


def reverse_edges(beams: Tensor, scan: Optional[int] = None, keep: Optional[int] = None) -> Tensor:
    """For every node the nodes that list it among their first `scan` neighbours, ordered by
    (rank in the lister's row, lister id), int32 [N, keep] padded with MAXINT.  The role of the
    reference's symmetrize_beams (kernels.py:534-550, dead code there)."""
    assert beams.dtype == torch.int32 and beams.is_contiguous()
    _lib.require_cuda(beams)
    (n, d) = beams.size()
    scan = d if scan is None else scan
    keep = max(1, d // 2) if keep is None else keep
    dev = beams.device
    deg = torch.zeros(n, dtype=torch.int32, device=dev)
    status = _lib.status_word(dev)
    check(lib().vl_reverse_edges(ptr(beams), n, d, scan, 0, ptr(deg), None, None, None, keep, None, ptr(status),
                                 stream_of(beams)), "vl_reverse_edges")
    offsets = torch.cumsum(deg, 0, dtype=torch.int64) - deg
    total = int(offsets[-1].item() + deg[-1].item()) if n else 0
    keys = torch.empty(max(total, 1), dtype=torch.int64, device=dev)
    cursor = torch.zeros(n, dtype=torch.int32, device=dev)
    out = torch.empty((n, keep), dtype=torch.int32, device=dev)
    check(lib().vl_reverse_edges(ptr(beams), n, d, scan, 1, ptr(deg), ptr(offsets), ptr(cursor), ptr(keys), keep,
                                 ptr(out), ptr(status), stream_of(beams)), "vl_reverse_edges")
    _lib.LAUNCHES += 1      # the second phase is two kernels (fill, select)
    return out


def connected_components(ids: Tensor, distances: Optional[Tensor] = None, threshold: float = MAXFLOAT) -> Tensor:
    """Cluster labels of a neighbour graph: int32 [N], the smallest id of each node's connected
    component, where x and ids[x, s] are linked (both ways) when the id is real and
    distances[x, s] <= threshold.  `ids` int32 [N, w] may be a column slice of a wider tensor
    (a Queue head).  The step the reference announces for `ANN.clusters` (README.md:24) and
    leaves as a stub (ann.py:466-467)."""
    assert ids.dtype == torch.int32 and ids.dim() == 2
    assert distances is None or (distances.dtype == torch.float32 and distances.size() == ids.size())
    _lib.require_cuda(ids, distances)
    (n, w) = ids.size()
    sliced = n > 1 and w > 0 and ids.stride(1) == 1 and ids.stride(0) >= w
    if sliced and (distances is None or distances.stride() == ids.stride()):
        ld = ids.stride(0)
    else:
        ids = ids.contiguous()
        distances = distances.contiguous() if distances is not None else None
        ld = w
    labels = torch.empty(n, dtype=torch.int32, device=ids.device)
    status = _lib.status_word(ids.device)
    check(lib().vl_connected_components(ptr(ids), ptr(distances), n, w, ld,
                                        float(threshold), ptr(labels), ptr(status), stream_of(ids)),
          "vl_connected_components")
    return labels


def symmetrize(vectors: Tensor, beams: Tensor, distances: Tensor, keep: Optional[int] = None, metric="cosine"):
    """The intent of the reference's `symmetrize` sketch (utils.py:92-103, dead code): give every
    node up to `keep` (default half its degree) of its reverse edges.  The new row is the
    distinct ids of: the best degree-keep forward neighbours, then the reverse neighbours, then
    the remaining forward ones - cut to the degree and ordered by distance.  Not in the
    reference's live code, so there is no parity target; it is assessed by recall."""
    (n, d) = beams.size()
    keep = max(1, d // 2) if keep is None else min(keep, d)
    rev = reverse_edges(beams, scan=d, keep=keep)
    rev_dist = calculate_distances(vectors, rev, metric=metric)
    own = torch.arange(n, device=beams.device, dtype=torch.int32).unsqueeze(1)
    rev = torch.where(rev == own, torch.full_like(rev, MAXINT), rev)
    # three priority classes, concatenated in priority order: 0 forward head, 1 reverse, 2 forward
    # tail.  Within a class the columns keep the order they arrive in (forward lists by distance,
    # reverse lists by the lister's rank), so "earlier column" means "better" throughout.
    ids = torch.cat([beams[:, : d - keep], rev, beams[:, d - keep:]], 1).contiguous()
    dist = torch.cat([distances[:, : d - keep], rev_dist, distances[:, d - keep:]], 1).contiguous()
    cls = torch.cat([torch.zeros((n, d - keep), dtype=torch.int32), torch.ones((n, keep), dtype=torch.int32),
                     torch.full((n, keep), 2, dtype=torch.int32)], 1).to(dist.device)
    cls = torch.where(ids == MAXINT, torch.full_like(cls, 3), cls)
    # drop repeated ids keeping the first (best class) occurrence
    by_id = torch.argsort(ids, dim=1, stable=True)
    sid = torch.gather(ids, 1, by_id)
    dup_sorted = torch.zeros_like(sid, dtype=torch.bool)
    dup_sorted[:, 1:] = sid[:, 1:] == sid[:, :-1]
    dup = torch.zeros_like(dup_sorted).scatter(1, by_id, dup_sorted)
    ids = torch.where(dup, torch.full_like(ids, MAXINT), ids)
    cls = torch.where(dup | (ids == MAXINT), torch.full_like(cls, 3), cls)
    keep_order = torch.argsort(cls, dim=1, stable=True)[:, :d]
    ids = torch.gather(ids, 1, keep_order).contiguous()
    dist = torch.gather(dist, 1, keep_order)
    dist = torch.where(ids == MAXINT, torch.full_like(dist, MAXFLOAT), dist).contiguous()
    sort_pairs_(ids, dist, dedup=False)
    return ids, dist

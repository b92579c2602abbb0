"""CPU oracle for the VectorLink ANN hot path -- TEST INFRASTRUCTURE ONLY.

A ctypes front end over ``vl_oracle.c`` (a plain-C restatement of the reference's
``vectorlink_gpu/kernels.py``, ``queue.py``, ``utils.py`` and ``ann.py``), taking and
returning NumPy arrays.  It is the checker for the CUDA path: only the test-suite, the
smoke check and the CPU-baseline / reference legs of the benchmark may import it.  The
product package never does.

Parity status: pinned (see the header of ``vl_oracle.c``).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional, Tuple

import numpy as np

MAXINT = 2147483647  # constants.py:5
MAXFLOAT = float(np.float32(3.4028e37))  # constants.py:6, as stored in fp32
COSINE = 0
SQL2 = 1

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "vl_oracle.c")
_SO = os.path.join(_HERE, "libvloracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile ``vl_oracle.c`` with gcc into ``libvloracle.so`` beside it."""
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(_SRC):
        cmd = ["gcc", "-O2", "-fno-fast-math", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC",
               "-o", _SO, _SRC, "-lm"]
        subprocess.check_call(cmd)
    return _SO


def metric_code(metric) -> int:
    if metric in (COSINE, "cosine"):
        return COSINE
    if metric in (SQL2, "l2", "sqeuclidean"):
        return SQL2
    raise ValueError(f"unknown metric {metric!r}")


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _p(a, ty):
    return a.ctypes.data_as(ctypes.POINTER(ty)) if a is not None else None


_F = ctypes.c_float
_I = ctypes.c_int32
_B = ctypes.c_uint8
_L = ctypes.c_int64


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_SO)
        _lib.vlo_pair_distance.restype = ctypes.c_float
        _lib.vlo_self_recall.restype = ctypes.c_int64
        _lib.vlo_connected_components.restype = ctypes.c_int64
        for name in ("vlo_queue_pop", "vlo_add_new_to_seen", "vlo_closest_vectors", "vlo_generate_ann",
                     "vlo_num_threads"):
            getattr(_lib, name).restype = ctypes.c_int
    return _lib


def num_threads() -> int:
    return int(lib().vlo_num_threads())


def set_num_threads(threads: int) -> int:
    """Use `threads` OpenMP threads from now on, whatever OMP_NUM_THREADS said at start-up."""
    lib().vlo_set_num_threads(ctypes.c_int(int(threads)))
    return num_threads()


def primes_table(count: int = 965) -> np.ndarray:
    """The reference's seed table (constants.py:10-980), regenerated rather than copied:
    the 584 consecutive primes from 10,000,349, the 75 consecutive primes from 1,009,007,
    the values 1, 2, 59063, 79193, then the consecutive primes 3..1999."""
    def sieve_range(lo, hi):
        n = hi - lo + 1
        mark = np.ones(n, dtype=bool)
        small = np.ones(int(hi ** 0.5) + 2, dtype=bool)
        small[:2] = False
        for p in range(2, len(small)):
            if small[p]:
                small[p * p::p] = False
                start = max(p * p, ((lo + p - 1) // p) * p)
                mark[start - lo::p] = False
        return (np.nonzero(mark)[0] + lo)

    a = sieve_range(10_000_349, 10_010_000)[:584]
    b = sieve_range(1_009_007, 1_010_100)[:75]
    c = np.array([1, 2, 59063, 79193])
    d = sieve_range(3, 1999)
    table = np.concatenate([a, b, c, d]).astype(np.int32)
    assert table.shape[0] == 965, table.shape
    return table[:count]


def seed_offsets(count: int) -> np.ndarray:
    """The seed table, continued past its 965 entries for widened seed scans (not in the
    reference): entry j = table[j mod 965] * (j div 965 + 1) + j, kept below 2^30."""
    table = primes_table().astype(np.int64)
    if count <= 965:
        return table[:count].astype(np.int32)
    j = np.arange(count, dtype=np.int64)
    ext = (table[j % 965] * (j // 965 + 1) + j) % (1 << 30)
    ext[:965] = table
    return ext.astype(np.int32)


def pair_distance(a, b, metric=COSINE) -> float:
    a, b = _f32(a), _f32(b)
    return float(lib().vlo_pair_distance(_p(a, _F), _p(b, _F), ctypes.c_int(a.shape[0]),
                                         ctypes.c_int(metric_code(metric))))


def calculate_distances(vectors, beams, metric=COSINE) -> np.ndarray:
    """kernels.py:174-201."""
    vectors, beams = _f32(vectors), _i32(beams)
    n, dim = vectors.shape
    assert beams.shape[0] == n
    w = beams.shape[1]
    out = np.empty((n, w), dtype=np.float32)
    lib().vlo_calculate_distances(_p(vectors, _F), _L(n), ctypes.c_int(dim), _p(beams, _I), ctypes.c_int(w),
                                  _p(out, _F), ctypes.c_int(metric_code(metric)))
    return out


def search_from_seeds(queries, visit, beams, vectors, metric=COSINE) -> Tuple[np.ndarray, np.ndarray]:
    """kernels.py:260-311."""
    queries, visit, beams, vectors = _f32(queries), _i32(visit), _i32(beams), _f32(vectors)
    b, v = visit.shape
    w = beams.shape[1]
    n, dim = vectors.shape
    idx = np.empty((b, v * w), dtype=np.int32)
    dist = np.empty((b, v * w), dtype=np.float32)
    lib().vlo_search_from_seeds(_p(queries, _F), _L(b), _p(visit, _I), ctypes.c_int(v), _p(beams, _I),
                                ctypes.c_int(w), _p(vectors, _F), _L(n), ctypes.c_int(dim), _p(idx, _I),
                                _p(dist, _F), ctypes.c_int(metric_code(metric)))
    return idx, dist


def punchout_excluded_(ids: np.ndarray, dist: np.ndarray, excl) -> None:
    """kernels.py:491-501; ids/dist may be column-sliced views of C-contiguous parents."""
    excl = _i32(excl)
    assert ids.dtype == np.int32 and dist.dtype == np.float32
    assert ids.strides[1] == 4 and dist.strides[1] == 4 and ids.strides[0] == dist.strides[0]
    ld = ids.strides[0] // 4
    b, q = ids.shape
    lib().vlo_punchout_excluded(_p(ids, _I), _p(dist, _F), _L(ld), _L(b), ctypes.c_int(q), _p(excl, _I),
                                ctypes.c_int(excl.shape[1]))


def queue_sort(ids, dist) -> Tuple[np.ndarray, np.ndarray]:
    """queue.py:15-18."""
    ids, dist = _i32(ids).copy(), _f32(dist).copy()
    b, cap = ids.shape
    lib().vlo_queue_sort(_p(ids, _I), _p(dist, _F), _L(b), ctypes.c_int(cap))
    return ids, dist


def dedup_sort(ids) -> np.ndarray:
    """utils.py:85-89."""
    ids = _i32(ids).copy()
    b, e = ids.shape
    lib().vlo_dedup_sort(_p(ids, _I), _L(b), ctypes.c_int(e))
    return ids


def add_new_to_seen_(seen: np.ndarray, visit) -> Optional[np.ndarray]:
    """utils.py:61-82; edits `seen` in place, returns it or None."""
    visit = _i32(visit)
    assert seen.dtype == np.int32 and seen.flags.c_contiguous
    b, e = seen.shape
    r = lib().vlo_add_new_to_seen(_p(seen, _I), _L(b), ctypes.c_int(e), _p(visit, _I), ctypes.c_int(visit.shape[1]))
    return seen if r else None


def prune_(beams, dist) -> Tuple[np.ndarray, np.ndarray]:
    """kernels.py:441-468 (rows must arrive sorted by distance, as generate_ann supplies them)."""
    beams, dist = _i32(beams).copy(), _f32(dist).copy()
    n, w = beams.shape
    lib().vlo_prune(_p(beams, _I), _p(dist, _F), _L(n), ctypes.c_int(w))
    return beams, dist


def circulants(rows: int, modulus: int, primes, row0: int = 0) -> np.ndarray:
    """utils.py:26-41."""
    primes = _i32(primes)
    out = np.empty((rows, primes.shape[0]), dtype=np.int32)
    lib().vlo_circulants(_L(rows), _L(row0), _L(modulus), _p(primes, _I), ctypes.c_int(primes.shape[0]), _p(out, _I))
    return out


class Queue:
    """queue.py:21-98 over NumPy arrays."""

    def __init__(self, num_queues: int, queue_length: int, capacity: int):
        assert queue_length < capacity
        self.length = queue_length
        self.indices = np.full((num_queues, capacity), MAXINT, dtype=np.int32)
        self.distances = np.full((num_queues, capacity), MAXFLOAT, dtype=np.float32)

    def insert(self, ids, dist, exclude=None, output_update=False):
        ids, dist = _i32(ids), _f32(dist)
        b, cap = self.indices.shape
        m = ids.shape[1]
        assert m <= cap - self.length
        changed = np.zeros((b, self.length), dtype=np.uint8) if output_update else None
        ex = _i32(exclude) if exclude is not None else None
        lib().vlo_queue_insert(_p(self.indices, _I), _p(self.distances, _F), _L(b), ctypes.c_int(cap),
                               ctypes.c_int(self.length), _p(ids, _I), _p(dist, _F), ctypes.c_int(m),
                               _p(ex, _I), ctypes.c_int(ex.shape[1] if ex is not None else 0), _p(changed, _B))
        return changed.astype(bool) if output_update else None

    def pop_n_ids(self, n: int) -> np.ndarray:
        b, cap = self.indices.shape
        take = min(self.length, n)
        out = np.empty((b, take), dtype=np.int32)
        lib().vlo_queue_pop(_p(self.indices, _I), _p(self.distances, _F), _L(b), ctypes.c_int(cap),
                            ctypes.c_int(self.length), ctypes.c_int(n), _p(out, _I))
        return out

    def initialize_from_queue(self, queue: "Queue") -> None:
        head = min(queue.length, self.length)
        self.indices[:, :head] = queue.indices[:, :head]
        self.distances[:, :head] = queue.distances[:, :head]

    def size(self):
        return self.indices.shape


def closest_vectors(queries, search_queue: Queue, vectors, beams, config: dict, exclude=None,
                    metric=COSINE) -> int:
    """ann.py:37-93; updates `search_queue` in place, returns the iteration count."""
    queries, vectors, beams = _f32(queries), _f32(vectors), _i32(beams)
    b, cap = search_queue.indices.shape
    n, dim = vectors.shape
    ex = _i32(exclude) if exclude is not None else None
    return int(lib().vlo_closest_vectors(
        _p(queries, _F), _L(b), _p(search_queue.indices, _I), _p(search_queue.distances, _F),
        ctypes.c_int(search_queue.length), ctypes.c_int(cap), _p(vectors, _F), _L(n), ctypes.c_int(dim),
        _p(beams, _I), ctypes.c_int(beams.shape[1]), ctypes.c_int(config["beam_size"]),
        ctypes.c_int(config["parallel_visit_count"]), ctypes.c_int(config["visit_queue_factor"]),
        ctypes.c_int(config["exclude_factor"]), ctypes.c_int(config["speculative_readahead"]),
        _p(ex, _I), ctypes.c_int(ex.shape[1] if ex is not None else 0), ctypes.c_int(metric_code(metric))))


DEFAULT_CONFIG = dict(prune=True, beam_size=24, parallel_visit_count=4, beam_queue_factor=3,
                      visit_queue_factor=3, exclude_factor=5, optimization_loops=3, batch_size=10_000,
                      recall_search_queue_factor=3, speculative_readahead=5)  # ann.py:357-372


def make_config(**kw) -> dict:
    cfg = dict(DEFAULT_CONFIG)
    cfg.update(kw)
    return cfg


def initial_search_queue(vectors, queries, config: dict, metric=COSINE) -> Queue:
    """ann.py:217-232, with the seed distances taken by the same summation tree as every
    other distance (the reference uses torch's sum order without the clamp there)."""
    vectors, queries = _f32(vectors), _f32(queries)
    q = config["recall_search_queue_factor"] * config["beam_size"]
    extra = max(q, config["parallel_visit_count"] * config["beam_size"])
    b = queries.shape[0]
    queue = Queue(b, q, q + extra)
    count = q * max(1, int(config.get("search_seed_factor", 1)))
    seeds = circulants(b, vectors.shape[0], seed_offsets(count))
    # distances of query b against the seed rows: search_from_seeds over a one-column "graph"
    ident = np.arange(vectors.shape[0], dtype=np.int32).reshape(-1, 1)
    _, d = search_from_seeds(queries, seeds, ident, vectors, metric)
    # piecewise inserts == the best q distinct (distance, id) pairs of all seeds
    for c in range(0, count, extra):
        queue.insert(seeds[:, c:c + extra], d[:, c:c + extra])
    if count > extra:   # a widened scan hands over only its best q; the columns behind start empty
        queue.indices[:, q:] = MAXINT
        queue.distances[:, q:] = MAXFLOAT
    return queue


def search(vectors, beams, queries, config: dict, metric=COSINE) -> Queue:
    """ann.py:469-477 (ANN.search)."""
    queue = initial_search_queue(vectors, queries, config, metric)
    closest_vectors(queries, queue, vectors, beams, config, None, metric)
    return queue


def self_recall(vectors, beams, config: dict, sample_size: int = 1000, metric=COSINE) -> int:
    """ann.py:235-259 / 456-464."""
    vectors, beams = _f32(vectors), _i32(beams)
    n, dim = vectors.shape
    sample = min(sample_size, n)
    pt = primes_table()
    return int(lib().vlo_self_recall(
        _p(vectors, _F), _L(n), ctypes.c_int(dim), _p(beams, _I), ctypes.c_int(beams.shape[1]), _L(sample),
        ctypes.c_int(config["beam_size"]), ctypes.c_int(config["parallel_visit_count"]),
        ctypes.c_int(config["visit_queue_factor"]), ctypes.c_int(config["exclude_factor"]),
        ctypes.c_int(config["recall_search_queue_factor"]), ctypes.c_int(config["speculative_readahead"]),
        _p(pt, _I), ctypes.c_int(metric_code(metric))))


def generate_ann(vectors, config: dict, metric=COSINE, return_full: bool = False):
    """ann.py:109-193.  Returns (beams[N,D], distances[N,D], loops_run, recall_found[, full...])."""
    vectors = _f32(vectors)
    n, dim = vectors.shape
    d = config["beam_size"]
    w = d * config["beam_queue_factor"]
    out_b = np.empty((n, d), dtype=np.int32)
    out_d = np.empty((n, d), dtype=np.float32)
    full_b = np.empty((n, w), dtype=np.int32) if return_full else None
    full_d = np.empty((n, w), dtype=np.float32) if return_full else None
    found = ctypes.c_int64(0)
    pt = primes_table()
    loops = lib().vlo_generate_ann(
        _p(vectors, _F), _L(n), ctypes.c_int(dim), ctypes.c_int(d), ctypes.c_int(config["beam_queue_factor"]),
        ctypes.c_int(config["parallel_visit_count"]), ctypes.c_int(config["visit_queue_factor"]),
        ctypes.c_int(config["exclude_factor"]), ctypes.c_int(config["optimization_loops"]),
        _L(config["batch_size"]), ctypes.c_int(config["recall_search_queue_factor"]),
        ctypes.c_int(config["speculative_readahead"]), ctypes.c_int(1 if config["prune"] else 0),
        _p(pt, _I), ctypes.c_int(metric_code(metric)), _p(out_b, _I), _p(out_d, _F), _p(full_b, _I),
        _p(full_d, _F), ctypes.byref(found))
    if return_full:
        return out_b, out_d, int(loops), int(found.value), full_b, full_d
    return out_b, out_d, int(loops), int(found.value)


def bruteforce_knn(vectors, queries, k: int, metric=COSINE, exclude_self: bool = False, self_base: int = 0):
    """Exact k nearest neighbours in double precision (ground truth for recall)."""
    vectors, queries = _f32(vectors), _f32(queries)
    n, dim = vectors.shape
    b = queries.shape[0]
    out = np.empty((b, k), dtype=np.int32)
    lib().vlo_bruteforce_knn(_p(vectors, _F), _L(n), ctypes.c_int(dim), _p(queries, _F), _L(b), ctypes.c_int(k),
                             ctypes.c_int(metric_code(metric)), ctypes.c_int(1 if exclude_self else 0),
                             _L(self_base), _p(out, _I))
    return out


def connected_components(ids, dist=None, threshold: float = MAXFLOAT):
    """(labels int32 [N], count of out-of-range ids): labels[x] = the smallest id of the connected
    component of x in the graph linking x and ids[x, s] wherever the id is real and
    dist[x, s] <= threshold.  Not in the reference (its `ANN.clusters` is a stub)."""
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    n, w = ids.shape
    d = _f32(dist) if dist is not None else None
    labels = np.empty(n, dtype=np.int32)
    bad = lib().vlo_connected_components(_p(ids, _I), _p(d, _F) if d is not None else None, _L(n), ctypes.c_int(w),
                                         ctypes.c_float(threshold), _p(labels, _I))
    return labels, int(bad)

"""The opt-in start graph from the tensor-core tile pass (csrc/vl_knn_tile.cu, knn_tile.py).

The reference has no such pass (its builds start from the circulant graph, utils.py:35-41), so
these tests check the pass against brute force and against the exact fp32 distance: what it
proposes, that the reranked lists carry exact distances in queue order, and that a build that
starts from them ends with a better graph than the circulant start after the same number of rounds."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
MAXINT = oracle.MAXINT
DEV = "cuda"


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def n(x):
    return x.cpu().numpy()


def status_clear():
    from vectorlink_gpu import _lib
    return _lib.read_status(torch.device(DEV)) == 0


def sift_like(rng, count, dim=128, centres=32):
    c = rng.uniform(0, 255, (centres, dim))
    pts = c[rng.integers(0, centres, count)] + rng.normal(0, 20, (count, dim))
    return np.round(pts).clip(0, 255).astype(np.float32)


def test_prepare_rounds_to_bf16_pads_and_sums_squares(built_lib):
    from vectorlink_gpu.knn_tile import prepare
    rng = np.random.default_rng(1)
    v = rng.standard_normal((333, 96)).astype(np.float32)
    rows, norms = prepare(t(v), want_norms=True)
    assert tuple(rows.shape) == (333, 128) and rows.dtype == torch.bfloat16
    assert torch.equal(rows[:, :96], t(v).to(torch.bfloat16)) and bool((rows[:, 96:] == 0).all())
    np.testing.assert_allclose(n(norms), (v.astype(np.float64) ** 2).sum(1), rtol=1e-5)


@pytest.mark.parametrize("count,segments,rows", [(1000, 1, (0, 1000)), (2500, 3, (300, 1700)), (130, 2, (0, 130)), (700, 2, (5, 650))])
def test_proposals_are_the_exact_top_of_every_list_on_integer_data(count, segments, rows, built_lib):
    """Integer-valued rows below 256 are exact in bf16 and their inner products are exact in the fp32
    accumulator, so every list must hold exactly the 16 nearest (squared L2, ties by id) of its
    candidates - one of the four 64-candidate quarters of every 256-candidate tile of its segment -
    the row itself left out."""
    from vectorlink_gpu.knn_tile import TILE_K, TILE_LISTS, prepare, proposals
    assert (TILE_K, TILE_LISTS) == (16, 4)
    rng = np.random.default_rng(count)
    v = sift_like(rng, count)
    rows_bf16, norms = prepare(t(v), want_norms=True)
    got = n(proposals(rows_bf16, norms, rows, (0, count), segments))
    assert status_clear()
    assert got.shape == (rows[1] - rows[0], segments * 64)
    per_segment = (count + segments - 1) // segments
    seg_len = (per_segment + 255) // 256 * 256                 # the kernel cuts the range at multiples of its tile width
    d = ((v[rows[0]:rows[1], None, :].astype(np.float64) - v[None, :, :].astype(np.float64)) ** 2).sum(2)
    d[np.arange(rows[1] - rows[0]), np.arange(rows[0], rows[1])] = np.inf
    ids = np.arange(count)
    for s in range(segments):
        lo, hi = s * seg_len, min(count, (s + 1) * seg_len)
        for cls in range(TILE_LISTS):
            part = got[:, (TILE_LISTS * s + cls) * TILE_K:(TILE_LISTS * s + cls + 1) * TILE_K]
            members = ids[(ids >= lo) & (ids < hi) & ((((ids - lo) // 64) % TILE_LISTS) == cls)]
            if len(members) == 0:
                assert (part == MAXINT).all()
                continue
            dm = d[:, members]
            order = members[np.lexsort((np.broadcast_to(members, dm.shape), dm), axis=1)[:, :TILE_K]]
            finite = np.take_along_axis(d, order, 1) < np.inf      # a short list may reach the row itself
            for r in range(got.shape[0]):
                want = order[r][finite[r]]
                assert np.array_equal(part[r, :len(want)], want), (s, cls, r)
                assert (part[r, len(want):] == MAXINT).all()


@pytest.mark.parametrize("count,dim,segments,rows,cands", [
    (5, 128, 1, (0, 5), (0, 5)),            # far less than one tile
    (40, 96, 4, (0, 40), (0, 40)),          # more segments than tiles: three of them are empty
    (300, 128, 1, (7, 8), (0, 300)),        # a single row
    (300, 200, 2, (0, 300), (100, 101)),    # a single candidate; rows streamed (padded dimension 256 > 128)
    (600, 64, 1, (250, 600), (0, 256)),     # candidates end exactly at a tile edge
])
def test_ragged_and_tiny_ranges(count, dim, segments, rows, cands, built_lib):
    """Every list holds the nearest of its class among the offered candidates, whatever the shape of the ranges."""
    from vectorlink_gpu.knn_tile import TILE_K, TILE_LISTS, prepare, proposals
    rng = np.random.default_rng(count + dim)
    v = sift_like(rng, count, dim, centres=4)
    rows_bf16, norms = prepare(t(v), want_norms=True)
    got = n(proposals(rows_bf16, norms, rows, cands, segments))
    assert status_clear()
    assert got.shape == (rows[1] - rows[0], segments * TILE_K * TILE_LISTS)
    span = cands[1] - cands[0]
    seg_len = ((span + segments - 1) // segments + 255) // 256 * 256
    d = ((v[rows[0]:rows[1], None, :].astype(np.float64) - v[None, :, :].astype(np.float64)) ** 2).sum(2)
    d[np.arange(rows[1] - rows[0]), np.arange(rows[0], rows[1])] = np.inf
    ids = np.arange(count)
    for s in range(segments):
        lo, hi = cands[0] + s * seg_len, min(cands[1], cands[0] + (s + 1) * seg_len)
        for cls in range(TILE_LISTS):
            part = got[:, (TILE_LISTS * s + cls) * TILE_K:(TILE_LISTS * s + cls + 1) * TILE_K]
            members = ids[(ids >= lo) & (ids < hi) & ((((ids - lo) // 64) % TILE_LISTS) == cls)]
            for r in range(got.shape[0]):
                dm = d[r, members]
                order = members[np.lexsort((members, dm))][:TILE_K]
                want = order[d[r, order] < np.inf]
                assert np.array_equal(part[r, :len(want)], want), (s, cls, r)
                assert (part[r, len(want):] == MAXINT).all()


@pytest.mark.parametrize("dim,metric", [(96, "cosine"), (768, "cosine"), (1024, "cosine"), (128, "l2")])
def test_start_graph_lists_are_exact_and_cover_the_true_neighbours(dim, metric, built_lib):
    """Unit-norm float rows: the bf16 scores are approximate, the lists are not - every stored
    distance equals the oracle's fp32 distance of that pair, rows are in (distance, id) order with
    unique ids and no self link, and the 10 true nearest neighbours are (almost) all there."""
    from vectorlink_gpu.knn_tile import knn_start_graph
    rng = np.random.default_rng(dim)
    count, width = 3000, 48
    if metric == "l2":
        v = sift_like(rng, count, dim)
    else:
        c = rng.standard_normal((30, dim))
        v = c[rng.integers(0, 30, count)] + 0.3 * rng.standard_normal((count, dim))
        v = (v / np.linalg.norm(v, axis=1, keepdims=True)).astype(np.float32)
    config = {"metric": metric}
    ids, dist = knn_start_graph(t(v), width, config)
    assert status_clear()
    ids, dist = n(ids), n(dist)
    assert ids.shape == (count, width) and ids.dtype == np.int32
    assert np.array_equal(oracle.calculate_distances(v, ids, metric=metric), dist)
    real = ids != MAXINT
    assert real.sum(1).min() >= 32
    assert np.all(np.diff(dist, axis=1) >= 0)
    srt = np.sort(ids, axis=1)
    assert not np.any((srt[:, 1:] == srt[:, :-1]) & (srt[:, 1:] != MAXINT))
    assert not np.any(ids == np.arange(count)[:, None])
    truth = oracle.bruteforce_knn(v, v[:400], 10, metric=metric, exclude_self=True)
    hit = np.mean([len(set(ids[r]) & set(truth[r])) / 10 for r in range(400)])
    assert hit >= 0.97, hit


def test_build_from_the_tile_pass_beats_the_circulant_start(built_lib):
    """Config-3-shaped rows (768-d unit vectors around many centres): after ONE optimisation round the
    graph that started from the tile pass has the higher recall@10 against brute force, and the default
    (`init="circulant"`) is untouched by the option."""
    from vectorlink_gpu import ANN
    rng = np.random.default_rng(3)
    count, dim = 6000, 768
    c = rng.standard_normal((100, dim))
    c /= np.linalg.norm(c, axis=1, keepdims=True)
    v = c[rng.integers(0, 100, count)] + 0.1 * rng.standard_normal((count, dim))
    v = (v / np.linalg.norm(v, axis=1, keepdims=True)).astype(np.float32)
    kw = dict(beam_size=16, visit_queue_factor=2, recall_search_queue_factor=2, optimization_loops=1)
    plain = ANN(t(v), **kw)
    again = ANN(t(v), init="circulant", **kw)
    assert torch.equal(plain.beams, again.beams) and "init" not in plain.configuration
    tiled = ANN(t(v), init="knn_tile", **kw)
    assert status_clear()
    truth = oracle.bruteforce_knn(v, v[:500], 10, exclude_self=True)

    def recall(ann):
        b = n(ann.beams[:500, :10])
        return np.mean([len(set(b[r]) & set(truth[r])) / 10 for r in range(500)])

    r_plain, r_tiled = recall(plain), recall(tiled)
    assert r_tiled > r_plain and r_tiled >= 0.9, (r_plain, r_tiled)
    assert np.array_equal(oracle.calculate_distances(v, n(tiled.beams)), n(tiled.distances))


def test_search_from_tensor_core_entry_points_vs_oracle_and_recall(built_lib):
    """`search_entry_sample`: the entry points come from the tile pass, everything after that is the
    reference's search - bit for bit the oracle's queue when it starts from the same seeds - and on
    clustered rows the queries now reach their cluster, which the circulant seeds rarely do."""
    from vectorlink_gpu import ANN
    from vectorlink_gpu.ann import query_distances
    rng = np.random.default_rng(12)
    count, dim = 12000, 64
    c = rng.standard_normal((300, dim)) * 3
    v = (c[rng.integers(0, 300, count)] + 0.3 * rng.standard_normal((count, dim))).astype(np.float32)
    v = (v / np.linalg.norm(v, axis=1, keepdims=True)).astype(np.float32)
    q = (c[rng.integers(0, 300, 200)] + 0.3 * rng.standard_normal((200, dim))).astype(np.float32)
    q = (q / np.linalg.norm(q, axis=1, keepdims=True)).astype(np.float32)
    kw = dict(beam_size=16, visit_queue_factor=2, recall_search_queue_factor=2)
    kn = oracle.bruteforce_knn(v, v, 16, exclude_self=True)
    kd = oracle.calculate_distances(v, kn)
    plain = ANN(t(v), beams=t(kn), distances=t(kd), **kw)
    tiled = ANN(t(v), beams=t(kn), distances=t(kd), search_entry_sample=4096, **kw)
    sq = tiled.search(t(q))
    assert status_clear()
    seeds = tiled._entry_seeds(t(q))
    assert tuple(seeds.shape) == (200, 64) and int(seeds.max()) < count
    sd = query_distances(t(q), t(v), seeds)
    cfg = oracle.make_config(**kw)
    oq = oracle.Queue(200, sq.length, sq.indices.size(1))
    oq.insert(n(seeds), n(sd))
    oracle.closest_vectors(q, oq, v, kn, cfg)
    assert np.array_equal(n(sq.indices), oq.indices) and np.array_equal(n(sq.distances), oq.distances)
    truth = oracle.bruteforce_knn(v, q, 10)

    def recall(queue):
        got = n(queue.indices[:, :10])
        return np.mean([len(set(got[i]) & set(truth[i])) / 10 for i in range(200)])

    r_plain, r_tiled = recall(plain.search(t(q))), recall(sq)
    assert r_tiled >= 0.95 and r_tiled > r_plain + 0.2, (r_plain, r_tiled)

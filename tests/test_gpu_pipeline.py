"""End-to-end parity of the drop-in API on the GPU: fused beam search, graph build, search,
against the reference's host-code fixtures, the CPU oracle and brute-force ground truth."""
import numpy as np
import pytest
import torch

import oracle
from conftest import assert_rows_match, cfg_of

pytestmark = pytest.mark.gpu
MAXINT = oracle.MAXINT
DEV = "cuda"


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def n(x):
    return x.cpu().numpy()


def unit(rng, rows, dim):
    v = rng.standard_normal((rows, dim)).astype(np.float32)
    return (v / np.linalg.norm(v, axis=1, keepdims=True)).astype(np.float32)


def gpu_queue_from(oq):
    from vectorlink_gpu.queue import Queue
    q = Queue(oq.indices.shape[0], oq.length, oq.indices.shape[1], device=DEV)
    q.indices.copy_(t(oq.indices))
    q.distances.copy_(t(oq.distances))
    return q


@pytest.mark.parametrize("which", ["c1", "small"])
@pytest.mark.parametrize("mode", ["fused", "stepwise"])
def test_search_vs_reference_host_code(which, mode, c1, small, built_lib):
    from vectorlink_gpu import ANN
    g = c1 if which == "c1" else small
    _, kw = cfg_of(g)
    ann = ANN(t(g["vectors"]), beams=t(g["beams"]), distances=t(g["distances"]), **kw)
    if mode == "stepwise":
        ann.configuration["stepwise"] = True
    sq = ann.search(t(g["queries"]))
    assert sq.length == int(g["search_length"]) and tuple(sq.indices.shape) == g["search_ids"].shape
    assert sq.indices.dtype == torch.int32 and sq.distances.dtype == torch.float32
    # the reference with kernel-order seed distances: bit for bit
    assert np.array_equal(n(sq.indices), g["search_tree_ids"])
    assert np.array_equal(n(sq.distances), g["search_tree_dist"])
    # the reference exactly as shipped: 1e-5 relative on distances, ids equal up to ties
    assert_rows_match(n(sq.indices), n(sq.distances), g["search_ids"], g["search_dist"], 1e-5, "search")
    one = ann.search(t(g["queries"][:1]))
    assert_rows_match(n(one.indices), n(one.distances), g["search1_ids"], g["search1_dist"], 1e-5, "single query")


@pytest.mark.parametrize("which", ["c1", "small"])
@pytest.mark.parametrize("mode", ["fused", "stepwise"])
def test_build_vs_reference_host_code(which, mode, c1, small, built_lib):
    from vectorlink_gpu.ann import generate_ann
    g = c1 if which == "c1" else small
    cfg, kw = cfg_of(g)
    cfg = dict(cfg)
    if mode == "stepwise":
        cfg["stepwise"] = True
    beams, dist = generate_ann(t(g["vectors"]), cfg)
    assert np.array_equal(n(beams), g["beams"])
    assert np.array_equal(n(dist), g["distances"])
    assert generate_ann.last_loops == 1


@pytest.mark.parametrize("mode", ["fused", "stepwise"])
def test_multi_round_build_vs_patched_reference(mode, multi, built_lib):
    """Three rounds of the reference's host code (repaired at the two accidental spots the fixture's
    generator names): rounds that start from pruned lists with MAXINT tails and carried distances."""
    from vectorlink_gpu.ann import generate_ann
    cfg, _ = cfg_of(multi)
    cfg = dict(cfg)
    if mode == "stepwise":
        cfg["stepwise"] = True
    beams, dist = generate_ann(t(multi["vectors"]), cfg)
    assert generate_ann.last_loops == int(multi["loops"]) == 3
    assert np.array_equal(n(beams), multi["beams"]) and np.array_equal(n(dist), multi["distances"])


def test_ann_constructor_is_a_drop_in(c1, built_lib):
    from vectorlink_gpu import ANN
    _, kw = cfg_of(c1)
    ann = ANN(vectors=t(c1["vectors"]), **kw)
    assert np.array_equal(n(ann.beams), c1["beams"]) and np.array_equal(n(ann.distances), c1["distances"])
    assert ann.beams.dtype == torch.int32 and ann.distances.dtype == torch.float32
    found, ratio = ann.recall()
    assert found == int(c1["self_recall_found"]) and ratio == found / 1000
    for key in ("prune", "beam_size", "parallel_visit_count", "beam_queue_factor", "visit_queue_factor",
                "exclude_factor", "optimization_loops", "batch_size", "recall_search_queue_factor",
                "speculative_readahead"):
        assert key in ann.configuration
    assert ann.log["vector_count"] == 2000 and ann.log["vector_dimension"] == 64 and ann.log["total_time"] > 0
    clusters = ann.clusters()
    assert tuple(clusters.indices.shape) == (2000, 32 + 64) and clusters.length == 32
    assert (n(clusters.indices[:, 0]) == np.arange(2000)).mean() > 0.99


def closest_both(vectors, beams, queries, oq, cfg, exclude=None, metric="cosine", stepwise=False, memo=True,
                 row_ticket=True):
    from vectorlink_gpu.ann import closest_vectors
    gq = gpu_queue_from(oq)
    config = dict(cfg)
    if not memo:
        config["memo"] = False
    if not row_ticket:
        config["row_ticket"] = False
    if metric != "cosine":
        config["metric"] = metric
    if stepwise:
        config["stepwise"] = True
    closest_vectors(t(queries), gq, t(vectors), t(beams), config, t(exclude) if exclude is not None else None)
    count = oracle.closest_vectors(queries, oq, vectors, beams, cfg, exclude, metric)
    return gq, oq, closest_vectors.last_count, count


CASES = [
    # name, N, dim, D, graph width, batch, cfg overrides
    ("default-search", 3000, 32, 24, 24, 64, {}),
    ("wide-build-queue", 1500, 48, 8, 24, 200, {}),
    ("pvc1", 1200, 16, 8, 8, 33, {"parallel_visit_count": 1}),
    ("readahead-hits-k_none", 1200, 16, 6, 6, 40, {"visit_queue_factor": 1, "exclude_factor": 6}),
    ("seen-not-multiple-of-pvc", 1200, 24, 7, 7, 20, {"parallel_visit_count": 3, "exclude_factor": 5}),
    ("no-seen-list", 800, 16, 8, 8, 10, {"exclude_factor": 0}),
    ("dim256", 500, 256, 8, 8, 7, {}),
    ("dim384", 400, 384, 8, 8, 6, {}),
    ("dim512", 400, 512, 8, 8, 6, {}),
    ("dim768", 300, 768, 8, 8, 5, {}),
    ("dim1024", 400, 1024, 8, 8, 6, {}),
    ("dim1536", 300, 1536, 8, 8, 4, {}),
]


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
@pytest.mark.parametrize("metric", ["cosine", "l2"])
def test_fused_closest_vectors_vs_oracle(case, metric, built_lib):
    name, nvec, dim, d, w, batch, over = case
    rng = np.random.default_rng(len(name) * 100 + dim)
    vectors = unit(rng, nvec, dim)
    if metric == "l2":
        vectors = np.round(vectors * 40 + 128).clip(0, 255).astype(np.float32)   # integer-valued: exact ties occur
    cfg = oracle.make_config(beam_size=d, **over)
    # a graph of near neighbours with some sentinels, so that the search has structure
    kn = oracle.bruteforce_knn(vectors, vectors, w, metric=metric, exclude_self=True)
    kn[rng.random(kn.shape) < 0.03] = MAXINT
    queries = vectors[:batch] if name == "wide-build-queue" else (
        unit(rng, batch, dim) if metric == "cosine" else np.round(unit(rng, batch, dim) * 40 + 128).astype(np.float32))
    if name == "wide-build-queue":            # the build's queue: seeded with the row's own list, self excluded
        seeds = oracle.circulants(batch, nvec, oracle.primes_table(w))
        sd = oracle.calculate_distances(vectors, np.vstack([seeds, np.zeros((nvec - batch, w), np.int32)]), metric=metric)[:batch]
        oq = oracle.Queue(batch, w, w + w * cfg["parallel_visit_count"])
        oq.insert(seeds, sd)
        exclude = np.arange(batch, dtype=np.int32).reshape(-1, 1)
    else:
        oq = oracle.initial_search_queue(vectors, queries, cfg, metric)
        exclude = None
    gq, oq, gcount, ocount = closest_both(vectors, kn, queries, oq, cfg, exclude, metric)
    assert gcount == ocount
    assert np.array_equal(n(gq.indices), oq.indices)
    assert np.array_equal(n(gq.distances), oq.distances)


def test_distance_memo_changes_nothing(built_lib):
    """The fused kernel's id -> distance memo only skips gathers of ids it has already met."""
    rng = np.random.default_rng(31)
    vectors = unit(rng, 4000, 64)
    cfg = oracle.make_config(beam_size=16, visit_queue_factor=2, recall_search_queue_factor=2)
    kn = oracle.bruteforce_knn(vectors, vectors, 16, exclude_self=True)
    queries = unit(rng, 50, 64)
    results = []
    for memo in (True, False):
        oq = oracle.initial_search_queue(vectors, queries, cfg)
        gq, oq, gcount, ocount = closest_both(vectors, kn, queries, oq, cfg, memo=memo)
        assert gcount == ocount
        assert np.array_equal(n(gq.indices), oq.indices) and np.array_equal(n(gq.distances), oq.distances)
        results.append(n(gq.indices))
    assert np.array_equal(results[0], results[1])


def test_memo_decision_of_the_build_changes_nothing(built_lib):
    """generate_ann switches the memo off for later rounds when its self-recall check gathered nearly
    every candidate; whichever way it decides, the graph equals the one built with the memo forced
    on or off."""
    from vectorlink_gpu.ann import generate_ann
    rng = np.random.default_rng(91)
    vectors = t(unit(rng, 5000, 32))
    cfg = oracle.make_config(beam_size=8, batch_size=1000)
    graphs = []
    for extra in ({}, {"memo": True}, {"memo": False}):
        b, d = generate_ann(vectors, dict(cfg, **extra))
        assert isinstance(generate_ann.memo_useful, bool)
        graphs.append((n(b), n(d)))
    for b, d in graphs[1:]:
        assert np.array_equal(b, graphs[0][0]) and np.array_equal(d, graphs[0][1])


def test_row_schedule_changes_nothing(built_lib):
    """More rows than the launch keeps in flight: warps that draw their next row from the shared
    counter and warps on a fixed stride produce the same queues, equal to the oracle's."""
    rng = np.random.default_rng(77)
    vectors = unit(rng, 3000, 32)
    cfg = oracle.make_config(beam_size=8, visit_queue_factor=2, recall_search_queue_factor=2, batch_size=20_000)
    kn = oracle.bruteforce_knn(vectors, vectors, 8, exclude_self=True)
    queries = unit(rng, 9000, 32)
    results = []
    for ticket in (True, False):
        oq = oracle.initial_search_queue(vectors, queries, cfg)
        gq, oq, gcount, ocount = closest_both(vectors, kn, queries, oq, cfg, row_ticket=ticket)
        assert gcount == ocount
        assert np.array_equal(n(gq.indices), oq.indices) and np.array_equal(n(gq.distances), oq.distances)
        results.append(n(gq.indices))
    assert np.array_equal(results[0], results[1])


@pytest.mark.parametrize("batch", [1, 2, 5])
def test_small_batches_stop_where_the_reference_stops(batch, built_lib):
    """With few rows the reference's batch-wide "nothing changed" check ends the loop early;
    the fused path must notice and reproduce the queue of that iteration, tail included."""
    rng = np.random.default_rng(99 + batch)
    vectors = unit(rng, 5000, 16)
    cfg = oracle.make_config(beam_size=8)
    kn = oracle.bruteforce_knn(vectors, vectors, 8, exclude_self=True)
    early = 0
    for trial in range(6):
        queries = unit(rng, batch, 16)
        oq = oracle.initial_search_queue(vectors, queries, cfg)
        gq, oq, gcount, ocount = closest_both(vectors, kn, queries, oq, cfg)
        assert gcount == ocount
        assert np.array_equal(n(gq.indices), oq.indices) and np.array_equal(n(gq.distances), oq.distances)
        early += ocount < 35
    assert early > 0        # the case under test did occur


def test_dry_visit_queues_take_the_stepwise_route(built_lib):
    """A graph so small that every row's visit queue runs out: the seen list then fills more
    slowly than the budgeted schedule assumes, and the result must still be the reference's."""
    rng = np.random.default_rng(5)
    vectors = unit(rng, 40, 8)
    cfg = oracle.make_config(beam_size=4, visit_queue_factor=2, exclude_factor=8)
    kn = oracle.bruteforce_knn(vectors, vectors, 4, exclude_self=True)
    queries = unit(rng, 3, 8)
    oq = oracle.initial_search_queue(vectors, queries, cfg)
    gq, oq, gcount, ocount = closest_both(vectors, kn, queries, oq, cfg)
    assert gcount == ocount
    assert np.array_equal(n(gq.indices), oq.indices) and np.array_equal(n(gq.distances), oq.distances)


def test_stale_tail_queue_shape_uses_operator_path(built_lib):
    """recall_search_queue_factor > parallel_visit_count leaves columns behind the candidates
    that survive from insert to insert (queue.py:47-55); only the operator path models that."""
    rng = np.random.default_rng(6)
    vectors = unit(rng, 900, 16)
    cfg = oracle.make_config(beam_size=6, recall_search_queue_factor=6, parallel_visit_count=3)
    kn = oracle.bruteforce_knn(vectors, vectors, 6, exclude_self=True)
    queries = unit(rng, 7, 16)
    oq = oracle.initial_search_queue(vectors, queries, cfg)
    gq, oq, gcount, ocount = closest_both(vectors, kn, queries, oq, cfg)
    assert gcount == ocount
    assert np.array_equal(n(gq.indices), oq.indices) and np.array_equal(n(gq.distances), oq.distances)


@pytest.mark.parametrize("metric,dim", [("l2", 128), ("cosine", 96)])
def test_multi_loop_build_vs_oracle(metric, dim, built_lib):
    """Clustered data where one round does not reach self-recall 1.0: later rounds start
    from pruned lists that carry sentinels."""
    from vectorlink_gpu.ann import generate_ann
    rng = np.random.default_rng(17)
    centres = rng.uniform(0, 255, (8, dim))
    pts = centres[rng.integers(0, 8, 1500)] + rng.normal(0, 20, (1500, dim))
    vectors = np.round(pts).clip(0, 255).astype(np.float32)
    if metric == "cosine":
        vectors = (vectors / np.linalg.norm(vectors, axis=1, keepdims=True)).astype(np.float32)
    cfg = oracle.make_config(beam_size=8, visit_queue_factor=2, recall_search_queue_factor=2, batch_size=400,
                             optimization_loops=2)
    wb, wd, loops, found, fb, fd = oracle.generate_ann(vectors, cfg, metric=metric, return_full=True)
    config = dict(cfg)
    config["metric"] = metric
    gb, gd = generate_ann(t(vectors), config)
    assert generate_ann.last_loops == loops
    assert np.array_equal(n(gb), wb) and np.array_equal(n(gd), wd)


def test_graph_and_search_recall_against_brute_force(built_lib):
    """Quality gate: recall@10 of .search and of the graph itself, on SIFT-like synthetic data."""
    from vectorlink_gpu import ANN
    rng = np.random.default_rng(0)
    dim, nvec = 128, 20000
    centres = rng.uniform(0, 255, (64, dim))
    vectors = np.round(centres[rng.integers(0, 64, nvec)] + rng.normal(0, 20, (nvec, dim))).clip(0, 255).astype(np.float32)
    queries = np.round(centres[rng.integers(0, 64, 200)] + rng.normal(0, 20, (200, dim))).clip(0, 255).astype(np.float32)
    kw = dict(beam_size=32, visit_queue_factor=2, recall_search_queue_factor=2, search_seed_factor=20)
    ann = ANN(t(vectors), metric="l2", **kw)
    sq = ann.search(t(queries))
    # the widened seed scan is the oracle's too, bit for bit
    osq = oracle.search(vectors, n(ann.beams), queries, oracle.make_config(**kw), metric="l2")
    assert np.array_equal(n(sq.indices), osq.indices) and np.array_equal(n(sq.distances), osq.distances)
    truth = oracle.bruteforce_knn(vectors, queries, 10, metric="l2")
    got = n(sq.indices[:, :10])
    recall = np.mean([len(set(got[i]) & set(truth[i])) / 10 for i in range(200)])
    assert recall >= 0.95, recall
    gtruth = oracle.bruteforce_knn(vectors, vectors[:300], 10, metric="l2", exclude_self=True)
    gb = n(ann.beams[:300, :10])
    grecall = np.mean([len(set(gb[i]) & set(gtruth[i])) / 10 for i in range(300)])
    assert grecall >= 0.9, grecall
    d = n(ann.distances)
    assert np.all(np.diff(d, axis=1) >= 0)                      # rows sorted by distance
    b = n(ann.beams)
    assert all(len(set(r[r != MAXINT])) == (r != MAXINT).sum() for r in b[:500])   # ids unique


def test_full_size_properties_config2_slice(built_lib):
    """Size-independent properties at the benchmark's dimension and degree on a 200k slice:
    sorted rows, unique ids, no self loops, distances equal to a recomputation."""
    from vectorlink_gpu import ANN
    from vectorlink_gpu.kernels import calculate_distances
    g = torch.Generator(device=DEV).manual_seed(0)
    centres = torch.rand((256, 128), device=DEV, generator=g) * 255
    assign = torch.randint(0, 256, (200_000,), device=DEV, generator=g)
    vectors = (centres[assign] + 20 * torch.randn((200_000, 128), device=DEV, generator=g)).round().clamp(0, 255)
    ann = ANN(vectors, beam_size=32, visit_queue_factor=2, recall_search_queue_factor=2, metric="l2",
              optimization_loops=1)
    b, d = ann.beams, ann.distances
    assert tuple(b.shape) == (200_000, 32)
    assert bool((d[:, 1:] >= d[:, :-1]).all())
    assert bool((b != torch.arange(200_000, device=DEV, dtype=torch.int32).unsqueeze(1)).all())
    srt = b.sort(dim=1).values
    assert bool(((srt[:, 1:] != srt[:, :-1]) | (srt[:, 1:] == MAXINT)).all())
    assert torch.equal(calculate_distances(vectors, b, metric="l2"), d)


def test_layered_search_and_recall_helpers(c1, built_lib):
    """search_layers / hnsw_calculate_recall (ann.py:96-106, 262-284) over a one-layer list equal
    the flat self-recall; ann_calculate_recall on the fixture graph finds every sampled row."""
    from vectorlink_gpu.ann import ann_calculate_recall, hnsw_calculate_recall
    cfg, _ = cfg_of(c1)
    v, b = t(c1["vectors"]), t(c1["beams"])
    flat = ann_calculate_recall(v, b, cfg, sample=v[:500])
    layered = hnsw_calculate_recall(v, [b], cfg, sample=v[:500])
    assert flat == layered and flat[0] == oracle.self_recall(c1["vectors"], c1["beams"], cfg, 500)


@pytest.mark.parametrize("batch_size", [1, 3, 50])
def test_build_with_tiny_batches_follows_the_reference_batch_coupling(batch_size, built_lib):
    """With batches of a few rows the reference's per-batch early exit happens inside the build;
    the single-launch build must repair exactly those batches."""
    from vectorlink_gpu.ann import generate_ann
    rng = np.random.default_rng(123)
    vectors = unit(rng, 240, 24)
    cfg = oracle.make_config(beam_size=6, batch_size=batch_size, optimization_loops=2)
    wb, wd, loops, found = oracle.generate_ann(vectors, cfg)
    gb, gd = generate_ann(t(vectors), dict(cfg))
    assert generate_ann.last_loops == loops
    assert np.array_equal(n(gb), wb) and np.array_equal(n(gd), wd)


# ---- the benchmark configurations' own queue shapes, bit for bit against the oracle ----------

def sift_like(rng, count, dim=128, centres=256):
    """Config-2 recipe: centres uniform in [0,255], point = centre + N(0, 20^2), rounded, clipped."""
    c = rng.uniform(0, 255, (centres, dim))
    pts = c[rng.integers(0, centres, count)] + rng.normal(0, 20, (count, dim))
    return np.round(pts).clip(0, 255).astype(np.float32)


def embed_like(rng, count, dim, centres, noise, unit_centres=True):
    """Config-3/5 recipe: centres N(0,1) (normalised for config 3), point = centre + N(0, noise^2)
    per dimension, renormalised."""
    c = rng.standard_normal((centres, dim))
    if unit_centres:
        c /= np.linalg.norm(c, axis=1, keepdims=True)
    pts = c[rng.integers(0, centres, count)] + noise * rng.standard_normal((count, dim))
    return (pts / np.linalg.norm(pts, axis=1, keepdims=True)).astype(np.float32)


def build_both(vectors, kw, metric, variants):
    """generate_ann on the GPU under every config variant against one oracle build."""
    from vectorlink_gpu.ann import generate_ann
    cfg = oracle.make_config(**kw)
    wb, wd, loops, found = oracle.generate_ann(vectors, cfg, metric=metric)
    tv = t(vectors)
    for extra in variants:
        config = dict(cfg, **extra)
        config["metric"] = metric
        gb, gd = generate_ann(tv, config)
        assert generate_ann.last_loops == loops, (extra, generate_ann.last_loops, loops)
        assert np.array_equal(n(gb), wb), f"{extra}: neighbour ids differ from the oracle"
        assert np.array_equal(n(gd), wd), f"{extra}: distances differ from the oracle"
    return wb, wd, loops


@pytest.mark.parametrize("batch_size", [10_000, 7_000])
def test_config2_shaped_build_and_search_vs_oracle(batch_size, built_lib):
    """Config 2's build shape (128-d, L2, degree 32, beam 64: graph width 96, 384 candidates per
    iteration, search queue 96, visit queue 64, seen list 320) on a 20,000-vector draw, three rounds,
    one batch per 10,000 rows and a split into three uneven batches; distance memo on, off and as the
    build decides.  Then `.search` over that graph with the reference's 64 seeds and the widened scan."""
    from vectorlink_gpu import ANN
    rng = np.random.default_rng(2)
    vectors = sift_like(rng, 20_000)
    queries = sift_like(rng, 300)
    kw = dict(beam_size=32, visit_queue_factor=2, recall_search_queue_factor=2, batch_size=batch_size)
    wb, wd, loops = build_both(vectors, kw, "l2", [{}, {"memo": True}, {"memo": False}])
    assert loops >= 2                                    # later rounds (memo, MAXINT tails) did run
    for seed_factor in (1, 30):
        skw = dict(kw, search_seed_factor=seed_factor) if seed_factor > 1 else kw
        ann = ANN(t(vectors), beams=t(wb), distances=t(wd), metric="l2", **skw)
        sq = ann.search(t(queries))
        osq = oracle.search(vectors, wb, queries, oracle.make_config(**skw), metric="l2")
        assert np.array_equal(n(sq.indices), osq.indices) and np.array_equal(n(sq.distances), osq.distances)


@pytest.mark.parametrize("dim,count", [(768, 4000), (1024, 3000)])
def test_config3_and_5_shaped_build_and_search_vs_oracle(dim, count, built_lib):
    """Configs 3 and 5: 768-d / 1024-d unit vectors, cosine, degree 64, beam 128 - graph width 192,
    768 candidates per iteration, search queue 192, visit queue 128, seen list 640, and the lane
    layout that keeps the query in shared memory.  Two rounds; memo on and off."""
    from vectorlink_gpu import ANN
    rng = np.random.default_rng(dim)
    vectors = embed_like(rng, count, dim, 40, 0.1 if dim == 768 else 0.05, unit_centres=(dim == 768))
    queries = embed_like(rng, 64, dim, 40, 0.1 if dim == 768 else 0.05, unit_centres=(dim == 768))
    vectors[1:40:8] = vectors[0:39:8]      # exact duplicates among the sampled rows: the self-recall check cannot
    #                                        reach 1.0 (the copy with the smaller id wins the tie), so round two runs
    kw = dict(beam_size=64, visit_queue_factor=2, recall_search_queue_factor=2, optimization_loops=2, batch_size=1500)
    wb, wd, loops = build_both(vectors, kw, "cosine", [{"memo": True}, {"memo": False}])
    assert loops == 2
    ann = ANN(t(vectors), beams=t(wb), distances=t(wd), **kw)
    sq = ann.search(t(queries))
    osq = oracle.search(vectors, wb, queries, oracle.make_config(**kw))
    assert np.array_equal(n(sq.indices), osq.indices) and np.array_equal(n(sq.distances), osq.distances)


def test_experiment_runner_and_grid_search_write_logs(tmp_path, built_lib):
    """The reference's runner (main.py) and its grid_search (ann.py:323-353) over the drop-in: a JSON
    log per experiment carrying the build parameters, the timing and the self-recall."""
    import importlib.util
    import json
    import os
    from conftest import PKG_ROOT
    from vectorlink_gpu.ann import grid_search
    spec = importlib.util.spec_from_file_location("vl_runner", os.path.join(PKG_ROOT, "main.py"))
    runner = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(runner)
    path = runner.main(["-c", "1500", "-d", "64", "-n", "8", "-P", "-p", "4", "-r", "2", "-q", "2", "--seed", "1",
                        "--log-dir", str(tmp_path / "log")])
    log = json.load(open(path))
    for key in ("prune", "beam_size", "parallel_visit_count", "total_time", "vector_count", "vector_dimension", "recall"):
        assert key in log
    assert log["vector_count"] == 1500 and log["vector_dimension"] == 64 and log["recall"] > 0.9
    rng = np.random.default_rng(4)
    logs = grid_search(t(unit(rng, 800, 32)), grid={"prune": [True, False], "beam_size": [6, 8]},
                       base={"visit_queue_factor": 2, "recall_search_queue_factor": 2}, log_dir=str(tmp_path / "grid"))
    assert len(logs) == 4 and len(os.listdir(tmp_path / "grid")) == 4
    assert {(l["prune"], l["beam_size"]) for l in logs} == {(True, 6), (True, 8), (False, 6), (False, 8)}

"""Operator-level parity of the CUDA kernels (through the C ABI) against the reference's
simulated kernels (fixtures) and the CPU oracle.  Integer and index results must be equal;
distances are expected bit-equal (same summation tree), which is stricter than the 1e-5
relative tolerance the drop-in promises."""
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


def unit(rng, rows, dim):
    v = rng.standard_normal((rows, dim)).astype(np.float32)
    return (v / np.linalg.norm(v, axis=1, keepdims=True)).astype(np.float32)


@pytest.mark.parametrize("dim", [64, 96, 128, 768, 1024, 1536])
def test_calculate_distances_vs_simulated_reference(kat, built_lib, dim):
    from vectorlink_gpu.kernels import calculate_distances
    d = calculate_distances(t(kat[f"k4_{dim}_vectors"]), t(kat[f"k4_{dim}_beams"]))
    assert np.array_equal(n(d), kat[f"k4_{dim}_out"])


@pytest.mark.parametrize("dim", [1024, 1536])
def test_search_from_seeds_vs_simulated_reference(kat, built_lib, dim):
    from vectorlink_gpu.kernels import search_from_seeds
    i, d = search_from_seeds(t(kat[f"k5_{dim}_queries"]), t(kat[f"k5_{dim}_visit"]), t(kat[f"k5_{dim}_beams"]),
                             t(kat[f"k5_{dim}_vectors"]))
    assert np.array_equal(n(i), kat[f"k5_{dim}_idx"])
    assert np.array_equal(n(d), kat[f"k5_{dim}_dist"])


@pytest.mark.parametrize("dim", [4, 8, 20, 33, 40, 64, 100, 128, 200, 256, 384, 512, 768, 1000, 1024, 1028, 2048, 2500])
@pytest.mark.parametrize("metric", ["cosine", "l2"])
def test_distance_tree_bit_exact_over_dimensions(built_lib, dim, metric):
    """Every lane layout (8x1 ... 32x8), unaligned dims and dims past 1024."""
    from vectorlink_gpu.kernels import calculate_distances, search_from_seeds
    rng = np.random.default_rng(dim)
    rows, w = 37, 9
    v = unit(rng, rows, dim) if metric == "cosine" else rng.integers(0, 256, (rows, dim)).astype(np.float32)
    beams = rng.integers(0, rows, (rows, w)).astype(np.int32)
    beams[rng.random((rows, w)) < 0.1] = MAXINT
    want = oracle.calculate_distances(v, beams, metric=metric)
    got = n(calculate_distances(t(v), t(beams), metric=metric))
    assert np.array_equal(got, want)
    q = unit(rng, 5, dim) if metric == "cosine" else rng.integers(0, 256, (5, dim)).astype(np.float32)
    visit = rng.integers(0, rows, (5, 3)).astype(np.int32)
    visit[1, 1] = MAXINT
    wi, wd = oracle.search_from_seeds(q, visit, beams, v, metric=metric)
    gi, gd = search_from_seeds(t(q), t(visit), t(beams), t(v), metric=metric)
    assert np.array_equal(n(gi), wi) and np.array_equal(n(gd), wd)


def test_empty_and_ragged_shapes(built_lib):
    from vectorlink_gpu.kernels import calculate_distances, search_from_seeds
    rng = np.random.default_rng(3)
    v = unit(rng, 10, 16)
    d = calculate_distances(t(v), torch.empty((10, 0), dtype=torch.int32, device=DEV))
    assert d.shape == (10, 0)
    i, d = search_from_seeds(t(v[:0]), torch.empty((0, 4), dtype=torch.int32, device=DEV),
                             t(np.zeros((10, 3), np.int32)), t(v))
    assert i.shape == (0, 12) and d.shape == (0, 12)


def test_bad_id_is_reported_not_dereferenced(built_lib):
    from vectorlink_gpu import _lib
    from vectorlink_gpu.kernels import calculate_distances
    rng = np.random.default_rng(4)
    v = unit(rng, 6, 16)
    beams = np.array([[1, 99, 2]] * 6, dtype=np.int32)      # 99 is outside [0, 6)
    _lib.read_status(DEV)
    d = n(calculate_distances(t(v), t(beams)))
    assert _lib.read_status(DEV) & 1
    assert np.all(d[:, 1] == oracle.MAXFLOAT)
    assert _lib.read_status(DEV) == 0


def test_queue_operator_trace_vs_reference_host_code(c1, built_lib):
    from vectorlink_gpu.queue import Queue
    q = Queue(6, 12, 28, device=DEV)
    q.insert(t(c1["op_ins0_ids"]), t(c1["op_ins0_dist"]))
    assert np.array_equal(n(q.indices), c1["op_q0_ids"]) and np.array_equal(n(q.distances), c1["op_q0_dist"])
    popped = q.pop_n_ids(3)
    assert np.array_equal(n(popped), c1["op_pop_ids"])
    assert np.array_equal(n(q.indices), c1["op_q1_ids"]) and np.array_equal(n(q.distances), c1["op_q1_dist"])
    changed = q.insert(t(c1["op_ins1_ids"]), t(c1["op_ins1_dist"]), exclude=t(c1["op_ins1_excl"]), output_update=True)
    assert np.array_equal(n(q.indices), c1["op_q2_ids"]) and np.array_equal(n(q.distances), c1["op_q2_dist"])
    assert np.array_equal(n(changed), c1["op_q2_changed"])


@pytest.mark.parametrize("cap,length,m", [(28, 12, 16), (480, 96, 384), (960, 192, 768), (33, 1, 32), (2, 1, 1),
                                          (4096, 1000, 3096), (64, 32, 0)])
def test_queue_insert_random_vs_oracle(built_lib, cap, length, m):
    from vectorlink_gpu.queue import Queue
    rng = np.random.default_rng(cap)
    b = 17
    universe = max(4, m // 2)                       # many repeated ids
    q = Queue(b, length, cap, device=DEV)
    o = oracle.Queue(b, length, cap)
    for step in range(3):
        ids = rng.integers(0, universe * (step + 1), (b, m)).astype(np.int32)
        dist = ((ids.astype(np.int64) * 7919) % 1009).astype(np.float32) / np.float32(1009.0)  # id -> distance, with ties
        ids[rng.random((b, m)) < 0.05] = MAXINT
        dist[ids == MAXINT] = oracle.MAXFLOAT
        excl = np.full((b, 6), MAXINT, dtype=np.int32)
        excl[:, :3] = rng.integers(0, universe, (b, 3))
        want_changed = o.insert(ids, dist, exclude=excl, output_update=True)
        got_changed = q.insert(t(ids), t(dist), exclude=t(excl), output_update=True)
        assert np.array_equal(n(q.indices), o.indices)
        assert np.array_equal(n(q.distances), o.distances)
        assert np.array_equal(n(got_changed), want_changed)
        assert np.array_equal(n(q.pop_n_ids(4)), o.pop_n_ids(4))


def test_seen_list_trace_vs_reference_host_code(c1, built_lib):
    from vectorlink_gpu.utils import add_new_to_seen_
    seen = torch.full((4, 7), MAXINT, dtype=torch.int32, device=DEV)
    for vis, want, alive in zip(c1["op_seen_visits"], c1["op_seen_trace"], c1["op_seen_alive"]):
        r = add_new_to_seen_(seen, t(vis)) if seen is not None else None
        assert (r is not None) == bool(alive)
        if r is None:
            seen = None
        else:
            assert np.array_equal(n(seen), want)


def test_dedup_helpers_vs_simulated_reference(kat, built_lib):
    from vectorlink_gpu.kernels import dedup_tensor_, dedup_tensor_pair_, punchout_duplicates_, punchout_excluded_
    from vectorlink_gpu.utils import dedup_sort, index_sort, queue_sort
    ids, dist = t(kat["k67_ids_in"]), t(kat["k67_dist_in"])
    dedup_tensor_pair_(ids, dist)
    assert np.array_equal(n(ids), kat["k67_ids_out"]) and np.array_equal(n(dist), kat["k67_dist_out"])
    pi, pd = punchout_duplicates_(t(kat["k67_ids_in"]), t(kat["k67_dist_in"]))
    assert np.array_equal(n(pi), kat["k67_sorted_ids_out"]) and np.array_equal(n(pd), kat["k67_sorted_dist_out"])
    qi, qd = queue_sort(t(kat["k67_ids_in"]), t(kat["k67_dist_in"]))
    assert np.array_equal(n(qi), kat["k67_sorted_ids_out"]) and np.array_equal(n(qd), kat["k67_sorted_dist_out"])
    s = t(kat["k68_in"])
    dedup_tensor_(s)
    assert np.array_equal(n(s), kat["k68_out"])
    assert np.array_equal(n(dedup_sort(t(kat["k68_in"]))), np.sort(kat["k68_out"], axis=1))
    ids, dist = t(kat["k10_ids_in"]), t(kat["k10_dist_in"])
    c0 = int(kat["k10_col0"])
    punchout_excluded_(ids.narrow(1, c0, ids.size(1) - c0), dist.narrow(1, c0, ids.size(1) - c0), t(kat["k10_excl"]))
    assert np.array_equal(n(ids), kat["k10_ids_out"]) and np.array_equal(n(dist), kat["k10_dist_out"])
    rng = np.random.default_rng(5)
    ri = rng.integers(0, 50, (9, 21)).astype(np.int32)
    rd = rng.integers(0, 7, (9, 21)).astype(np.float32)
    si, sd = index_sort(t(ri), t(rd))
    order = np.lexsort((ri, rd), axis=1)
    assert np.array_equal(n(si), np.take_along_axis(ri, order, 1)) and np.array_equal(n(sd), np.take_along_axis(rd, order, 1))


@pytest.mark.parametrize("tag", ["a", "b"])
def test_prune_vs_simulated_reference(kat, built_lib, tag):
    from vectorlink_gpu.kernels import prune_
    b, d = prune_(t(kat[f"k9{tag}_beams_in"]), t(kat[f"k9{tag}_dist_in"]))
    assert np.array_equal(n(b), kat[f"k9{tag}_beams_out"])
    assert np.array_equal(n(d), kat[f"k9{tag}_dist_out"])


@pytest.mark.parametrize("rows,w", [(500, 48), (300, 96), (64, 192), (100, 7)])
def test_prune_random_vs_oracle(built_lib, rows, w):
    from vectorlink_gpu.kernels import prune_
    rng = np.random.default_rng(rows + w)
    v = unit(rng, rows, 12)
    full = ((1.0 - v @ v.T) / 2.0).astype(np.float32)
    np.fill_diagonal(full, np.inf)
    order = np.argsort(full, axis=1, kind="stable")[:, :w].astype(np.int32)
    d = np.take_along_axis(full, order, axis=1).astype(np.float32)
    wb, wd = oracle.prune_(order, d)
    gb, gd = prune_(t(order), t(d))
    assert np.array_equal(n(gb), wb) and np.array_equal(n(gd), wd)
    assert (wb == MAXINT).any()
    gb2, gd2 = prune_(t(order), t(d), out_cols=max(1, w // 3))
    assert np.array_equal(n(gb2), wb[:, :max(1, w // 3)])


def test_circulants_vs_reference_host_code(c1, built_lib):
    from vectorlink_gpu.utils import generate_circulant_beams, generate_queue_circulants, primes
    assert np.array_equal(n(generate_circulant_beams(50, primes(9, DEV))), c1["op_circ_beams"])
    assert np.array_equal(n(generate_queue_circulants(7, 50, primes(9, DEV))), c1["op_circ_queue"])


def test_reverse_edges_vs_numpy(built_lib):
    from vectorlink_gpu.kernels import reverse_edges
    rng = np.random.default_rng(8)
    nn, d, scan, keep = 300, 12, 8, 5
    beams = rng.integers(0, nn, (nn, d)).astype(np.int32)
    beams[rng.random((nn, d)) < 0.1] = MAXINT
    got = n(reverse_edges(t(beams), scan=scan, keep=keep))
    want = np.full((nn, keep), MAXINT, dtype=np.int32)
    lists = [[] for _ in range(nn)]
    for r in range(scan):                       # rank-major, source ascending
        for x in range(nn):
            y = beams[x, r]
            if y != MAXINT:
                lists[y].append(x)
    for y in range(nn):
        row = lists[y][:keep]
        want[y, :len(row)] = row
    assert np.array_equal(got, want)


def test_symmetrize_adds_reverse_edges_and_keeps_rows_well_formed(built_lib):
    from vectorlink_gpu.kernels import symmetrize, calculate_distances
    rng = np.random.default_rng(9)
    v = unit(rng, 800, 16)
    kn = oracle.bruteforce_knn(v, v, 12, exclude_self=True)
    d = oracle.calculate_distances(v, kn)
    ids, dist = symmetrize(t(v), t(kn), t(d))
    ids, dist = n(ids), n(dist)
    assert ids.shape == kn.shape
    assert np.all(np.diff(dist, axis=1) >= 0)
    for r in range(800):
        real = ids[r][ids[r] != MAXINT]
        assert len(set(real)) == len(real) and r not in real
    assert np.array_equal(n(calculate_distances(t(v), t(ids))), dist)
    # the best half of the forward edges survives; reverse edges made it in where they exist
    assert all(set(kn[r, :6]) <= set(ids[r]) for r in range(800))
    fwd = [set(row) for row in kn]
    gained = sum(1 for x in range(800) for y in ids[x] if y != MAXINT and y not in fwd[x] and x in fwd[y])
    assert gained > 0


def test_symmetrize_cut_inside_the_forward_tail_keeps_the_closest(built_lib):
    """Rows whose reverse neighbours repeat forward ones leave room for part of the forward tail:
    the columns kept from it must be its closest ones (a NumPy model of the three priority classes)."""
    from vectorlink_gpu.kernels import reverse_edges, symmetrize
    rng = np.random.default_rng(10)
    nn, d, keep = 600, 12, 6
    v = unit(rng, nn, 8)                       # low dimension: neighbour relations are mostly mutual
    kn = oracle.bruteforce_knn(v, v, d, exclude_self=True)
    dd = oracle.calculate_distances(v, kn)
    ids, dist = symmetrize(t(v), t(kn), t(dd), keep=keep)
    ids = n(ids)
    rev = n(reverse_edges(t(kn), scan=d, keep=keep))
    into_tail = 0
    for x in range(nn):
        want = []
        for y in list(kn[x, : d - keep]) + [r for r in rev[x] if r != x] + list(kn[x, d - keep:]):
            if y != MAXINT and y not in want:
                want.append(y)
        tail_kept = [y for y in want[:d] if y in kn[x, d - keep:] and y not in rev[x]]
        into_tail += 0 < len(tail_kept) < keep
        # the kept part of the tail is a prefix of it (its closest entries)
        tail = [y for y in kn[x, d - keep:] if y not in rev[x]]
        assert tail_kept == tail[:len(tail_kept)]
        assert sorted(want[:d]) == sorted(y for y in ids[x] if y != MAXINT)
    assert into_tail > 0


def test_full_prune_scan_vs_numpy(built_lib):
    """prune_(full=True): every neighbour of y is a detour witness; rows in rising slot order see
    their own punches, other rows are read as they came in."""
    from vectorlink_gpu.kernels import prune_
    rng = np.random.default_rng(21)
    rows, w = 120, 10
    v = unit(rng, rows, 6)
    full = ((1.0 - v @ v.T) / 2.0).astype(np.float32)
    np.fill_diagonal(full, np.inf)
    order = np.argsort(full, axis=1, kind="stable")[:, :w].astype(np.int32)
    d = np.take_along_axis(full, order, axis=1).astype(np.float32)
    wb, wd = order.copy(), d.copy()
    for x in range(rows):
        for s in range(w):
            y = wb[x, s]
            if y == MAXINT:
                continue
            hits = []
            for j in range(w):                         # one warp pass: all lanes decide, then punch
                z, dz = order[y, j], d[y, j]
                xi = -1
                for i in range(w):
                    if wb[x, i] == z:
                        xi = i
                if xi >= 0 and wd[x, xi] > wd[x, s] and wd[x, xi] > dz:
                    hits.append(xi)
            for xi in hits:
                wb[x, xi], wd[x, xi] = MAXINT, np.float32(oracle.MAXFLOAT)
    key = np.lexsort((wb, wd), axis=1)
    wb, wd = np.take_along_axis(wb, key, 1), np.take_along_axis(wd, key, 1)
    gb, gd = prune_(t(order), t(d), full=True)
    assert np.array_equal(n(gb), wb) and np.array_equal(n(gd), wd)
    fb, _ = prune_(t(order), t(d))
    assert (n(gb) == MAXINT).sum() > (n(fb) == MAXINT).sum()       # prunes more than the first-neighbour test


def test_prune_of_a_row_range_equals_the_full_prune_on_those_rows(built_lib):
    """vl_prune_rows: witnesses are read from every row, only the rows of the range are written."""
    from vectorlink_gpu.kernels import prune_
    rng = np.random.default_rng(33)
    rows, w = 500, 12
    v = unit(rng, rows, 8)
    kn = oracle.bruteforce_knn(v, v, w, exclude_self=True)
    d = oracle.calculate_distances(v, kn)
    full_b, full_d = prune_(t(kn), t(d))
    out_b = torch.full((rows, w), -7, dtype=torch.int32, device=DEV)
    out_d = torch.full((rows, w), -7.0, dtype=torch.float32, device=DEV)
    prune_(t(kn), t(d), rows=(123, 377), out=(out_b, out_d))
    assert torch.equal(out_b[123:377], full_b[123:377]) and torch.equal(out_d[123:377], full_d[123:377])
    assert bool((out_b[:123] == -7).all()) and bool((out_b[377:] == -7).all())
    wb, wd = oracle.prune_(kn, d)
    assert np.array_equal(n(full_b), wb) and np.array_equal(n(full_d), wd)

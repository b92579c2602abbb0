"""Generates the golden fixtures in this directory from the reference's own code.

Needs a checkout of the reference (read only), named by VL_REFERENCE_ROOT:

    VL_REFERENCE_ROOT=<checkout> python tests/golden/make_golden.py sim    # -> kat_sim.npz   (a few minutes)
    VL_REFERENCE_ROOT=<checkout> python tests/golden/make_golden.py host   # -> c1_host.npz, small_host.npz, multi_host.npz

``sim``  runs the reference's real Numba kernels in the Numba CUDA simulator on micro-cases
         (about one second per simulated block, so only tens of blocks per case).
``host`` runs the reference's own queue.py / utils.py / ann.py on CPU tensors with the
         seven global kernels replaced by the C oracle (see reference_shim.py).

The fixtures hold inputs and outputs; the tests never import the reference.
"""
from __future__ import annotations

import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.abspath(os.path.join(HERE, "..", "..")))

from reference_shim import load_reference  # noqa: E402


def unit_rows(rng, n, dim):
    v = rng.standard_normal((n, dim)).astype(np.float32)
    return (v / np.linalg.norm(v, axis=1, keepdims=True)).astype(np.float32)


def make_sim():
    import torch
    ref = load_reference("simulator")
    K = ref.kernels
    MAXINT = ref.constants.MAXINT
    out = {}
    rng = np.random.default_rng(1234)

    # K4: calculate_distances (kernels.py:174-201) at several dimensions
    for dim in (64, 96, 128, 768, 1024, 1536):
        n, w = 5, 3
        v = unit_rows(rng, n, dim)
        beams = rng.integers(0, n, size=(n, w)).astype(np.int32)
        beams[1, 2] = MAXINT
        t0 = time.time()
        d = K.calculate_distances(torch.from_numpy(v), torch.from_numpy(beams))
        print(f"K4 dim={dim}: {n*w} blocks in {time.time()-t0:.1f}s", flush=True)
        out[f"k4_{dim}_vectors"] = v
        out[f"k4_{dim}_beams"] = beams
        out[f"k4_{dim}_out"] = d.numpy().copy()

    # K5: search_from_seeds (kernels.py:260-311); the simulator can only run it at
    # dim >= 1024 (below that the kernel indexes past its dim-sized dynamic buffer)
    for dim in (1024, 1536):
        n, w, b, vcount = 6, 3, 2, 2
        v = unit_rows(rng, n, dim)
        q = unit_rows(rng, b, dim)
        beams = rng.integers(0, n, size=(n, w)).astype(np.int32)
        visit = np.array([[4, 1], [MAXINT, 2]], dtype=np.int32)
        t0 = time.time()
        idx, d = K.search_from_seeds(torch.from_numpy(q), torch.from_numpy(visit), torch.from_numpy(beams),
                                     torch.from_numpy(v))
        print(f"K5 dim={dim}: {b*vcount*w} blocks in {time.time()-t0:.1f}s", flush=True)
        out[f"k5_{dim}_vectors"] = v
        out[f"k5_{dim}_queries"] = q
        out[f"k5_{dim}_beams"] = beams
        out[f"k5_{dim}_visit"] = visit
        out[f"k5_{dim}_idx"] = idx.numpy().copy()
        out[f"k5_{dim}_dist"] = d.numpy().copy()

    # K6+K7: dedup_tensor_pair_ (kernels.py:383-397) on rows sorted by (distance, id)
    ids = np.array([[3, 3, 5, 7, 7, 7, 9, MAXINT, MAXINT, MAXINT],
                    [1, 2, 3, 4, 5, 6, 7, 8, 9, 10],
                    [4, 4, 4, 4, MAXINT, MAXINT, MAXINT, MAXINT, MAXINT, MAXINT]], dtype=np.int32)
    dist = np.sort(rng.random((3, 10)).astype(np.float32), axis=1)
    dist[ids == MAXINT] = np.float32(ref.constants.MAXFLOAT)
    out["k67_ids_in"] = ids.copy()
    out["k67_dist_in"] = dist.copy()
    ti, td = torch.from_numpy(ids.copy()), torch.from_numpy(dist.copy())
    K.dedup_tensor_pair_(ti, td)
    out["k67_ids_out"] = ti.numpy().copy()
    out["k67_dist_out"] = td.numpy().copy()
    # punchout_duplicates_ = the same followed by the sort (kernels.py:400-406)
    pi, pd = K.punchout_duplicates_(torch.from_numpy(ids.copy()), torch.from_numpy(dist.copy()))
    out["k67_sorted_ids_out"] = pi.numpy().copy()
    out["k67_sorted_dist_out"] = pd.numpy().copy()

    # K6+K8: dedup_tensor_ (kernels.py:370-380) on sorted id rows
    seen = np.array([[1, 1, 2, 8, 8, MAXINT, MAXINT], [5, 6, 7, 8, 9, 10, 11]], dtype=np.int32)
    out["k68_in"] = seen.copy()
    ts = torch.from_numpy(seen.copy())
    K.dedup_tensor_(ts)
    out["k68_out"] = ts.numpy().copy()

    # K10: punchout_excluded_ (kernels.py:491-501) on column-sliced views, as Queue.insert calls it
    qi = rng.integers(0, 12, size=(3, 10)).astype(np.int32)
    qd = rng.random((3, 10)).astype(np.float32)
    excl = np.array([[2, 5, MAXINT, 7], [MAXINT, 1, 2, 3], [0, 1, 2, 3]], dtype=np.int32)
    out["k10_ids_in"] = qi.copy()
    out["k10_dist_in"] = qd.copy()
    out["k10_excl"] = excl
    out["k10_col0"] = np.int64(4)
    ti, td = torch.from_numpy(qi.copy()), torch.from_numpy(qd.copy())
    K.punchout_excluded_(ti.narrow(1, 4, 6), td.narrow(1, 4, 6), torch.from_numpy(excl))
    out["k10_ids_out"] = ti.numpy().copy()
    out["k10_dist_out"] = td.numpy().copy()

    # K9: prune_ (kernels.py:441-468) on a small graph whose rows are sorted by distance
    for tag, (n, w, dim) in {"a": (14, 6, 8), "b": (40, 8, 4)}.items():
        v = unit_rows(rng, n, dim)
        full = ((1.0 - v @ v.T) / 2.0).astype(np.float32)
        np.fill_diagonal(full, np.inf)
        order = np.argsort(full, axis=1, kind="stable")[:, :w].astype(np.int32)
        d = np.take_along_axis(full, order, axis=1).astype(np.float32)
        if tag == "b":                      # a row that already carries sentinels
            order[3, -2:] = MAXINT
            d[3, -2:] = np.float32(ref.constants.MAXFLOAT)
        out[f"k9{tag}_beams_in"] = order.copy()
        out[f"k9{tag}_dist_in"] = d.copy()
        pb, pd = K.prune_(torch.from_numpy(order.copy()), torch.from_numpy(d.copy()))
        out[f"k9{tag}_beams_out"] = pb.numpy().copy()
        out[f"k9{tag}_dist_out"] = pd.numpy().copy()
        print(f"K9 {tag}: punched {(pb.numpy() == MAXINT).sum() - (order == MAXINT).sum()} edges", flush=True)

    np.savez_compressed(os.path.join(HERE, "kat_sim.npz"), **out)
    print("wrote kat_sim.npz")


def run_host_case(ref, vectors, queries, kwargs, single_query=True):
    import torch
    A = ref.ann
    tv = torch.from_numpy(vectors)
    res = {"vectors": vectors, "queries": queries}
    for k, val in kwargs.items():
        res[f"cfg_{k}"] = np.int64(val)
    t0 = time.time()
    ann = A.ANN(tv, **kwargs)
    res["build_seconds"] = np.float64(time.time() - t0)
    res["beams"] = ann.beams.numpy().copy()
    res["stale_distances"] = ann.distances.numpy().copy()      # ann.py:190-193 returns the initial ones
    res["distances"] = ref.kernels.calculate_distances(tv, ann.beams).numpy().copy()
    found, ratio = ann.recall()
    res["self_recall_found"] = np.int64(found)

    tq = torch.from_numpy(queries)
    if single_query:
        # un-patched reference: ANN.search works as shipped for one query row (ann.py:211-214)
        one = ann.search(tq[:1])
        res["search1_ids"] = one.indices.numpy().copy()
        res["search1_dist"] = one.distances.numpy().copy()
        res["search1_length"] = np.int64(one.length)

    # batched search needs the broadcast the authors intended: q1[B,dim] -> [B,1,dim]
    orig = A.query_cosine_distances
    A.query_cosine_distances = lambda q1, q2: orig(q1.unsqueeze(1), q2)
    sq = ann.search(tq)
    res["search_ids"] = sq.indices.numpy().copy()
    res["search_dist"] = sq.distances.numpy().copy()
    res["search_length"] = np.int64(sq.length)

    # the same with seed distances taken by the kernels' summation order instead of torch's
    def tree_seed(q1, q2):
        b, qn, dim = q2.shape
        out = torch.empty((b, qn), dtype=torch.float32)
        import oracle
        for i in range(b):
            ident = np.arange(qn, dtype=np.int32).reshape(-1, 1)
            _, d = oracle.search_from_seeds(q1[i:i + 1].numpy(), np.arange(qn, dtype=np.int32)[None, :], ident,
                                            q2[i].numpy())
            out[i] = torch.from_numpy(d[0])
        return out
    A.query_cosine_distances = tree_seed
    sq = ann.search(tq)
    res["search_tree_ids"] = sq.indices.numpy().copy()
    res["search_tree_dist"] = sq.distances.numpy().copy()
    A.query_cosine_distances = orig
    return res, ann


def make_host():
    import torch
    ref = load_reference("host")
    U, Q = ref.utils, ref.queue
    MAXINT = ref.constants.MAXINT

    # the reference's prime table must equal the regenerated one the product and oracle use
    import oracle
    assert np.array_equal(ref.constants.PRIMES.numpy(), oracle.primes_table()), "prime table mismatch"

    # config 1 of the benchmark plan: 2,000 x 64, seed 0, N(0,1) rows L2-normalised,
    # 100 queries drawn the same way from the same generator; degree 16, beam 32.
    torch.manual_seed(0)
    v = torch.nn.functional.normalize(torch.randn(2000, 64, dtype=torch.float32), dim=1).numpy().copy()
    q = torch.nn.functional.normalize(torch.randn(100, 64, dtype=torch.float32), dim=1).numpy().copy()
    kwargs = dict(beam_size=16, recall_search_queue_factor=2, visit_queue_factor=2)
    res, ann = run_host_case(ref, v, q, kwargs)
    print(f"c1: build {float(res['build_seconds']):.1f}s self-recall {int(res['self_recall_found'])}", flush=True)

    # operator-level traces from the same data: Queue.insert / pop_n_ids / add_new_to_seen_
    tv = torch.from_numpy(v)
    rng = np.random.default_rng(7)
    b, length, m = 6, 12, 16
    queue = Q.Queue(b, length, length + m)
    ids0 = rng.integers(0, 40, size=(b, m)).astype(np.int32)
    ids0[0, 3] = MAXINT
    d0 = (ids0.astype(np.float32) * np.float32(0.013)) % np.float32(0.2)   # same id -> same distance
    d0[ids0 == MAXINT] = np.float32(ref.constants.MAXFLOAT)
    queue.insert(torch.from_numpy(ids0), torch.from_numpy(d0))
    res["op_ins0_ids"] = ids0
    res["op_ins0_dist"] = d0
    res["op_q0_ids"] = queue.indices.numpy().copy()
    res["op_q0_dist"] = queue.distances.numpy().copy()
    popped = queue.pop_n_ids(3)
    res["op_pop_ids"] = popped.numpy().copy()
    res["op_q1_ids"] = queue.indices.numpy().copy()
    res["op_q1_dist"] = queue.distances.numpy().copy()
    ids1 = rng.integers(0, 40, size=(b, m)).astype(np.int32)
    d1 = (ids1.astype(np.float32) * np.float32(0.013)) % np.float32(0.2)
    excl = np.full((b, 5), MAXINT, dtype=np.int32)
    excl[:, 0] = rng.integers(0, 40, size=b)
    excl[:, 1] = rng.integers(0, 40, size=b)
    excl[2, 1] = MAXINT
    excl[2, 2] = ids1[2, 0]                      # after a MAXINT: never reached by the scan
    changed = queue.insert(torch.from_numpy(ids1), torch.from_numpy(d1), exclude=torch.from_numpy(excl),
                           output_update=True)
    res["op_ins1_ids"] = ids1
    res["op_ins1_dist"] = d1
    res["op_ins1_excl"] = excl
    res["op_q2_ids"] = queue.indices.numpy().copy()
    res["op_q2_dist"] = queue.distances.numpy().copy()
    res["op_q2_changed"] = changed.numpy().copy()

    seen = torch.full((4, 7), MAXINT, dtype=torch.int32)
    trace = []
    visits = [np.array([[5, 9], [3, MAXINT], [8, 8], [1, 2]], dtype=np.int32),
              np.array([[4, 6], [7, 2], [MAXINT, MAXINT], [9, 3]], dtype=np.int32),
              np.array([[1, 0], [6, 5], [2, 4], [8, 7]], dtype=np.int32),
              np.array([[11, 12], [13, 14], [15, 16], [17, 18]], dtype=np.int32),
              np.array([[21, 22], [23, 24], [25, 26], [27, 28]], dtype=np.int32)]
    alive = []
    for vis in visits:
        r = U.add_new_to_seen_(seen, torch.from_numpy(vis)) if seen is not None else None
        alive.append(r is not None)
        if r is None:
            trace.append(np.full((4, 7), -1, dtype=np.int32))
            seen = None
        else:
            seen = r
            trace.append(seen.numpy().copy())
    res["op_seen_visits"] = np.stack(visits)
    res["op_seen_trace"] = np.stack(trace)
    res["op_seen_alive"] = np.array(alive)

    # circulant seeds (utils.py:26-41)
    res["op_circ_beams"] = U.generate_circulant_beams(50, U.primes(9)).numpy().copy()
    res["op_circ_queue"] = U.generate_queue_circulants(7, 50, U.primes(9)).numpy().copy()

    np.savez_compressed(os.path.join(HERE, "c1_host.npz"), **res)
    print("wrote c1_host.npz")

    # a second, smaller case at the reference's default parameters, a dimension that is not
    # a power of two, and a graph small enough that queues run dry and searches stop early
    rng = np.random.default_rng(11)
    v2 = unit_rows(rng, 300, 40)
    q2 = unit_rows(rng, 5, 40)
    res2, _ = run_host_case(ref, v2, q2, dict(beam_size=8, batch_size=128))
    print(f"small: build {float(res2['build_seconds']):.1f}s self-recall {int(res2['self_recall_found'])}", flush=True)
    np.savez_compressed(os.path.join(HERE, "small_host.npz"), **res2)
    print("wrote small_host.npz")
    make_multi(ref)


def make_multi(ref):
    """A build that needs several rounds, from the PATCHED reference -> multi_host.npz.

    As shipped, generate_ann never rebinds `beam_distances` (ann.py:172 assigns prune_'s second
    result to an unused name), so a second round would pair the new neighbour lists with the
    first round's circulant distances.  Both c1 and small reach self-recall 1.0 in round one and
    never get there.  Here the one name at that statement (and at its no-prune twin, ann.py:174)
    is changed in the function's text in memory - nothing else - so that rounds two and three run
    on consistent lists: pruned rows with MAXINT tails, re-seeding with carried distances."""
    import inspect
    import torch
    A = ref.ann
    src = inspect.getsource(A.generate_ann)
    assert src.count("(beams, distances) = ") == 2
    exec(compile(src.replace("(beams, distances) = ", "(beams, beam_distances) = "), "<patched generate_ann>", "exec"),
         A.__dict__)
    # Second patch, same style: the last sort of punchout_duplicates_ (kernels.py:402) and of prune_
    # (kernels.py:466) is torch's default, which is not stable; among entries at exactly the same
    # distance it may undo the (distance, id) order index_sort established, differently per torch
    # build and device (seen on this CPU: two ids at one distance swap, the "head changed" test
    # fires, the loop runs 25 iterations instead of 10).  `stable=True` there makes the tie order
    # the one index_sort defines, which is also what the oracle and the CUDA path implement.
    K = ref.kernels
    for name in ("punchout_duplicates_", "prune_"):
        fsrc = inspect.getsource(getattr(K, name))
        assert fsrc.count("distances.sort()") == 1
        exec(compile(fsrc.replace("distances.sort()", "distances.sort(stable=True)"), f"<patched {name}>", "exec"),
             K.__dict__)
        for mod in (ref.queue, ref.utils, ref.ann):
            if hasattr(mod, name):
                setattr(mod, name, getattr(K, name))
    rounds = []
    stamp = A.print_timestamp
    A.print_timestamp = lambda msg: rounds.append(msg) if str(msg).startswith("start of cagra loop") else None
    rng = np.random.default_rng(17)
    dim, count = 48, 1800
    centres = rng.uniform(0, 255, (12, dim))
    pts = centres[rng.integers(0, 12, count)] + rng.normal(0, 20, (count, dim))
    v = np.round(pts).clip(0, 255).astype(np.float32)
    v = (v / np.linalg.norm(v, axis=1, keepdims=True)).astype(np.float32)
    kwargs = dict(beam_size=8, visit_queue_factor=2, recall_search_queue_factor=2, batch_size=500)
    t0 = time.time()
    ann = A.ANN(torch.from_numpy(v), **kwargs)
    A.print_timestamp = stamp
    res = {"vectors": v, "beams": ann.beams.numpy().copy(), "distances": ann.distances.numpy().copy(),
           "loops": np.int64(len(rounds))}
    for k, val in kwargs.items():
        res[f"cfg_{k}"] = np.int64(val)
    found, _ = ann.recall()
    res["self_recall_found"] = np.int64(found)
    assert np.array_equal(res["distances"], ref.kernels.calculate_distances(torch.from_numpy(v), ann.beams).numpy())
    print(f"multi: {len(rounds)} rounds in {time.time() - t0:.1f}s, self-recall {found}", flush=True)
    assert len(rounds) >= 2, "the case must not converge in one round"
    np.savez_compressed(os.path.join(HERE, "multi_host.npz"), **res)
    print("wrote multi_host.npz")


if __name__ == "__main__":
    what = sys.argv[1] if len(sys.argv) > 1 else "all"
    if what in ("sim", "all"):
        make_sim()
    if what in ("host", "all"):
        make_host()
    if what == "multi":
        make_multi(load_reference("host"))

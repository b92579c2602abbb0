"""Host-side driver logic that needs no GPU."""
import numpy as np
import torch

import oracle


def cfg(**kw):
    return oracle.make_config(**kw)


def test_loop_bounds_match_the_oracle_iteration_counts(c1, small):
    from vectorlink_gpu.ann import loop_bounds
    from conftest import cfg_of
    for g in (c1,):
        config, _ = cfg_of(g)
        q = oracle.initial_search_queue(g["vectors"], g["queries"], config)
        n = oracle.closest_vectors(g["queries"], q, g["vectors"], g["beams"], config)
        k_none, n_checks, n_max = loop_bounds(config)
        assert n == n_max and k_none <= n_max and n_checks == k_none // config["speculative_readahead"]


def test_loop_bounds_closed_form():
    from vectorlink_gpu.ann import loop_bounds
    assert loop_bounds(cfg(beam_size=16)) == (61, 12, 65)                       # E=240: 61 productive, leaves at 65
    assert loop_bounds(cfg(beam_size=32, visit_queue_factor=2)) == (81, 16, 85)  # E=320
    assert loop_bounds(cfg(beam_size=64, visit_queue_factor=2)) == (161, 32, 165)
    assert loop_bounds(cfg(beam_size=8, exclude_factor=0)) == (1, 0, 5)
    k_none, n_checks, n_max = loop_bounds(cfg(beam_size=6, visit_queue_factor=1, exclude_factor=6, parallel_visit_count=4))
    assert (k_none, n_checks, n_max) == (10, 2, 15)                              # k_none on a check iteration


def test_natural_end_reads_the_first_quiet_check():
    from vectorlink_gpu.ann import _natural_end
    config = cfg(beam_size=16)
    assert _natural_end([1] * 12, config) == 65
    assert _natural_end([1, 1, 0] + [1] * 9, config) == 15
    assert _natural_end([0] * 12, config) == 5


def test_fused_shape_rule():
    from vectorlink_gpu.ann import _fused_shape_ok
    v = torch.zeros(8, 64)
    c = cfg(beam_size=16)
    assert _fused_shape_ok(v, 48, 48, 48 + 4 * 48, c)            # build queue
    assert _fused_shape_ok(v, 16, 48, 48 + 64, c)                # search queue (Q=48, pvc*D=64)
    assert not _fused_shape_ok(v, 16, 96, 192, cfg(beam_size=16, recall_search_queue_factor=6))  # stale columns
    assert not _fused_shape_ok(torch.zeros(8, 30), 48, 48, 240, c)  # rows not 16-byte chunks


def test_seed_table_equals_the_oracle_table():
    from vectorlink_gpu.constants import PRIMES_HOST, MAXINT, MAXFLOAT
    assert np.array_equal(PRIMES_HOST.numpy(), oracle.primes_table())
    assert MAXINT == oracle.MAXINT and float(np.float32(MAXFLOAT)) == oracle.MAXFLOAT


def test_readme_alias_imports():
    import vectorlink
    from vectorlink.ann import ANN
    from vectorlink_gpu import ANN as ANN2
    assert ANN is ANN2


def test_runner_flags_and_defaults_are_the_reference_runners():
    """main.py:24-98 of the reference: same flags, and defaults that differ from ANN's own
    (3 parallel visits, recall queue factor 6, pruning off unless -P)."""
    import importlib.util
    import os
    from conftest import PKG_ROOT
    spec = importlib.util.spec_from_file_location("vl_runner", os.path.join(PKG_ROOT, "main.py"))
    runner = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(runner)
    args = runner.make_parser().parse_args([])
    params = runner.build_params(args)
    assert params == {"vector_count": 10_000, "vector_dimension": 1536, "prune": False, "beam_size": 24,
                      "parallel_visit_count": 3, "beam_queue_factor": 3, "visit_queue_factor": 3, "exclude_factor": 5,
                      "optimization_loops": 3, "batch_size": 10_000, "recall_search_queue_factor": 6,
                      "speculative_readahead": 5}
    args = runner.make_parser().parse_args("-c 500 -d 64 -n 8 -P -p 4 -r 2 -q 2 -l 1 -L -C".split())
    params = runner.build_params(args)
    assert params["vector_count"] == 500 and params["prune"] is True and params["parallel_visit_count"] == 4
    assert params["recall_search_queue_factor"] == 2 and params["optimization_loops"] == 1


def test_bench_groups_launches_by_phase_and_keeps_the_fraction_honest():
    """bench.launch_classes / roofline_of on fake launch records: the headline fraction is the
    gathered bytes of the later build rounds, never the schedule's bytes."""
    import torch
    import bench

    class Ev:
        def __init__(self, t):
            self.t = t

        def elapsed_time(self, other):
            return other.t - self.t

    def rec(tag, t0, t1, evals, gathered, memo):
        st = torch.zeros(24, dtype=torch.int64)
        st[1] = gathered
        return {"start": Ev(t0), "end": Ev(t1), "rows": 1000, "graph_w": 96, "iterations": 81, "evals": evals,
                "memo": memo, "stats": st, "tag": tag}

    prof = [rec("round0", 0, 1000, 10**9, 10**9, False), rec("self_recall", 1000, 1001, 10**5, 3 * 10**4, True),
            rec("round1", 1001, 1501, 10**9, 2 * 10**8, True), rec("round2", 1501, 1901, 10**9, 10**8, True)]
    cls = bench.launch_classes(prof, 1, 128)
    assert set(cls) == {"build_round0", "self_recall", "build_later_rounds"}
    later = cls["build_later_rounds"]
    assert later["launches_per_step"] == 2 and later["ms_per_launch"] == 450
    assert abs(later["gathered_fraction"] - 0.15) < 1e-12
    roof = bench.roofline_of(cls, {}, 6534.5, "test", "none", 128, 0.99)
    assert roof["class"] == "build_later_rounds" and roof["rows_served_from"] == "DRAM"
    assert abs(roof["achieved"] - 3e8 * 524 / 0.9 / 1e9) < 1e-6
    assert roof["frac"] < 1.0 and roof["classes"]["build_later_rounds"]["vs_reference_schedule"] > roof["frac"]
    assert roof["traffic"] is None          # no capture on record for this workload name


def test_tile_pass_wrappers_refuse_cpu_tensors(built_lib):
    import torch
    from vectorlink_gpu import _lib, knn_tile
    import pytest as _pytest
    with _pytest.raises(_lib.VlError):
        knn_tile.prepare(torch.zeros(4, 64), want_norms=True)

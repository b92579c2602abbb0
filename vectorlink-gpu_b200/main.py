"""Experiment runner: build an index over random unit vectors, measure its self-recall, write a
JSON log.  Same flags and defaults as the reference's runner (main.py:22-98 - note that they
differ from ANN's own defaults: 3 parallel visits, recall queue factor 6, pruning off unless -P),
same log location (./log/experiment-<time>.log).  The log is what `ANN.dump_logs()` returns: the
build parameters plus total_time, recall, GPU and commit.

    python main.py -c 100000 -d 128 -n 32 -P
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import Dict, Optional

HERE = os.path.dirname(os.path.abspath(__file__))
if HERE not in sys.path:
    sys.path.insert(0, HERE)

# (flag, long name, type, default, help) - main.py:24-98 of the reference
INT_OPTIONS = [
    ("-c", "--vector-count", 10_000, "number of vectors"),
    ("-d", "--vector-dimension", 1536, "dimension of vectors"),
    ("-n", "--beam_size", 24, "beam size (max number of neighbors)"),
    ("-l", "--optimization_loops", 3, "build rounds"),
    ("-x", "--exclude_factor", 5, "visited list = this many times the visit queue"),
    ("-q", "--visit_queue_factor", 3, "visit queue = this many times the beam"),
    ("-f", "--beam_queue_factor", 3, "build-time lists = this many times the beam"),
    ("-b", "--batch_size", 10_000, "rows per batch of a build round"),
    ("-r", "--recall_search_queue_factor", 6, "search queue = this many times the beam"),
    ("-p", "--parallel_visit_count", 3, "nodes expanded per iteration"),
    ("-s", "--speculative_readahead", 5, "iterations between progress checks"),
]
BUILD_KEYS = ["prune", "beam_size", "parallel_visit_count", "beam_queue_factor", "visit_queue_factor", "exclude_factor",
              "optimization_loops", "batch_size", "recall_search_queue_factor", "speculative_readahead"]


def make_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    for short, long_name, default, text in INT_OPTIONS:
        parser.add_argument(short, long_name, type=int, default=default, help=text)
    parser.add_argument("-P", "--prune", action="store_true", default=False, help="prune beams")
    # accepted for compatibility; the reference parses them and never reads them
    parser.add_argument("-L", "--layered", action="store_true", default=False, help="(unused, as in the reference)")
    parser.add_argument("-C", "--cagra", action="store_true", default=False, help="(unused, as in the reference)")
    # additions
    parser.add_argument("--metric", default="cosine", choices=["cosine", "l2"])
    parser.add_argument("--init", default="circulant", choices=["circulant", "knn_tile"], help="start graph of the build")
    parser.add_argument("--seed", type=int, default=None, help="seed of the random vectors")
    parser.add_argument("--log-dir", default="./log")
    return parser


def build_params(args: argparse.Namespace) -> Dict:
    """The configuration dictionary of the reference's runner (main.py:103-116)."""
    params = {"vector_count": args.vector_count, "vector_dimension": args.vector_dimension}
    params.update({key: getattr(args, key) for key in BUILD_KEYS})
    return params


def run_experiment(vectors, configuration: Dict, extra: Optional[Dict] = None) -> Dict:
    """Build over `vectors` with the runner's configuration, measure self-recall; returns the log."""
    from vectorlink_gpu.ann import ANN
    kwargs = {k: v for k, v in configuration.items() if k in BUILD_KEYS}
    kwargs.update(extra or {})
    started = time.time()
    ann = ANN(vectors=vectors, **kwargs)
    log = ann.dump_logs()
    log["experiment_seconds"] = time.time() - started
    for key in ("vector_count", "vector_dimension"):
        log.setdefault(key, configuration.get(key))
    return log


def write_log(log: Dict, log_dir: str) -> str:
    os.makedirs(log_dir, exist_ok=True)
    path = os.path.join(log_dir, f"experiment-{time.time()}.log")
    with open(path, "w") as out:
        json.dump(log, out)
    return path


def main(argv=None) -> str:
    import torch
    from vectorlink_gpu.utils import generate_random_vectors
    args = make_parser().parse_args(argv)
    if args.seed is not None:
        torch.manual_seed(args.seed)
    vectors = generate_random_vectors(number_of_vectors=args.vector_count, dimensions=args.vector_dimension)
    extra = {}
    if args.metric != "cosine":
        extra["metric"] = args.metric
    if args.init != "circulant":
        extra["init"] = args.init
    log = run_experiment(vectors, build_params(args), extra)
    print(log)
    return write_log(log, args.log_dir)


if __name__ == "__main__":
    main()

"""Timing and profiler scopes.

Keeps the three public names of the reference's module (vectorlink_gpu/log.py: `timed`,
`log_time`, `CLOSEST_VECTORS_BATCH_TIME`) on top of one primitive, `DeviceTimer`: a context
manager that brackets a region with CUDA events on torch's current stream and with an NVTX
range, so the same scope shows up by name on a profiler timeline.  Nothing here synchronises
the device unless timing was asked for with VECTORLINK_DEBUG (the reference's decorator is
always on and synchronises twice per decorated call).
"""
from __future__ import annotations

import functools
import time
from contextlib import contextmanager

import torch

from .constants import DEBUG

CLOSEST_VECTORS_BATCH_TIME = 0.0


@contextmanager
def nvtx_range(name: str):
    """Named NVTX range around a host-side region (free when no profiler is attached)."""
    pushed = False
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        pushed = True
    try:
        yield
    finally:
        if pushed:
            torch.cuda.nvtx.range_pop()


class DeviceTimer:
    """`with DeviceTimer("name") as t: ...` then `t.device_seconds` / `t.wall_seconds`.
    Leaving the block waits for the device (that is what makes the two figures meaningful)."""

    def __init__(self, name: str = "region"):
        self.name = name
        self.device_seconds = 0.0
        self.wall_seconds = 0.0

    def __enter__(self):
        self._range = nvtx_range(self.name)
        self._range.__enter__()
        self._first = torch.cuda.Event(enable_timing=True)
        self._last = torch.cuda.Event(enable_timing=True)
        self._t0 = time.perf_counter()
        self._first.record()
        return self

    def __exit__(self, *exc):
        self._last.record()
        self._last.synchronize()
        self.wall_seconds = time.perf_counter() - self._t0
        self.device_seconds = self._first.elapsed_time(self._last) * 1e-3
        self._range.__exit__(*exc)
        return False


def timed(fn):
    """(result, device seconds, wall seconds) of calling `fn()`."""
    with DeviceTimer(getattr(fn, "__name__", "timed")) as t:
        result = fn()
    return result, t.device_seconds, t.wall_seconds


def log_time(func):
    """Decorator: with VECTORLINK_DEBUG set, time every call and print both clocks; the longest
    wall time of `closest_vectors` is kept in CLOSEST_VECTORS_BATCH_TIME.  Otherwise the
    function is returned untouched."""
    if not DEBUG:
        return func

    @functools.wraps(func)
    def measured(*args, **kwargs):
        global CLOSEST_VECTORS_BATCH_TIME
        with DeviceTimer(func.__name__) as t:
            out = func(*args, **kwargs)
        print(f"{func.__name__}: device {t.device_seconds:.6f} s, wall {t.wall_seconds:.6f} s")
        if func.__name__ == "closest_vectors" and t.wall_seconds > CLOSEST_VECTORS_BATCH_TIME:
            CLOSEST_VECTORS_BATCH_TIME = t.wall_seconds
        return out

    return measured

"""Timing helpers of the reference (vectorlink_gpu/log.py).  The reference's decorator is
always on (its DEBUG test never sees False); here it is on only when VECTORLINK_DEBUG is set,
so that no operator synchronises the device behind the caller's back."""
import time

import torch

from .constants import DEBUG


def timed(fn):
    wall_start = time.time()
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    start.record()
    result = fn()
    end.record()
    torch.cuda.synchronize()
    wall_end = time.time()
    return result, start.elapsed_time(end) / 1_000, (wall_end - wall_start)


CLOSEST_VECTORS_BATCH_TIME = 0.0


def log_time(func):
    if not DEBUG:
        return func

    def wrapper(*args, **kwargs):
        global CLOSEST_VECTORS_BATCH_TIME
        (result, cuda_time, wall_time) = timed(lambda: func(*args, **kwargs))
        print(f"[{func.__name__}]\n\tCUDA time: {cuda_time}\n\tWALL time {wall_time}")
        if func.__name__ == "closest_vectors":
            CLOSEST_VECTORS_BATCH_TIME = max(wall_time, CLOSEST_VECTORS_BATCH_TIME)
        return result

    wrapper.__name__ = func.__name__
    return wrapper

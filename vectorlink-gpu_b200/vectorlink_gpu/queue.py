"""Batched fixed-capacity sorted queues (vectorlink_gpu/queue.py), device resident."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
from torch import Tensor

from . import _lib
from ._lib import check, lib, ptr, stream_of
from .constants import MAXFLOAT, MAXINT
from .utils import queue_sort  # noqa: F401  (re-exported like the reference module does)


class Queue:
    """queue.py:21-28: `indices` int32 [num_queues, capacity] and `distances` fp32 of the same
    shape, filled with MAXINT / MAXFLOAT; after any insert every row is ordered by
    (distance, id), ids are unique and the sentinels come last."""

    def __init__(self, num_queues: int, queue_length: int, capacity: int, device="cuda"):
        assert queue_length < capacity
        self.length = queue_length
        self.indices = torch.full((num_queues, capacity), MAXINT, dtype=torch.int32, device=device)
        self.distances = torch.full((num_queues, capacity), MAXFLOAT, dtype=torch.float32, device=device)

    def initialize_from_queue(self, queue: "Queue"):
        """queue.py:30-35."""
        head_length = min(queue.length, self.length)
        self.indices.narrow(1, 0, head_length).copy_(queue.indices.narrow(1, 0, head_length))
        self.distances.narrow(1, 0, head_length).copy_(queue.distances.narrow(1, 0, head_length))

    def insert(self, vector_id_batch: Tensor, distances_batch: Tensor, exclude: Optional[Tensor] = None,
               output_update: bool = False):
        """queue.py:37-61: candidates into the columns behind `length`, excluded ids punched,
        whole row re-ordered and de-duplicated; optionally returns head != previous head.
        The reference rebinds `.indices`/`.distances` to freshly sorted tensors; here the rows are
        sorted in place, so a caller that kept the old tensors sees the new contents."""
        (batches, size_per_batch) = vector_id_batch.size()
        (_, capacity) = self.indices.size()
        assert size_per_batch <= capacity - self.length
        ids = vector_id_batch.contiguous()
        dist = distances_batch.contiguous()
        assert ids.dtype == torch.int32 and dist.dtype == torch.float32
        _lib.require_cuda(self.indices, ids, dist, exclude)
        if exclude is not None:
            exclude = exclude.contiguous()
            assert exclude.dtype == torch.int32 and exclude.size(0) == batches
        changed = None
        if output_update:
            changed = torch.empty((batches, self.length), dtype=torch.uint8, device=self.indices.device)
        check(lib().vl_queue_insert(ptr(self.indices), ptr(self.distances), ctypes.c_int64(batches), capacity,
                                    self.length, ptr(ids), ptr(dist), size_per_batch, ptr(exclude),
                                    exclude.size(1) if exclude is not None else 0, ptr(changed),
                                    stream_of(self.indices)), "vl_queue_insert")
        if output_update:
            return changed.bool()
        return None

    def print(self, tail: Optional[bool] = False):
        """queue.py:78-85: show the heads (ids, then distances); with `tail` also the columns
        behind `length`."""
        sections = [("head", 0, self.length)]
        if tail:
            sections.append(("tail", self.length, self.indices.size(1) - self.length))
        for label, start, width in sections:
            print(f"-- {label}: columns {start}..{start + width - 1}")
            print(self.indices.narrow(1, start, width))
            print(self.distances.narrow(1, start, width))

    def pop_n_ids(self, n: int):
        """queue.py:87-95: the first min(length, n) ids; their slots become sentinels and the
        row is not re-sorted."""
        (batches, capacity) = self.indices.size()
        take = min(self.length, n)
        out = torch.empty((batches, take), dtype=torch.int32, device=self.indices.device)
        check(lib().vl_queue_pop(ptr(self.indices), ptr(self.distances), ctypes.c_int64(batches), capacity,
                                 self.length, n, ptr(out), stream_of(self.indices)), "vl_queue_pop")
        return out

    def size(self):
        return self.indices.size()

"""Host-side helpers with the reference's names (vectorlink_gpu/utils.py)."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
from torch import Tensor

from . import _lib
from ._lib import check, lib, ptr, stream_of
from .constants import MAXINT, primes_on
from .kernels import sort_pairs_


def generate_random_vectors(number_of_vectors: int, dimensions: int = 1536, device="cuda") -> Tensor:
    """utils.py:15-19."""
    return torch.nn.functional.normalize(
        torch.randn(number_of_vectors, dimensions, dtype=torch.float32, device=device), dim=1)


def primes(size: int, device="cuda") -> Tensor:
    """utils.py:22-23: the first `size` entries of the seed table.  Past the table's 965
    entries (which no reference configuration reaches) further offsets are derived from it:
    entry j is table[j mod 965] * (j div 965 + 1) + j, kept below 2^30."""
    table = primes_on(device)
    if size <= table.numel():
        return table.narrow(0, 0, size)
    j = torch.arange(size, device=table.device, dtype=torch.int64)
    ext = (table.long()[j % table.numel()] * (j // table.numel() + 1) + j) % (1 << 30)
    ext[: table.numel()] = table.long()
    return ext.to(torch.int32)


def generate_queue_circulants(batch_size: int, num_vecs: int, primes: Tensor, first_row: int = 0) -> Tensor:
    """utils.py:26-32: seeds[b, j] = sort_j(b + p_j) mod num_vecs; `first_row` (added) numbers the
    rows from there, for a batch that is a slice of a larger one."""
    indices = torch.arange(first_row, first_row + batch_size, device=primes.device, dtype=torch.int32)
    # the reference sorts every row of (b + p_j); adding b keeps the order, so sorting the offsets once
    # gives the same rows
    circulant_neighbors = indices.unsqueeze(1) + primes.sort().values.unsqueeze(0)
    return (circulant_neighbors % num_vecs).contiguous()


def generate_circulant_beams(num_vecs: int, primes: Tensor) -> Tensor:
    """utils.py:35-41: beams[i, j] = sort_j(i + p_j) mod num_vecs."""
    return generate_queue_circulants(num_vecs, num_vecs, primes)


def index_sort(beams: Tensor, beam_distances: Tensor):
    """utils.py:44-53: rows ordered by (distance, id); returns new tensors."""
    ns = beams.contiguous().clone()
    nds = beam_distances.contiguous().clone()
    sort_pairs_(ns, nds, dedup=False)
    return (ns, nds)


def queue_sort(beams: Tensor, beam_distances: Tensor):
    """utils.py:56-58 / queue.py:15-18: index_sort, punch repeated ids, sentinels last."""
    ns = beams.contiguous().clone()
    nds = beam_distances.contiguous().clone()
    sort_pairs_(ns, nds, dedup=True)
    return (ns, nds)


def dedup_sort(tensor: Tensor):
    """utils.py:85-89: each row sorted, repeats punched to MAXINT, sorted again."""
    assert tensor.dtype == torch.int32
    out = tensor.contiguous().clone()
    _lib.require_cuda(out)
    (b, e) = out.size()
    check(lib().vl_dedup_sort_ids(ptr(out), ctypes.c_int64(b), e, stream_of(out)), "vl_dedup_sort_ids")
    return out


def add_new_to_seen_(seen: Tensor, indices: Tensor) -> Optional[Tensor]:
    """utils.py:61-82: append the popped ids at the first column that is MAXINT in every
    row and dedup_sort the rows; None when no such column is left.  Like the reference this
    reads one number back from the device."""
    assert seen.dtype == torch.int32 and seen.is_contiguous()
    assert indices.dtype == torch.int32 and indices.is_contiguous()
    _lib.require_cuda(seen, indices)
    (dim1, dim2) = seen.size()
    scratch = torch.empty(max(dim2, 1) + 1, dtype=torch.int32, device=seen.device)
    first = scratch[-1:]
    check(lib().vl_seen_add(ptr(seen), ctypes.c_int64(dim1), dim2, ptr(indices), indices.size(1), ptr(scratch),
                            ptr(first), stream_of(seen)), "vl_seen_add")
    if int(first.item()) < 0:
        return None
    return seen

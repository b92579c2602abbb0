"""ctypes binding of libvlgpu.so, the C-ABI library holding the sm_100a kernels.

There is no CPU fallback: if the library is missing or a call is rejected, an exception is
raised.  Entry points and their argument meaning are declared in include/vlgpu.h.
"""
from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libvlgpu.so")

c_i32p = ctypes.POINTER(ctypes.c_int32)
c_f32p = ctypes.POINTER(ctypes.c_float)
c_u8p = ctypes.POINTER(ctypes.c_uint8)
c_u32p = ctypes.POINTER(ctypes.c_uint32)
c_intp = ctypes.POINTER(ctypes.c_int)

EXPORTS = [
    "vl_last_error", "vl_abi_version", "vl_calculate_distances", "vl_search_from_seeds", "vl_queue_insert",
    "vl_queue_pop", "vl_punchout_excluded", "vl_dedup_adjacent", "vl_sort_pairs", "vl_dedup_sort_ids",
    "vl_seen_add", "vl_seen_add_noalloc", "vl_prune", "vl_prune_rows", "vl_reverse_edges", "vl_connected_components", "vl_beam_search",
    "vl_beam_search_plan", "vl_knn_prepare", "vl_knn_tile",
]


class BeamParams(ctypes.Structure):
    """Mirror of `vl_beam_params` (include/vlgpu.h)."""
    _fields_ = [
        ("vectors", ctypes.c_void_p), ("n", ctypes.c_int64), ("dim", ctypes.c_int32), ("metric", ctypes.c_int32),
        ("graph", ctypes.c_void_p), ("graph_w", ctypes.c_int32), ("pvc", ctypes.c_int32),
        ("queries", ctypes.c_void_p), ("rows", ctypes.c_int64),
        ("seed_ids", ctypes.c_void_p), ("seed_dist", ctypes.c_void_p), ("seed_ld", ctypes.c_int64),
        ("seed_cols", ctypes.c_int32), ("sq_len", ctypes.c_int32), ("vq_len", ctypes.c_int32),
        ("seen_cap", ctypes.c_int32),
        ("out_ids", ctypes.c_void_p), ("out_dist", ctypes.c_void_p), ("out_ld", ctypes.c_int64),
        ("out_cols", ctypes.c_int32), ("n_iters", ctypes.c_int32), ("readahead", ctypes.c_int32),
        ("dump_last", ctypes.c_int32), ("exclude_w", ctypes.c_int32),
        ("exclude", ctypes.c_void_p), ("self_base", ctypes.c_int64), ("group_rows", ctypes.c_int64),
        ("changed_flags", ctypes.c_void_p), ("n_checks", ctypes.c_int32), ("memo_entries", ctypes.c_int32),
        ("group_full", ctypes.c_void_p), ("status", ctypes.c_void_p),
        ("memo", ctypes.c_void_p), ("memo_slots", ctypes.c_int64), ("stats", ctypes.c_void_p),
        ("flags", ctypes.c_int32), ("reserved", ctypes.c_int32), ("row_ticket", ctypes.c_void_p),
        ("group_row0", ctypes.c_int64),
    ]


_lib = None
LAUNCHES = 0   # kernels of this library launched so far (kept by the Python wrappers)


class VlError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    """The loaded library; raises if it was not built (python vectorlink-gpu_b200/build.py)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise VlError(f"{LIB_PATH} is missing: build it with `python vectorlink-gpu_b200/build.py` "
                          "(there is no CPU fallback)")
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.vl_last_error.restype = ctypes.c_char_p
        for name in EXPORTS[1:]:
            getattr(_lib, name).restype = ctypes.c_int
        P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
        _lib.vl_calculate_distances.argtypes = [P, L, I, P, L, P, I, P, I, P, P]
        _lib.vl_search_from_seeds.argtypes = [P, L, P, I, P, I, P, L, I, P, P, I, P, P]
        _lib.vl_queue_insert.argtypes = [P, P, L, I, I, P, P, I, P, I, P, P]
        _lib.vl_queue_pop.argtypes = [P, P, L, I, I, I, P, P]
        _lib.vl_punchout_excluded.argtypes = [P, P, L, L, L, I, P, I, P]
        _lib.vl_dedup_adjacent.argtypes = [P, P, L, I, P]
        _lib.vl_sort_pairs.argtypes = [P, P, L, I, I, P]
        _lib.vl_dedup_sort_ids.argtypes = [P, L, I, P]
        _lib.vl_seen_add.argtypes = [P, L, I, P, I, P, P, P]
        _lib.vl_seen_add_noalloc.argtypes = [P, L, I, P, I, P, P]
        _lib.vl_prune.argtypes = [P, P, L, I, I, P, P, I, P, P]
        _lib.vl_prune_rows.argtypes = [P, P, L, I, L, L, I, P, P, I, P, P]
        _lib.vl_reverse_edges.argtypes = [P, L, I, I, I, P, P, P, P, I, P, P, P]
        _lib.vl_connected_components.argtypes = [P, P, L, I, L, ctypes.c_float, P, P, P]
        _lib.vl_knn_prepare.argtypes = [P, L, I, P, I, P, P]
        _lib.vl_knn_tile.argtypes = [P, L, I, P, L, L, L, L, I, P, P, P]
        _lib.vl_beam_search.argtypes = [ctypes.POINTER(BeamParams), P]
        _lib.vl_beam_search_plan.argtypes = [ctypes.POINTER(BeamParams), c_intp, c_intp, c_intp]
    return _lib


KERNELS_PER_CALL = {"vl_dedup_adjacent": 2, "vl_seen_add": 3, "vl_seen_add_noalloc": 3, "vl_connected_components": 3}   # every other entry point launches one


def check(rc: int, what: str) -> None:
    global LAUNCHES
    if rc != 0:
        raise VlError(f"{what} failed ({rc}): {lib().vl_last_error().decode()}")
    LAUNCHES += KERNELS_PER_CALL.get(what, 1)


def ptr(t):
    """Device address of a tensor (None -> NULL)."""
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def stream_of(t: torch.Tensor):
    """torch's current stream on the tensor's device, as the void* the C ABI takes."""
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise VlError("vectorlink_gpu runs on CUDA tensors only (there is no CPU path); got a tensor on "
                          f"{t.device}")


_status = {}


def _device_key(device) -> torch.device:
    d = torch.device(device)
    if d.type == "cuda" and d.index is None:
        d = torch.device("cuda", torch.cuda.current_device())
    return d


def status_word(device) -> torch.Tensor:
    """One int32 per device that kernels OR VL_STATUS_* bits into."""
    key = _device_key(device)
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=key)
    return _status[key]


def read_status(device) -> int:
    """Reads and clears the status word (a device sync)."""
    s = status_word(device)
    v = int(s.item())
    if v:
        s.zero_()
    return v

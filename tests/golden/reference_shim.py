"""Loads the read-only reference package on a CPU-only machine (fixture generation only).

Used by ``make_golden.py`` on a machine that has a checkout of the reference
(``VL_REFERENCE_ROOT`` names it); nothing in the test-suite imports this at run time.

The reference cannot be imported without a GPU as shipped: ``constants.py`` builds its
prime table with ``device="cuda"``, ``ann.py`` imports ``datafusion`` (not installed),
and the kernels reach ``numba.cuda.syncthreads / shared / external_stream`` through the
``numba`` global, which the Numba CUDA simulator does not provide.  ``load_reference``
supplies exactly those missing pieces and returns the reference's own modules:

* ``mode="simulator"`` - the reference's real ``@cuda.jit`` kernels run in the Numba
  CUDA simulator.  Two repairs make their well-defined intent executable: the static
  shared buffer is zero-filled per block (``kernels.py:138`` reads slots nobody wrote
  when dim < 1024) and ``warp_reduce`` (``kernels.py:27-35``) runs in lockstep as a warp
  does on hardware (the simulator's free-running threads race through it otherwise).
* ``mode="host"`` - the reference's ``queue.py``, ``utils.py`` and ``ann.py`` and the launch
  wrappers of ``kernels.py`` run verbatim on CPU tensors; only the seven ``@cuda.jit``
  global kernels are replaced by launchable stand-ins backed by the C oracle, so that
  whole builds and searches finish in seconds instead of months.
"""
from __future__ import annotations

import os
import re
import sys
import threading
import types

REFERENCE_ROOT = os.environ.get("VL_REFERENCE_ROOT")



def _parse_constants(path):
    text = open(path).read()
    maxint = int(re.search(r"^MAXINT\s*=\s*(\d+)", text, re.M).group(1))
    maxfloat = float(re.search(r"^MAXFLOAT\s*=\s*([0-9.e+]+)", text, re.M).group(1))
    body = text[text.index("torch.tensor("):]
    body = body[body.index("[") + 1: body.index("]")]
    primes = [int(t) for t in re.findall(r"\d+", body)]
    return maxint, maxfloat, primes


def load_reference(mode: str):
    assert mode in ("simulator", "host")
    if not REFERENCE_ROOT or not os.path.isdir(os.path.join(REFERENCE_ROOT, "vectorlink_gpu")):
        raise RuntimeError("set VL_REFERENCE_ROOT to a checkout of vectorlink-ai/vectorlink-gpu")
    os.environ["NUMBA_ENABLE_CUDASIM"] = "1"
    import numpy as np
    import torch
    import numba
    import numba.cuda
    from numba.cuda.simulator import kernel as simkernel

    maxint, maxfloat, primes = _parse_constants(os.path.join(REFERENCE_ROOT, "vectorlink_gpu", "constants.py"))

    # constants.py:4-7,10-980 on the CPU; DEBUG=False switches the always-on log_time off
    consts = types.ModuleType("vectorlink_gpu.constants")
    consts.MAXINT = maxint
    consts.MAXFLOAT = maxfloat
    consts.DEVICE = "cpu"
    consts.DEBUG = False
    consts.PRIMES = torch.tensor(primes, dtype=torch.int32)
    sys.modules["vectorlink_gpu.constants"] = consts

    # ann.py:14 / datafusion.py:3-4 import a package that is not installed; it is I/O only
    dfm = types.ModuleType("datafusion")
    dfm.DataFrame = object
    dfm.col = lambda *a, **k: None
    dfm.SessionContext = object
    osm = types.ModuleType("datafusion.object_store")
    osm.GoogleCloud = object
    osm.AmazonS3 = object
    osm.LocalFileSystem = object
    dfm.object_store = osm
    sys.modules.setdefault("datafusion", dfm)
    sys.modules.setdefault("datafusion.object_store", osm)

    # kernels.py:16,48,100,119,138,217 call these through the `numba` global
    class _Shared:
        def __init__(self):
            self.lock = threading.Lock()
            self.blocks = {}

        def array(self, shape, dtype):
            from numba.core import types as nbtypes
            from numba.np import numpy_support
            if isinstance(dtype, nbtypes.Type):
                dtype = numpy_support.as_dtype(dtype)
            if shape == 0:
                return simkernel._get_kernel_context().shared.array(0, dtype)
            frame = sys._getframe(1)
            key = (id(threading.current_thread()._manager), frame.f_code.co_filename, frame.f_lineno)
            with self.lock:
                arr = self.blocks.get(key)
                if arr is None:
                    if len(self.blocks) > 64:
                        self.blocks.clear()
                    arr = np.zeros(shape, dtype)
                    self.blocks[key] = arr
                return arr

    numba.cuda.syncthreads = lambda: threading.current_thread().syncthreads()
    numba.cuda.shared = _Shared()
    numba.cuda.external_stream = lambda ptr: 0

    # simulator threads cannot store NumPy scalars into torch tensors: hand kernels views
    orig_call = simkernel.FakeCUDAKernel.__call__
    if not getattr(simkernel.FakeCUDAKernel, "_vl_patched", False):
        def call(self, *args):
            args = [a.detach().numpy() if isinstance(a, torch.Tensor) else a for a in args]
            # the simulator refuses strided views (Queue.insert passes column slices to
            # punchout_excluded_, kernels.py:471): run on a packed copy and write it back
            packed = [np.ascontiguousarray(a) if isinstance(a, np.ndarray) else a for a in args]
            result = orig_call(self, *packed)
            for a, c in zip(args, packed):
                if isinstance(a, np.ndarray) and c is not a:
                    a[...] = c
            return result
        simkernel.FakeCUDAKernel.__call__ = call
        simkernel.FakeCUDAKernel._vl_patched = True

    if REFERENCE_ROOT not in sys.path:
        sys.path.insert(0, REFERENCE_ROOT)
    for name in [m for m in sys.modules if m == "vectorlink_gpu" or m.startswith("vectorlink_gpu.")]:
        if name != "vectorlink_gpu.constants":
            del sys.modules[name]
    import vectorlink_gpu.kernels as K
    K.numba_current_stream = lambda: 0          # kernels.py:14-16 asks torch for a CUDA stream

    if mode == "simulator":
        def warp_reduce(vec, t):                # kernels.py:27-35 in lockstep
            me = threading.current_thread()
            for off in (32, 16, 8, 4, 2, 1):
                v = vec[t] + vec[t + off] if t < 32 else None
                me.syncthreads()
                if t < 32:
                    vec[t] = v
                me.syncthreads()
        K.warp_reduce = warp_reduce
        return types.SimpleNamespace(kernels=K, constants=consts)

    # ---- host mode: stand-ins for the seven global kernels, backed by the C oracle ----
    repo = os.path.abspath(os.path.join(os.path.dirname(__file__), "..", ".."))
    if repo not in sys.path:
        sys.path.insert(0, repo)
    import oracle
    import ctypes

    class Launch:
        def __init__(self, fn):
            self.fn = fn

        def __getitem__(self, cfg):
            return self

        def __call__(self, *args):
            self.fn(*[a.detach().numpy() if isinstance(a, torch.Tensor) else a for a in args])

    def k_distances(vectors, beams, out):                       # kernels.py:130-171
        out[...] = oracle.calculate_distances(vectors, beams)

    def k_search(q, visit, beams, vectors, idx_out, dist_out):  # kernels.py:204-257
        i, d = oracle.search_from_seeds(q, visit, beams, vectors)
        idx_out[...] = i
        dist_out[...] = d

    FLAG = np.int32(1 << 30)

    def k_mark(ids):                                            # kernels.py:314-330
        left = ids[:, :-1] & ~FLAG
        right = ids[:, 1:] & ~FLAG
        ids[:, 1:][left == right] |= FLAG

    def k_punch_pair(ids, dist):                                # kernels.py:333-349
        hit = (ids & FLAG) != 0
        ids[hit] = maxint
        dist[hit] = np.float32(maxfloat)

    def k_punch(ids):                                           # kernels.py:352-367
        ids[(ids & FLAG) != 0] = maxint

    def k_prune(beams, dist):                                   # kernels.py:409-438
        n, w = beams.shape
        oracle.lib().vlo_prune_punch(beams.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)),
                                     dist.ctypes.data_as(ctypes.POINTER(ctypes.c_float)),
                                     ctypes.c_int64(n), ctypes.c_int(w))

    def k_excluded(ids, dist, excl):                            # kernels.py:471-488
        oracle.punchout_excluded_(ids, dist, excl)

    K.cuda_distances_kernel = Launch(k_distances)
    K.cuda_search_from_seeds_kernel = Launch(k_search)
    K.mark_kernel = Launch(k_mark)
    K.punchout_pair_kernel = Launch(k_punch_pair)
    K.punchout_kernel = Launch(k_punch)
    K.prune_kernel = Launch(k_prune)
    K.punchout_excluded_kernel = Launch(k_excluded)

    import vectorlink_gpu.utils as U
    import vectorlink_gpu.queue as Q
    import vectorlink_gpu.ann as A
    return types.SimpleNamespace(kernels=K, utils=U, queue=Q, ann=A, constants=consts)

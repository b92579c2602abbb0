"""vl_seen_add_noalloc - the visited-list update for callers that cannot allocate.

Some users of the library have no allocator to call when they need the update: their
framework took all of the GPU's memory at start-up, or they run in a loop where cudaMalloc
(which stalls the whole device) is not allowed.  The entry point keeps its scratch flags in a
fixed array inside the library instead of a caller buffer.  This test drives it through the C
ABI and checks it against vl_seen_add on two calls in a row - the second call meets the flags
the first one left behind, which the entry point must clear itself.

The file sorts last so that a run stopping at the first failure has already run every other
test; it also passes when run alone in a fresh process.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
MAXINT = 2147483647


def _call_pair(lib, seen_a, seen_b, visit, scratch, first_a, first_b, stream):
    b, e = seen_a.shape
    v = visit.shape[1]
    rc = lib.vl_seen_add(seen_a.data_ptr(), b, e, visit.data_ptr(), v, scratch.data_ptr(), first_a.data_ptr(), stream)
    assert rc == 0, lib.vl_last_error()
    rc = lib.vl_seen_add_noalloc(seen_b.data_ptr(), b, e, visit.data_ptr(), v, first_b.data_ptr(), stream)
    assert rc == 0, lib.vl_last_error()


def test_noalloc_matches_the_scratch_variant_on_two_calls_in_a_row(built_lib):
    from vectorlink_gpu import _lib
    lib = _lib.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    rng = np.random.default_rng(42)
    b, e, v = 37, 320, 4
    # everything the calls touch is created before them: the entry point itself allocates nothing
    seen_a = torch.full((b, e), MAXINT, dtype=torch.int32, device=dev)
    seen_b = seen_a.clone()
    scratch = torch.empty(e + 1, dtype=torch.int32, device=dev)
    first_a = torch.zeros(1, dtype=torch.int32, device=dev)
    first_b = torch.zeros(1, dtype=torch.int32, device=dev)
    visits = []
    for step in range(2):
        vis = rng.integers(0, 5000, size=(b, v)).astype(np.int32)
        vis[rng.random((b, v)) < 0.15] = MAXINT          # rows whose visit queue ran dry
        if step == 1:
            vis[3, 0] = visits[0][3, 1]                  # a repeated id: must be deduplicated
        visits.append(vis)
    for step in range(2):
        vis = torch.from_numpy(visits[step]).to(dev)
        _call_pair(lib, seen_a, seen_b, vis, scratch, first_a, first_b, stream)
        torch.cuda.synchronize(dev)
        assert int(first_a.item()) == int(first_b.item()) == step * v   # integer results: equal
        assert torch.equal(seen_a, seen_b)
    got = seen_b.cpu().numpy()
    assert np.all(np.diff(got.astype(np.int64), axis=1) >= 0)           # rows ascending, sentinels last
    real = [set(r[r != MAXINT]) for r in got]
    want = [set(np.concatenate([visits[0][i], visits[1][i]])) - {MAXINT} for i in range(b)]
    assert real == want

    # a narrower list right after a wider one: stale flags beyond its width must not matter,
    # and a full list reports -1 with the same rows left untouched
    small_a = torch.arange(6, dtype=torch.int32, device=dev).repeat(5, 1).contiguous()
    small_b = small_a.clone()
    vis = torch.full((5, 2), 9, dtype=torch.int32, device=dev)
    _call_pair(lib, small_a, small_b, vis, scratch, first_a, first_b, stream)
    torch.cuda.synchronize(dev)
    assert int(first_a.item()) == int(first_b.item()) == -1
    assert torch.equal(small_a, small_b)


def test_noalloc_rejects_lists_wider_than_its_fixed_scratch(built_lib):
    from vectorlink_gpu import _lib
    lib = _lib.lib()
    dev = torch.device("cuda", 0)
    wide = torch.full((1, 4097), MAXINT, dtype=torch.int32, device=dev)
    vis = torch.zeros((1, 1), dtype=torch.int32, device=dev)
    first = torch.zeros(1, dtype=torch.int32, device=dev)
    rc = lib.vl_seen_add_noalloc(wide.data_ptr(), 1, 4097, vis.data_ptr(), 1, first.data_ptr(), None)
    assert rc != 0
    assert b"4096" in lib.vl_last_error()

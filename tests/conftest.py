import os
import sys

import numpy as np
import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
PKG_ROOT = os.path.join(ROOT, "vectorlink-gpu_b200")
for p in (ROOT, PKG_ROOT):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    # keep the no-allocation entry point's test last whatever the file order on disk
    items.sort(key=lambda it: 1 if "test_zz_" in it.nodeid else 0)


@pytest.fixture(scope="session")
def kat():
    return dict(np.load(os.path.join(GOLDEN, "kat_sim.npz")))


@pytest.fixture(scope="session")
def c1():
    return dict(np.load(os.path.join(GOLDEN, "c1_host.npz")))


@pytest.fixture(scope="session")
def small():
    return dict(np.load(os.path.join(GOLDEN, "small_host.npz")))


@pytest.fixture(scope="session")
def multi():
    """A three-round build by the reference's host code with two one-token repairs (the carried
    distances, stable final sorts): see make_golden.make_multi."""
    return dict(np.load(os.path.join(GOLDEN, "multi_host.npz")))


@pytest.fixture(scope="session")
def built_lib():
    """libvlgpu.so, compiled on demand (nvcc cross-compiles without a GPU)."""
    sys.path.insert(0, PKG_ROOT)
    import build as vl_build
    return vl_build.build()


def cfg_of(fixture):
    """The ANN keyword arguments a host fixture was generated with."""
    import oracle
    kw = {k[4:]: int(v) for k, v in fixture.items() if k.startswith("cfg_")}
    return oracle.make_config(**kw), kw


def assert_rows_match(ids, dist, ref_ids, ref_dist, rtol=1e-5, what=""):
    """Distances within `rtol` relative; ids equal except where the two orders differ only
    inside a run of distances that tie within `rtol` (then the id multisets of the run agree)."""
    ids, dist, ref_ids, ref_dist = map(np.asarray, (ids, dist, ref_ids, ref_dist))
    assert ids.shape == ref_ids.shape, (what, ids.shape, ref_ids.shape)
    tol = rtol * np.maximum(np.abs(ref_dist), 1e-30)
    assert np.all(np.abs(dist - ref_dist) <= tol), f"{what}: distance mismatch, max abs {np.abs(dist - ref_dist).max()}"
    bad_rows = np.nonzero((ids != ref_ids).any(axis=1))[0]
    for r in bad_rows:
        cols = np.nonzero(ids[r] != ref_ids[r])[0]
        for c in cols:
            d = ref_dist[r, c]
            run = np.abs(ref_dist[r] - d) <= rtol * max(abs(d), 1e-30)
            assert sorted(ids[r][run]) == sorted(ref_ids[r][run]), f"{what}: row {r} col {c}: ids differ outside a tie"

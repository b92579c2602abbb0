"""Cluster extraction (connected components of the thresholded neighbour graph).  The reference
has no such code to compare with (`ANN.clusters` is a stub there), so the CPU oracle is checked
against SciPy's connected_components, and the CUDA path against the oracle (equal labels)."""
import numpy as np
import pytest
import torch

import oracle

MAXINT = oracle.MAXINT


def random_graph(rng, nodes, w, p_sentinel=0.2, spread=None):
    """Neighbour lists that link node x to ids near x (many mid-sized components) plus distances."""
    spread = spread or max(2, nodes // 50)
    ids = (np.arange(nodes)[:, None] + rng.integers(-spread, spread + 1, (nodes, w))) % max(nodes, 1)
    ids = ids.astype(np.int32)
    ids[rng.random((nodes, w)) < p_sentinel] = MAXINT
    dist = rng.random((nodes, w)).astype(np.float32)
    dist[ids == MAXINT] = oracle.MAXFLOAT
    return ids, dist


def scipy_labels(ids, dist, threshold):
    from scipy.sparse import coo_matrix
    from scipy.sparse.csgraph import connected_components
    nodes, w = ids.shape
    rows = np.repeat(np.arange(nodes), w)
    cols = ids.reshape(-1).astype(np.int64)
    keep = (cols != MAXINT) & (cols >= 0) & (cols < nodes)
    if dist is not None:
        keep &= dist.reshape(-1) <= np.float32(threshold)
    g = coo_matrix((np.ones(keep.sum(), dtype=np.int8), (rows[keep], cols[keep])), shape=(nodes, nodes))
    _, comp = connected_components(g, directed=False)
    smallest = np.full(comp.max() + 1 if nodes else 0, nodes, dtype=np.int64)
    np.minimum.at(smallest, comp, np.arange(nodes))
    return smallest[comp].astype(np.int32)


CASES = [(1, 1, 0.5), (7, 3, 0.5), (500, 4, 0.3), (2000, 8, 0.1), (2000, 8, 0.9), (5000, 2, 1.0), (300, 40, 0.02)]


@pytest.mark.parametrize("nodes,w,threshold", CASES)
def test_oracle_components_match_scipy(nodes, w, threshold):
    rng = np.random.default_rng(nodes * 31 + w)
    ids, dist = random_graph(rng, nodes, w)
    labels, bad = oracle.connected_components(ids, dist, threshold)
    assert bad == 0
    assert np.array_equal(labels, scipy_labels(ids, dist, threshold))
    labels, _ = oracle.connected_components(ids)                      # no distances: every real id links
    assert np.array_equal(labels, scipy_labels(ids, None, 0.0))


def test_oracle_components_skip_and_count_bad_ids():
    ids = np.array([[1, -5], [MAXINT, 99], [MAXINT, MAXINT]], dtype=np.int32)
    labels, bad = oracle.connected_components(ids)
    assert bad == 2 and labels.tolist() == [0, 0, 2]


# ------------------------------------------------------------------ CUDA path (through the C ABI)

def t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to("cuda")


@pytest.mark.gpu
@pytest.mark.parametrize("nodes,w,threshold", CASES + [(200_000, 16, 0.05), (200_000, 16, 0.5)])
def test_cuda_components_equal_oracle(built_lib, nodes, w, threshold):
    from vectorlink_gpu.kernels import connected_components
    rng = np.random.default_rng(nodes * 17 + w)
    ids, dist = random_graph(rng, nodes, w)
    want, _ = oracle.connected_components(ids, dist, threshold)
    got = connected_components(t(ids), t(dist), threshold).cpu().numpy()
    assert np.array_equal(got, want)
    want, _ = oracle.connected_components(ids)
    assert np.array_equal(connected_components(t(ids)).cpu().numpy(), want)


@pytest.mark.gpu
def test_cuda_components_long_chain_and_star(built_lib):
    """Worst shapes for a union-find: one path through every node (deep trees while hooks race)
    and one hub that everybody links to (all hooks hit one root)."""
    from vectorlink_gpu.kernels import connected_components
    nodes = 300_000
    chain = np.full((nodes, 1), MAXINT, dtype=np.int32)
    chain[:-1, 0] = np.arange(1, nodes)
    assert int(connected_components(t(chain)).max()) == 0
    back = np.full((nodes, 1), MAXINT, dtype=np.int32)
    back[1:, 0] = np.arange(0, nodes - 1)
    assert int(connected_components(t(back)).max()) == 0
    star = np.full((nodes, 1), nodes - 1, dtype=np.int32)
    assert int(connected_components(t(star)).max()) == 0
    perm = np.random.default_rng(5).permutation(nodes).astype(np.int32)
    ring = np.empty((nodes, 1), dtype=np.int32)
    ring[perm, 0] = np.roll(perm, 1)
    ring[perm[0], 0] = MAXINT                       # open the ring: still one component
    assert int(connected_components(t(ring)).max()) == 0


@pytest.mark.gpu
def test_cuda_components_edge_cases(built_lib):
    from vectorlink_gpu import _lib
    from vectorlink_gpu.kernels import connected_components
    assert connected_components(torch.empty((0, 4), dtype=torch.int32, device="cuda")).numel() == 0
    assert connected_components(torch.empty((5, 0), dtype=torch.int32, device="cuda")).tolist() == [0, 1, 2, 3, 4]
    lonely = torch.full((6, 3), MAXINT, dtype=torch.int32, device="cuda")
    assert connected_components(lonely).tolist() == list(range(6))
    # ids outside [0, N) are skipped and reported in the status word, never dereferenced
    status = _lib.status_word(torch.device("cuda"))
    status.zero_()
    bad = t(np.array([[1, -5], [MAXINT, 99], [MAXINT, MAXINT]], dtype=np.int32))
    assert connected_components(bad).tolist() == [0, 0, 2]
    assert int(status.item()) & 1
    status.zero_()
    # NaN distances never link; the threshold is inclusive
    ids = t(np.array([[1], [2], [0]], dtype=np.int32))
    dist = t(np.array([[0.25], [np.nan], [0.5]], dtype=np.float32))
    assert connected_components(ids, dist, 0.25).tolist() == [0, 0, 2]
    assert connected_components(ids, dist, 0.5).tolist() == [0, 0, 0]


@pytest.mark.gpu
def test_cuda_components_on_queue_heads(built_lib):
    """Column slices of a wider tensor (the head of a Queue) are read in place."""
    from vectorlink_gpu.kernels import connected_components
    rng = np.random.default_rng(3)
    ids, dist = random_graph(rng, 4000, 12)
    want, _ = oracle.connected_components(ids[:, :5], dist[:, :5], 0.4)
    got = connected_components(t(ids)[:, :5], t(dist)[:, :5], 0.4).cpu().numpy()
    assert np.array_equal(got, want)


@pytest.mark.gpu
def test_cluster_labels_recover_planted_clusters(built_lib):
    """Well separated blobs: the components of the built graph under a threshold between the
    within-blob and between-blob distances are exactly the blobs."""
    from vectorlink_gpu import ANN
    g = torch.Generator().manual_seed(11)
    centres = torch.nn.functional.normalize(torch.randn(12, 64, generator=g), dim=1)
    member = torch.randint(0, 12, (3000,), generator=g)     # (a regular i % 12 layout would keep the prime seed
    first = torch.stack([(member == c).nonzero()[0, 0] for c in range(12)])      # offsets out of a row's own blob)
    expect = first[member].to(torch.int32)
    v = torch.nn.functional.normalize(centres[member] + 0.02 * torch.randn(3000, 64, generator=g), dim=1).cuda()
    ann = ANN(vectors=v, beam_size=16)
    labels = ann.cluster_labels(0.05)
    assert torch.equal(labels.cpu(), expect)                            # the smallest id of the row's blob
    want, _ = oracle.connected_components(ann.beams.cpu().numpy(), ann.distances.cpu().numpy(), 0.05)
    assert np.array_equal(labels.cpu().numpy(), want)
    queues = ann.clusters()
    from_queues = ann.cluster_labels(0.05, queues)
    head = slice(0, queues.length)
    want, _ = oracle.connected_components(queues.indices[:, head].cpu().numpy(), queues.distances[:, head].cpu().numpy(), 0.05)
    assert np.array_equal(from_queues.cpu().numpy(), want)
    # the blobs share no graph link, so a row whose seeds all fall into other blobs never reaches its
    # own and stays alone unless a neighbour's queue lists it: nearly all rows, not all
    assert (from_queues.cpu() == expect).float().mean() > 0.99

"""Pins the CPU oracle (oracle/neighbor_oracle.c) before anything trusts it:
against the reference's own known-answer tests, against fixtures produced by
running the reference (tests/golden), and, when it is built, against the
reference's compiled CPU path live on seeded inputs."""
import os

import numpy as np
import pytest
import torch

from oracle import neighbor_oracle as orc
from oracle import reference_cpu as refcpu

from _parity import (assert_knn_equal, assert_radius_equal, degrees, edge_set, load_golden)

GOLDEN = load_golden(os.path.join(os.path.dirname(__file__), "golden", "reference_cpu_cases.npz"))
DTYPES = [np.float32, np.float64]

SQUARE2 = [[-1, -1], [-1, +1], [+1, +1], [+1, -1]]


# ---- known answers held by the reference's tests -------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
def test_kat_knn(dtype):
    """test/test_knn.py:14-52."""
    x = np.array(SQUARE2 * 2, dtype=dtype)
    y = np.array([[1, 0], [-1, 0]], dtype=dtype)
    bx, by = np.array([0, 0, 0, 0, 1, 1, 1, 1]), np.array([0, 1])
    assert edge_set(orc.knn_api(x, y, 2)) == {(0, 2), (0, 3), (1, 0), (1, 1)}
    assert edge_set(orc.knn_api(x, y, 2, bx, by)) == {(0, 2), (0, 3), (1, 4), (1, 5)}
    assert edge_set(orc.knn_api(x, y, 2, bx, by, cosine=True)) == {(0, 2), (0, 3), (1, 4), (1, 5)}
    bx, by = np.array([0, 0, 0, 0, 2, 2, 2, 2]), np.array([0, 2])  # skipped batch id
    assert edge_set(orc.knn_api(x, y, 2, bx, by)) == {(0, 2), (0, 3), (1, 4), (1, 5)}


@pytest.mark.parametrize("dtype", DTYPES)
def test_kat_knn_graph(dtype):
    """test/test_knn.py:55-75 and the README's knn_graph example."""
    x = np.array(SQUARE2, dtype=dtype)
    t2s = {(0, 1), (0, 3), (1, 0), (1, 2), (2, 1), (2, 3), (3, 0), (3, 2)}
    assert edge_set(orc.knn_graph_api(x, 2, flow="target_to_source")) == t2s
    assert edge_set(orc.knn_graph_api(x, 2, flow="source_to_target")) == {(b, a) for a, b in t2s}


def test_kat_knn_graph_large_vs_kdtree():
    """test/test_knn.py:78-88."""
    import scipy.spatial

    x = torch.randn(1000, 3, generator=torch.Generator().manual_seed(0)).numpy()
    e = orc.knn_graph_api(x, 5, flow="target_to_source", loop=True)
    _, col = scipy.spatial.cKDTree(x).query(x, k=5)
    assert edge_set(e) == {(i, j) for i, ns in enumerate(col) for j in ns}


@pytest.mark.parametrize("dtype", DTYPES)
def test_kat_radius(dtype):
    """test/test_radius.py:23-61."""
    x = np.array(SQUARE2 * 2, dtype=dtype)
    y = np.array([[0, 0], [0, 1]], dtype=dtype)
    bx, by = np.array([0, 0, 0, 0, 1, 1, 1, 1]), np.array([0, 1])
    full = {(0, 0), (0, 1), (0, 2), (0, 3), (1, 1), (1, 2), (1, 5), (1, 6)}
    assert edge_set(orc.radius_api(x, y, 2, max_num_neighbors=4)) == full
    batched = {(0, 0), (0, 1), (0, 2), (0, 3), (1, 5), (1, 6)}
    assert edge_set(orc.radius_api(x, y, 2, bx, by, max_num_neighbors=4)) == batched
    bx, by = np.array([0, 0, 0, 0, 2, 2, 2, 2]), np.array([0, 2])
    assert edge_set(orc.radius_api(x, y, 2, bx, by, max_num_neighbors=4)) == batched


@pytest.mark.parametrize("dtype", DTYPES)
def test_kat_radius_graph(dtype):
    """test/test_radius.py:64-116."""
    x = np.array(SQUARE2, dtype=dtype)
    t2s = {(0, 1), (0, 3), (1, 0), (1, 2), (2, 1), (2, 3), (3, 0), (3, 2)}
    assert edge_set(orc.radius_graph_api(x, 2.5, flow="target_to_source")) == t2s
    assert edge_set(orc.radius_graph_api(x, 2.5, flow="source_to_target")) == {(b, a) for a, b in t2s}
    e = orc.radius_graph_api(x, 100, flow="source_to_target", max_num_neighbors=1)
    assert set(degrees(e, 1, 4).tolist()) == {1}
    dup = np.full((4, 2), -1, dtype=dtype)
    e = orc.radius_graph_api(dup, 100, flow="source_to_target", max_num_neighbors=1)
    assert set(degrees(e, 1, 4).tolist()) == {1}
    x8 = np.array(SQUARE2 * 2, dtype=dtype)
    b = np.array([0, 0, 0, 0, 1, 1, 1, 1])
    e = orc.radius_graph_api(x8, 100, batch=b, flow="source_to_target", max_num_neighbors=1)
    assert set(degrees(e, 1, 8).tolist()) == {1}
    assert [int(i / 4) for i in e[0]] == b.tolist()


def test_kat_radius_graph_large_vs_kdtree():
    """test/test_radius.py:119-133."""
    import scipy.spatial

    x = torch.randn(1000, 3, generator=torch.Generator().manual_seed(1)).numpy()
    e = orc.radius_graph_api(x, 0.5, flow="target_to_source", loop=True, max_num_neighbors=2000)
    col = scipy.spatial.cKDTree(x).query_ball_point(x, r=0.5)
    truth = {(i, j) for i, ns in enumerate(col) for j in ns}
    got = edge_set(e)
    # the kd-tree works in float64: allow only pairs that sit on the boundary
    for i, j in got ^ truth:
        d = np.linalg.norm(x[i].astype(np.float64) - x[j].astype(np.float64))
        assert abs(d - 0.5) < 1e-6


def test_segment_ptr_matches_bucketize():
    g = torch.Generator().manual_seed(3)
    for _ in range(20):
        b = torch.sort(torch.randint(0, 9, (int(torch.randint(1, 60, (1,), generator=g)),), generator=g)).values
        want = torch.bucketize(torch.arange(10), b)
        assert orc.segment_ptr(b.numpy(), 9).tolist() == want.tolist()


# ---- fixtures produced by running the reference ---------------------------------------------

def _run_oracle(c, fused):
    a, kind = c["args"], c["kind"]
    if kind == "knn":
        return orc.knn_api(c["x"], c["y"], a["k"], c["batch_x"], c["batch_y"],
                           batch_size=a["batch_size"], fused=fused)
    if kind == "knn_graph":
        return orc.knn_graph_api(c["x"], a["k"], c["batch"], a["loop"], a["flow"], fused=fused)
    if kind == "radius":
        return orc.radius_api(c["x"], c["y"], a["r"], c["batch_x"], c["batch_y"],
                              a["max_num_neighbors"], a["batch_size"], fused=fused)
    return orc.radius_graph_api(c["x"], a["r"], c["batch"], a["loop"], a["max_num_neighbors"],
                                a["flow"], fused=fused)


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_oracle_matches_golden(name, fused):
    c = GOLDEN[name]
    got = _run_oracle(c, fused)
    want = c["edge_index"]
    if c["kind"] == "knn":
        assert_knn_equal(got, want, c["x"], c["y"], query_row=0)
    elif c["kind"] == "knn_graph":
        q = 1 if c["args"]["flow"] == "source_to_target" else 0
        assert_knn_equal(got, want, c["x"], c["x"], query_row=q)
    elif c["untruncated"] is None:
        assert_radius_equal(got, want)
    else:
        # truncated: the CPU path keeps tree-order hits, the CUDA path the lowest x
        # indices; degrees agree and every kept edge is a true hit.
        q = 0 if c["kind"] == "radius" or c["args"]["flow"] == "target_to_source" else 1
        m = (c["y"] if c["kind"] == "radius" else c["x"]).shape[0]
        assert np.array_equal(degrees(got, q, m), degrees(want, q, m))
        full = edge_set(c["untruncated"])
        assert edge_set(got) <= full
        # "first hits in x-index order": got == per query the lowest neighbours of the full set
        nb = 1 - q
        fe = c["untruncated"]
        order = np.lexsort((fe[nb], fe[q]))
        fe = fe[:, order]
        rank = np.arange(fe.shape[1]) - np.searchsorted(fe[q], fe[q], side="left")
        keep = fe[:, rank < c["args"]["max_num_neighbors"]]
        assert edge_set(keep) == edge_set(got)


# ---- live against the compiled reference CPU path --------------------------------------------

needs_ref = pytest.mark.skipif(not refcpu.available(), reason="oracle/_ref is not built")


@needs_ref
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_oracle_vs_reference_cpu_knn_live(dtype):
    g = torch.Generator().manual_seed(11)
    sizes = [700, 0, 1300, 64]
    bx = torch.cat([torch.full((s,), i) for i, s in enumerate(sizes)])
    x = torch.randn(bx.numel(), 3, generator=g, dtype=dtype)
    ptr = torch.from_numpy(orc.segment_ptr(bx.numpy(), len(sizes)))
    want = refcpu.knn(x, x, ptr, ptr, 21).numpy()
    got = orc.knn(x.numpy(), x.numpy(), 21, ptr.numpy(), ptr.numpy())
    assert_knn_equal(got, want, x.numpy(), x.numpy())


@needs_ref
def test_oracle_vs_reference_cpu_radius_live():
    g = torch.Generator().manual_seed(12)
    x = torch.rand(6000, 3, generator=g)
    y = x[torch.randperm(6000, generator=g)[:1500].sort().values]
    want = refcpu.radius(x, y, None, None, 0.08, 100000).numpy()
    for fused in (True, False):
        got = orc.radius(x.numpy(), y.numpy(), 0.08, max_num_neighbors=100000, fused=fused)
        assert_radius_equal(got, want)

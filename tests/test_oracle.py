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


# ---- 16-bit restatement: pinned here against torch's own fp16 / bf16 tensor arithmetic (the same
# c10::Half / c10::BFloat16 definition the reference's kernels are instantiated with) and the
# reference's half-precision known-answer cases; on the GPU against the reference's CUDA kernels ----

def _dist16(x16, y16):
    """Per-operation rounded squared distances [m, n] computed with torch 16-bit tensors."""
    d = torch.zeros(y16.shape[0], x16.shape[0], dtype=x16.dtype)
    for j in range(x16.shape[1]):
        diff = (x16[None, :, j].float() - y16[:, None, j].float()).to(x16.dtype)
        prod = (diff.float() * diff.float()).to(x16.dtype)
        d = (d.float() + prod.float()).to(x16.dtype)
    return d


@pytest.mark.parametrize("kind,dtype", [("f16", torch.float16), ("bf16", torch.bfloat16)])
def test_oracle_16bit_matches_torch_16bit_arithmetic(kind, dtype):
    g = torch.Generator().manual_seed(16)
    x = (torch.randn(400, 3, generator=g) * 3).to(dtype)
    y = (torch.randn(30, 3, generator=g) * 3).to(dtype)
    d = _dist16(x, y)
    want = []
    for q in range(30):
        cand = [i for i in range(400) if float(d[q, i]) < float("inf")]
        want += [(q, i) for i in sorted(cand, key=lambda i: (float(d[q, i]), i))[:6]]
    got = orc.knn(x.float().numpy(), y.float().numpy(), 6, round16=kind)
    assert list(map(tuple, got.T.tolist())) == want
    r = 1.3
    r2 = float(torch.tensor(r * r, dtype=torch.float64).float().to(dtype))
    want = [(q, i) for q in range(30) for i in range(400) if float(d[q, i]) < r2]
    got = orc.radius(x.float().numpy(), y.float().numpy(), r, max_num_neighbors=4000, round16=kind)
    assert list(map(tuple, got.T.tolist())) == want
    got = orc.radius(x.float().numpy(), y.float().numpy(), r, max_num_neighbors=3, round16=kind)
    trunc = []
    for q in range(30):
        trunc += [e for e in want if e[0] == q][:3]
    assert list(map(tuple, got.T.tolist())) == trunc


def test_oracle_16bit_reference_known_answers():
    """test/test_knn.py:16-52 and test/test_radius.py:25-61 at half precision."""
    x = np.array([[-1, -1], [-1, 1], [1, 1], [1, -1]] * 2, dtype=np.float32)
    y = np.array([[1, 0], [-1, 0]], dtype=np.float32)
    px, py = np.array([0, 4, 8]), np.array([0, 1, 2])
    for kind in ("f16", "bf16"):
        e = orc.knn(x, y, 2, round16=kind)
        assert set(map(tuple, e.T.tolist())) == {(0, 2), (0, 3), (1, 0), (1, 1)}
        e = orc.knn(x, y, 2, px, py, round16=kind)
        assert set(map(tuple, e.T.tolist())) == {(0, 2), (0, 3), (1, 4), (1, 5)}
        e = orc.knn(x, y, 2, px, py, cosine=True, round16=kind)
        assert set(map(tuple, e.T.tolist())) == {(0, 2), (0, 3), (1, 4), (1, 5)}
    yr = np.array([[0, 0], [0, 1]], dtype=np.float32)
    for kind in ("f16", "bf16"):
        e = orc.radius(x, yr, 2, max_num_neighbors=4, round16=kind)
        assert set(map(tuple, e.T.tolist())) == {(0, 0), (0, 1), (0, 2), (0, 3), (1, 1), (1, 2), (1, 5), (1, 6)}
        e = orc.radius(x, yr, 2, px, py, max_num_neighbors=4, round16=kind)
        assert set(map(tuple, e.T.tolist())) == {(0, 0), (0, 1), (0, 2), (0, 3), (1, 5), (1, 6)}


# ---- nearest and farthest point sampling ------------------------------------------------------------

SQ8 = [[-1, -1], [-1, 1], [1, 1], [1, -1], [-2, -2], [-2, 2], [2, 2], [2, -2]]


def _fps_out_ptr(ptr, ratio, dtype=torch.float32):
    """Per-segment sample boundaries as csrc/cuda/fps_cuda.cu:83-86 forms them."""
    ptr = torch.as_tensor(ptr)
    deg = ptr[1:] - ptr[:-1]
    cnt = (deg.to(dtype) * torch.as_tensor(ratio, dtype=dtype)).ceil().long().cumsum(0)
    return torch.cat([torch.zeros(1, dtype=torch.long), cnt]).numpy()


def test_oracle_nearest_known_answers():
    """test/test_nearest.py:11-36."""
    x = np.array(SQ8, dtype=np.float32)
    y = np.array([[-1, 0], [1, 0], [-2, 0], [2, 0]], dtype=np.float32)
    out = orc.nearest(x, y, np.array([0, 4, 8]), np.array([0, 2, 4]))
    assert out.tolist() == [0, 0, 1, 1, 2, 2, 3, 3]
    assert orc.nearest(x, y).tolist() == [0, 0, 1, 1, 2, 2, 3, 3]
    assert orc.nearest(x.astype(np.float64), y.astype(np.float64)).tolist() == [0, 0, 1, 1, 2, 2, 3, 3]
    assert orc.nearest(x, y, round16="f16").tolist() == [0, 0, 1, 1, 2, 2, 3, 3]


def test_oracle_nearest_tie_order_follows_the_reference_reduction():
    """Equal minima: the reference's 1024-thread stride prefers the smaller (offset mod 1024)."""
    y = np.full((3000, 2), 5.0, dtype=np.float32)
    y[[2, 1025, 2050], :] = 0.0          # three points at distance 0 from the query
    x = np.zeros((1, 2), dtype=np.float32)
    assert orc.nearest(x, y).tolist() == [1025]      # offsets mod 1024: 2, 1, 2
    y[1025, :] = 5.0
    assert orc.nearest(x, y).tolist() == [2]         # (2, 2) before (2, 2050)
    # nothing below 1e38: index 0 as the kernel leaves it
    y[:] = np.inf
    assert orc.nearest(x, y).tolist() == [0]


def test_oracle_fps_known_answers():
    """test/test_fps.py:16-62 with random_start=False."""
    x = np.array(SQ8, dtype=np.float32)
    assert orc.fps(x, [0, 4, 8], _fps_out_ptr([0, 4, 8], 0.5)).tolist() == [0, 2, 4, 6]
    assert orc.fps(x, [0, 4, 8], _fps_out_ptr([0, 4, 8], [0.5, 0.5])).tolist() == [0, 2, 4, 6]
    assert sorted(orc.fps(x, [0, 8], _fps_out_ptr([0, 8], 0.5)).tolist()) == [0, 5, 6, 7]
    assert sorted(orc.fps(x.astype(np.float64), [0, 8], _fps_out_ptr([0, 8], 0.5)).tolist()) == [0, 5, 6, 7]
    assert sorted(orc.fps(x, [0, 8], _fps_out_ptr([0, 8], 0.5), round16="f16").tolist()) == [0, 5, 6, 7]


def test_oracle_fps_matches_reference_cpu_path():
    """csrc/cpu/fps_cpu.cpp on random clouds (no equal distances, so its first-maximum rule and
    unfused arithmetic pick the same points)."""
    g = torch.Generator().manual_seed(31)
    x = torch.randn(3 * 700, 3, generator=g)
    ptr = torch.tensor([0, 700, 1400, 2100])
    for ratio in (0.5, 0.1):
        want = refcpu.fps(x, ptr, torch.tensor(ratio), False)
        got = orc.fps(x.numpy(), ptr.numpy(), _fps_out_ptr(ptr, ratio))
        assert got.tolist() == want.tolist()
    xd = x.double()
    want = refcpu.fps(xd, ptr, torch.tensor(0.25, dtype=torch.float64), False)
    assert orc.fps(xd.numpy(), ptr.numpy(), _fps_out_ptr(ptr, 0.25, torch.float64)).tolist() == want.tolist()


def test_oracle_fps_tie_order_follows_the_reference_reduction():
    """All points beyond the 5e4 cap tie; the reference's 256-thread stride prefers the smaller
    (offset mod 256), then the lower index."""
    x = np.zeros((600, 1), dtype=np.float32)
    x[[3, 258, 515], 0] = 1000.0         # squared distance 1e6 -> clamped to 5e4, three-way tie
    out = orc.fps(x, [0, 600], np.array([0, 3]))
    assert out.tolist()[:2] == [0, 258]  # offsets mod 256: 3, 2, 3

"""GPU parity through the public API (the reference's Python signatures over
torch.ops.torch_cluster.*): the reference's own known-answer tests, the fixtures produced by
running the reference, and the Python-level oracle."""
import os

import numpy as np
import pytest
import torch

from oracle import neighbor_oracle as orc

from _parity import assert_knn_equal, assert_radius_equal, degrees, edge_set, load_golden

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
GOLDEN = load_golden(os.path.join(os.path.dirname(__file__), "golden", "reference_cpu_cases.npz"))
SQUARE2 = [[-1, -1], [-1, +1], [+1, +1], [+1, -1]]
ALL_DTYPES = [torch.half, torch.bfloat16, torch.float, torch.double]


def T(a, dtype=None):
    return None if a is None else torch.as_tensor(a, dtype=dtype).to(DEV)


def to_set(e):
    return set((i, j) for i, j in e.t().tolist())


# ---- the reference's known-answer tests, run against this library -----------------------------------

@pytest.mark.parametrize("dtype", [torch.half, torch.float, torch.double])
def test_knn(dtype):
    """test/test_knn.py:14-52."""
    from pytorch_cluster_b200 import knn

    x = T(SQUARE2 * 2, dtype)
    y = T([[1, 0], [-1, 0]], dtype)
    batch_x, batch_y = T([0, 0, 0, 0, 1, 1, 1, 1]), T([0, 1])
    assert to_set(knn(x, y, 2)) == {(0, 2), (0, 3), (1, 0), (1, 1)}
    jit = torch.jit.script(knn)
    assert to_set(jit(x, y, 2)) == {(0, 2), (0, 3), (1, 0), (1, 1)}
    assert to_set(knn(x, y, 2, batch_x, batch_y)) == {(0, 2), (0, 3), (1, 4), (1, 5)}
    assert to_set(knn(x, y, 2, batch_x, batch_y, cosine=True)) == {(0, 2), (0, 3), (1, 4), (1, 5)}
    batch_x, batch_y = T([0, 0, 0, 0, 2, 2, 2, 2]), T([0, 2])  # skipped batch id
    assert to_set(knn(x, y, 2, batch_x, batch_y)) == {(0, 2), (0, 3), (1, 4), (1, 5)}


@pytest.mark.parametrize("dtype", [torch.half, torch.float, torch.double])
def test_knn_graph(dtype):
    """test/test_knn.py:55-75."""
    from pytorch_cluster_b200 import knn_graph

    x = T(SQUARE2, dtype)
    t2s = {(0, 1), (0, 3), (1, 0), (1, 2), (2, 1), (2, 3), (3, 0), (3, 2)}
    s2t = {(b, a) for a, b in t2s}
    assert to_set(knn_graph(x, k=2, flow='target_to_source')) == t2s
    assert to_set(knn_graph(x, k=2, flow='source_to_target')) == s2t
    jit = torch.jit.script(knn_graph)
    assert to_set(jit(x, k=2, flow='source_to_target')) == s2t


def test_knn_graph_large():
    """test/test_knn.py:78-88."""
    import scipy.spatial

    from pytorch_cluster_b200 import knn_graph

    x = torch.randn(1000, 3, generator=torch.Generator().manual_seed(0))
    e = knn_graph(x.to(DEV), k=5, flow='target_to_source', loop=True)
    _, col = scipy.spatial.cKDTree(x.numpy()).query(x.numpy(), k=5)
    assert to_set(e.cpu()) == {(i, j) for i, ns in enumerate(col) for j in ns}


@pytest.mark.parametrize("dtype", ALL_DTYPES)
def test_radius(dtype):
    """test/test_radius.py:23-61."""
    from pytorch_cluster_b200 import radius

    x = T(SQUARE2 * 2, dtype)
    y = T([[0, 0], [0, 1]], dtype)
    batch_x, batch_y = T([0, 0, 0, 0, 1, 1, 1, 1]), T([0, 1])
    full = {(0, 0), (0, 1), (0, 2), (0, 3), (1, 1), (1, 2), (1, 5), (1, 6)}
    assert to_set(radius(x, y, 2, max_num_neighbors=4)) == full
    jit = torch.jit.script(radius)
    assert to_set(jit(x, y, 2, max_num_neighbors=4)) == full
    batched = {(0, 0), (0, 1), (0, 2), (0, 3), (1, 5), (1, 6)}
    assert to_set(radius(x, y, 2, batch_x, batch_y, max_num_neighbors=4)) == batched
    batch_x, batch_y = T([0, 0, 0, 0, 2, 2, 2, 2]), T([0, 2])
    assert to_set(radius(x, y, 2, batch_x, batch_y, max_num_neighbors=4)) == batched


@pytest.mark.parametrize("dtype", ALL_DTYPES)
def test_radius_graph(dtype):
    """test/test_radius.py:64-116."""
    from pytorch_cluster_b200 import radius_graph

    x = T(SQUARE2, dtype)
    t2s = {(0, 1), (0, 3), (1, 0), (1, 2), (2, 1), (2, 3), (3, 0), (3, 2)}
    s2t = {(b, a) for a, b in t2s}
    assert to_set(radius_graph(x, r=2.5, flow='target_to_source')) == t2s
    assert to_set(radius_graph(x, r=2.5, flow='source_to_target')) == s2t
    jit = torch.jit.script(radius_graph)
    assert to_set(jit(x, r=2.5, flow='source_to_target')) == s2t

    def deg(e):
        return set(torch.unique(e[1], return_counts=True)[1].tolist())

    assert deg(radius_graph(x, r=100, flow='source_to_target', max_num_neighbors=1)) == {1}
    dup = T([[-1, -1]] * 4, dtype)
    assert deg(radius_graph(dup, r=100, flow='source_to_target', max_num_neighbors=1)) == {1}
    x8 = T(SQUARE2 * 2, dtype)
    b = T([0, 0, 0, 0, 1, 1, 1, 1])
    e = radius_graph(x8, r=100, batch=b, flow='source_to_target', max_num_neighbors=1)
    assert deg(e) == {1}
    assert [int(i / 4) for i in e[0].tolist()] == b.tolist()


def test_radius_graph_large():
    """test/test_radius.py:119-133 (the kd-tree works in float64: boundary pairs may differ)."""
    import scipy.spatial

    from pytorch_cluster_b200 import radius_graph

    x = torch.randn(1000, 3, generator=torch.Generator().manual_seed(1))
    e = radius_graph(x.to(DEV), r=0.5, flow='target_to_source', loop=True, max_num_neighbors=2000)
    col = scipy.spatial.cKDTree(x.numpy()).query_ball_point(x.numpy(), r=0.5)
    truth = {(i, j) for i, ns in enumerate(col) for j in ns}
    for i, j in to_set(e.cpu()) ^ truth:
        assert abs(np.linalg.norm(x[i].double().numpy() - x[j].double().numpy()) - 0.5) < 1e-6


def test_readme_examples_order():
    """README.md:178-191, 207-220: the printed edge order of the 4-point examples."""
    from pytorch_cluster_b200 import knn_graph, radius_graph

    x = T([[-1., -1.], [-1., 1.], [1., -1.], [1., 1.]])
    batch = T([0, 0, 0, 0])
    e = knn_graph(x, k=2, batch=batch, loop=False)
    assert e.tolist() == [[1, 2, 0, 3, 0, 3, 1, 2], [0, 0, 1, 1, 2, 2, 3, 3]]
    e = radius_graph(x, r=2.5, batch=batch, loop=False)
    assert e.tolist() == [[1, 2, 0, 3, 0, 3, 1, 2], [0, 0, 1, 1, 2, 2, 3, 3]]


# ---- fixtures produced by running the reference's CPU path ---------------------------------------------

@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_matches_reference_fixture(name):
    import pytorch_cluster_b200 as pc

    c = GOLDEN[name]
    a, kind = c["args"], c["kind"]
    if kind == "knn":
        got = pc.knn(T(c["x"]), T(c["y"]), a["k"], T(c["batch_x"]), T(c["batch_y"]), batch_size=a["batch_size"])
        assert_knn_equal(got.cpu().numpy(), c["edge_index"], c["x"], c["y"], query_row=0)
    elif kind == "knn_graph":
        got = pc.knn_graph(T(c["x"]), a["k"], T(c["batch"]), loop=a["loop"], flow=a["flow"])
        q = 1 if a["flow"] == "source_to_target" else 0
        assert_knn_equal(got.cpu().numpy(), c["edge_index"], c["x"], c["x"], query_row=q)
    else:
        if kind == "radius":
            got = pc.radius(T(c["x"]), T(c["y"]), a["r"], T(c["batch_x"]), T(c["batch_y"]),
                            max_num_neighbors=a["max_num_neighbors"], batch_size=a["batch_size"])
            q, m = 0, c["y"].shape[0]
        else:
            got = pc.radius_graph(T(c["x"]), a["r"], T(c["batch"]), loop=a["loop"],
                                  max_num_neighbors=a["max_num_neighbors"], flow=a["flow"])
            q, m = (1 if a["flow"] == "source_to_target" else 0), c["x"].shape[0]
        got = got.cpu().numpy()
        if c["untruncated"] is None:
            assert_radius_equal(got, c["edge_index"])
        else:
            assert np.array_equal(degrees(got, q, m), degrees(c["edge_index"], q, m))
            assert edge_set(got) <= edge_set(c["untruncated"])


# ---- the Python-level oracle: exact arrays, order included ------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_api_equals_oracle_exactly(dtype):
    import pytorch_cluster_b200 as pc

    g = torch.Generator().manual_seed(5)
    sizes = [700, 0, 1300, 64, 9]
    batch = torch.cat([torch.full((s,), i) for i, s in enumerate(sizes)])
    x = torch.rand(batch.numel(), 3, generator=g, dtype=dtype)
    for loop in (False, True):
        for flow in ("source_to_target", "target_to_source"):
            got = pc.knn_graph(x.to(DEV), 12, batch.to(DEV), loop=loop, flow=flow).cpu().numpy()
            want = orc.knn_graph_api(x.numpy(), 12, batch.numpy(), loop, flow)
            assert np.array_equal(got, want)
            got = pc.radius_graph(x.to(DEV), 0.1, batch.to(DEV), loop=loop, flow=flow,
                                  max_num_neighbors=20).cpu().numpy()
            want = orc.radius_graph_api(x.numpy(), 0.1, batch.numpy(), loop, 20, flow)
            assert np.array_equal(got, want)
    y = torch.rand(300, 3, generator=g, dtype=dtype)
    by = torch.sort(torch.randint(0, 5, (300,), generator=g)).values
    got = pc.knn(x.to(DEV), y.to(DEV), 7, batch.to(DEV), by.to(DEV)).cpu().numpy()
    assert np.array_equal(got, orc.knn_api(x.numpy(), y.numpy(), 7, batch.numpy(), by.numpy()))
    got = pc.radius(x.to(DEV), y.to(DEV), 0.15, batch.to(DEV), by.to(DEV), batch_size=5).cpu().numpy()
    assert np.array_equal(got, orc.radius_api(x.numpy(), y.numpy(), 0.15, batch.numpy(), by.numpy(),
                                              batch_size=5))


def test_api_edge_cases():
    import pytorch_cluster_b200 as pc

    e = pc.knn(torch.empty(0, 3, device=DEV), torch.rand(4, 3, device=DEV), 3)
    assert e.shape == (2, 0) and e.dtype == torch.long
    e = pc.radius(torch.rand(4, 3, device=DEV), torch.empty(0, 3, device=DEV), 1.0)
    assert e.shape == (2, 0)
    x1 = torch.rand(50, device=DEV)  # 1-D input is treated as [N, 1]
    got = pc.knn(x1, x1, 3).cpu().numpy()
    assert np.array_equal(got, orc.knn_api(x1.cpu().numpy(), x1.cpu().numpy(), 3))
    with pytest.raises(RuntimeError, match="smaller than or equal to 100"):
        pc.knn(torch.rand(200, 3, device=DEV), torch.rand(4, 3, device=DEV), 101)
    with pytest.raises(RuntimeError, match="must be CUDA tensor"):
        pc.knn(torch.rand(20, 3), torch.rand(4, 3), 2)
    with pytest.raises(RuntimeError, match="Input mismatch"):
        pc.knn(torch.rand(20, 3, device=DEV), torch.rand(4, 2, device=DEV), 2)
    xt = torch.rand(3, 20, device=DEV).t()  # non-contiguous input is made contiguous by the wrapper
    got = pc.knn(xt, xt, 2).cpu().numpy()
    assert np.array_equal(got, orc.knn_api(xt.cpu().numpy(), xt.cpu().numpy(), 2))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_knn_graph_fused_tail_equals_reference_composition(dtype):
    """knn_graph runs as one operator; it must equal knn + flow swap + `row != col` mask + stack
    (torch_cluster/knn.py:131-144), also where exact duplicates push a point's own index out of its
    k + 1 nearest (then nothing is dropped for it) and where segments are shorter than k."""
    import pytorch_cluster_b200 as pc

    g = torch.Generator().manual_seed(9)
    base = torch.rand(300, 3, generator=g, dtype=dtype)
    x = torch.cat([base, base[:40], base[:40], base[:40], torch.rand(7, 3, generator=g, dtype=dtype)])
    batch = torch.cat([torch.zeros(420, dtype=torch.long), torch.full((7,), 2, dtype=torch.long)])
    for k in (1, 2, 5, 12):
        for loop in (False, True):
            for flow in ("source_to_target", "target_to_source"):
                got = pc.knn_graph(x.to(DEV), k, batch.to(DEV), loop=loop, flow=flow).cpu().numpy()
                want = orc.knn_graph_api(x.numpy(), k, batch.numpy(), loop, flow)
                assert np.array_equal(got, want), (k, loop, flow)
                found = pc.knn(x.to(DEV), x.to(DEV), k if loop else k + 1, batch.to(DEV), batch.to(DEV))
                row, col = (found[1], found[0]) if flow == "source_to_target" else (found[0], found[1])
                if not loop:
                    keep = row != col
                    row, col = row[keep], col[keep]
                assert np.array_equal(got, torch.stack([row, col]).cpu().numpy())


# ---- host-buffer entry point -----------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float, torch.double])
@pytest.mark.parametrize("flow", ["source_to_target", "target_to_source"])
def test_knn_graph_host_equals_device_call(dtype, flow):
    from pytorch_cluster_b200 import knn_graph, knn_graph_host

    g = torch.Generator().manual_seed(77)
    sizes = [900, 300, 1, 2000, 650, 40, 1200]
    x = torch.randn(sum(sizes), 3, generator=g, dtype=dtype)
    x[900:1201] = torch.randn(301, 3, generator=g, dtype=dtype)  # keep every segment >= k + 1 except the single row
    batch = torch.arange(len(sizes)).repeat_interleave(torch.tensor(sizes))
    k = 12
    want = knn_graph(x.to(DEV), k, batch.to(DEV), flow=flow).cpu()
    got = knn_graph_host(x.pin_memory(), k, batch.pin_memory(), flow=flow)  # one-row segment: the general route
    assert torch.equal(got, want)
    keep = batch != 2
    xr, br = x[keep].contiguous(), batch[keep].contiguous()
    want = knn_graph(xr.to(DEV), k, br.to(DEV), flow=flow).cpu()
    out = torch.empty(2, xr.shape[0] * k, dtype=torch.long).pin_memory()
    for groups in (1, 2, 4, 16):
        out.fill_(-7)
        got = knn_graph_host(xr.pin_memory(), k, br.pin_memory(), flow=flow, out=out, num_groups=groups)
        assert got.data_ptr() == out.data_ptr() and torch.equal(got, want)
    # no batch vector, unpinned input, other routes
    assert torch.equal(knn_graph_host(xr, k), knn_graph(xr.to(DEV), k).cpu())
    assert torch.equal(knn_graph_host(xr, k, br, loop=True), knn_graph(xr.to(DEV), k, br.to(DEV), loop=True).cpu())

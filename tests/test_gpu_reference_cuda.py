"""GPU parity against the reference's own CUDA kernels, compiled unmodified for sm_100a
(``oracle/_ref/ref_cluster_cuda.so``): the product's operators must return the very same
``edge_index`` tensors — values and order — as ``knn_cuda`` (csrc/cuda/knn_cuda.cu:86-135) and
``radius_cuda`` (csrc/cuda/radius_cuda.cu:44-96) on the same device tensors.  (``bench.py --impl reference-cuda`` times the two side by side.)"""
import pytest
import torch

from oracle import reference_cuda as refc

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not refc.available(), reason="oracle/_ref/ref_cluster_cuda.so not built")]

DEV = "cuda:0"


def _ptr(clouds, per):
    return torch.arange(clouds + 1, device=DEV, dtype=torch.long) * per


def _ours_knn(x, y, px, py, k, cosine=False):
    import pytorch_cluster_b200  # noqa: F401

    return torch.ops.torch_cluster.knn(x, y, px, py, k, cosine, 1)


def _ours_radius(x, y, px, py, r, max_nn, ignore_same):
    import pytorch_cluster_b200  # noqa: F401

    return torch.ops.torch_cluster.radius(x, y, px, py, r, max_nn, 1, ignore_same)


def _same(a, b):
    assert a.shape == b.shape, (a.shape, b.shape)
    if not torch.equal(a, b):
        bad = (a != b).any(0).nonzero().flatten()
        raise AssertionError(f"{bad.numel()} differing edges, first at {int(bad[0])}: "
                             f"{a[:, bad[0]].tolist()} vs {b[:, bad[0]].tolist()}")


@pytest.mark.parametrize("dtype", [torch.float, torch.double])
@pytest.mark.parametrize("dim", [1, 2, 3, 5, 8, 11, 16])
def test_knn_small_dims(dtype, dim):
    g = torch.Generator().manual_seed(100 + dim)
    x = torch.randn(3000, dim, generator=g).to(DEV, dtype)
    y = torch.randn(700, dim, generator=g).to(DEV, dtype)
    px = torch.tensor([0, 1000, 1000, 2500, 3000], device=DEV)
    py = torch.tensor([0, 300, 350, 600, 700], device=DEV)
    for k in (1, 7, 33, 100):
        _same(_ours_knn(x, y, px, py, k), refc.knn(x, y, px, py, k))
    _same(_ours_knn(x, y, None, None, 16), refc.knn(x, y, None, None, 16))


def test_knn_ties_and_duplicates():
    g = torch.Generator().manual_seed(7)
    x = torch.randint(0, 4, (4096, 3), generator=g).float().to(DEV)  # heavy ties on a 4^3 lattice
    px = _ptr(4, 1024)
    for k in (5, 21, 64):
        _same(_ours_knn(x, x, px, px, k), refc.knn(x, x, px, px, k))


def test_knn_graph_batched_full_size():
    """32 clouds x 4096 points, 3-D, op k = 21, fp32 and fp64."""
    g = torch.Generator().manual_seed(2)
    x = torch.randn(32 * 4096, 3, generator=g).to(DEV)
    p = _ptr(32, 4096)
    _same(_ours_knn(x, x, p, p, 21), refc.knn(x, x, p, p, 21))
    xd = x.double()
    _same(_ours_knn(xd, xd, p, p, 21), refc.knn(xd, xd, p, p, 21))


def test_knn_bipartite_two_clouds():
    """A quarter of the large bipartite configuration: 2 x (131072 points, 8192 queries), k = 32."""
    g = torch.Generator().manual_seed(3)
    x = (100 * torch.rand(2 * 131072, 3, generator=g)).to(DEV)
    y = (100 * torch.rand(2 * 8192, 3, generator=g)).to(DEV)
    px, py = _ptr(2, 131072), _ptr(2, 8192)
    _same(_ours_knn(x, y, px, py, 32), refc.knn(x, y, px, py, 32))


def test_knn_bipartite_full_size():
    """8 clouds x (131072 points, 8192 queries), 3-D in [0, 100)^3, k = 32."""
    g = torch.Generator().manual_seed(3)
    x = (100 * torch.rand(8 * 131072, 3, generator=g)).to(DEV)
    y = (100 * torch.rand(8 * 8192, 3, generator=g)).to(DEV)
    px, py = _ptr(8, 131072), _ptr(8, 8192)
    _same(_ours_knn(x, y, px, py, 32), refc.knn(x, y, px, py, 32))


@pytest.mark.parametrize("cosine", [False, True])
@pytest.mark.parametrize("dim", [32, 64, 128])
def test_knn_feature_space_tensor_path(cosine, dim):
    """16 clouds x 2048 points: the tensor-core candidate path against the reference's exact kernel."""
    g = torch.Generator().manual_seed(4)
    x = torch.randn(16 * 2048, dim, generator=g).to(DEV)
    p = _ptr(16, 2048)
    _same(_ours_knn(x, x, p, p, 21, cosine), refc.knn(x, x, p, p, 21, cosine))


@pytest.mark.parametrize("dim", [32, 64, 128])
def test_knn_graph_feature_space_in_one_call(dim):
    """knn_graph on feature vectors: the re-rank of the tensor-core candidates writes the final edge rows; equal
    to the reference's composition (k + 1 neighbours by its CUDA kernel, self matches dropped, rows by flow) —
    also where exact duplicates push a row out of its own list, which takes the general route."""
    import pytorch_cluster_b200 as pc

    g = torch.Generator().manual_seed(40 + dim)
    x = torch.randn(8 * 2048, dim, generator=g).to(DEV)
    batch = torch.arange(8, device=DEV).repeat_interleave(2048)
    p = _ptr(8, 2048)

    def composed(xx, flow, cosine=False):
        e = refc.knn(xx, xx, p, p, 21, cosine)          # row 0 = query, row 1 = neighbour
        e = e[:, e[0] != e[1]]
        return e.flip(0) if flow == "source_to_target" else e

    for flow in ("source_to_target", "target_to_source"):
        _same(pc.knn_graph(x, 20, batch, flow=flow), composed(x, flow))
        _same(pc.knn_graph(x, 20, batch, flow=flow, cosine=True), composed(x, flow, True))
    dup = x.clone()
    dup[:30] = dup[0]  # 30 copies of one row: some are pushed out of their own lists
    _same(pc.knn_graph(dup, 20, batch), composed(dup, "source_to_target"))
    from pytorch_cluster_b200 import cabi

    fast, odd = cabi.knn_graph(x, 20, p, True, workspace=True)
    assert odd == 0
    _same(fast, composed(x, "source_to_target"))


@pytest.mark.parametrize("cosine", [False, True])
def test_knn_general_dim(cosine):
    g = torch.Generator().manual_seed(14)
    x = torch.randn(5000, 19, generator=g).to(DEV)
    y = torch.randn(900, 19, generator=g).to(DEV)
    px = torch.tensor([0, 2000, 5000], device=DEV)
    py = torch.tensor([0, 500, 900], device=DEV)
    for k in (3, 40):
        _same(_ours_knn(x, y, px, py, k, cosine), refc.knn(x, y, px, py, k, cosine))


def _mixture(clouds, points, seed=5):
    g = torch.Generator().manual_seed(seed)
    centres = torch.rand(clouds, 32, 3, generator=g)
    pick = torch.randint(0, 32, (clouds, points), generator=g)
    x = torch.gather(centres, 1, pick.unsqueeze(-1).expand(-1, -1, 3)) + 0.02 * torch.randn(clouds, points, 3, generator=g)
    bg = torch.rand(clouds, points, generator=g) < 0.2
    x[bg] = torch.rand(int(bg.sum()), 3, generator=g)
    return x.clamp_(0, 0.99999994).reshape(clouds * points, 3).contiguous().to(DEV)


@pytest.mark.parametrize("max_nn", [1, 32, 64, 300])
@pytest.mark.parametrize("ignore_same", [False, True])
def test_radius_mixture(max_nn, ignore_same):
    x = _mixture(8, 8192)
    p = _ptr(8, 8192)
    _same(_ours_radius(x, x, p, p, 0.05, max_nn, ignore_same), refc.radius(x, x, p, p, 0.05, max_nn, ignore_same))
    xd = x.double()
    _same(_ours_radius(xd, xd, p, p, 0.05, max_nn, ignore_same),
          refc.radius(xd, xd, p, p, 0.05, max_nn, ignore_same))


def test_radius_untruncated_and_bipartite():
    x = _mixture(4, 8192)
    p = _ptr(4, 8192)
    _same(_ours_radius(x, x, p, p, 0.05, 8192, True), refc.radius(x, x, p, p, 0.05, 8192, True))
    keep = torch.cat([torch.randperm(8192, generator=torch.Generator().manual_seed(9))[:2048].sort().values + 8192 * c
                      for c in range(4)]).to(DEV)
    y = x[keep].contiguous()
    py = _ptr(4, 2048)
    _same(_ours_radius(x, y, p, py, 0.05, 64, False), refc.radius(x, y, p, py, 0.05, 64, False))


@pytest.mark.parametrize("dim", [1, 2, 6, 8, 12])
def test_radius_dims(dim):
    g = torch.Generator().manual_seed(200 + dim)
    x = torch.rand(6000, dim, generator=g).to(DEV)
    y = torch.rand(1500, dim, generator=g).to(DEV)
    px = torch.tensor([0, 2500, 2500, 6000], device=DEV)
    py = torch.tensor([0, 700, 800, 1500], device=DEV)
    r = 0.03 if dim == 1 else 0.25
    for max_nn in (16, 5000):
        _same(_ours_radius(x, y, px, py, r, max_nn, False), refc.radius(x, y, px, py, r, max_nn, False))


def _reference_radius_per_cloud(x, y, clouds, nx, ny, r, max_nn, ignore_same):
    """The reference's CUDA operator run cloud by cloud (ptr = None) with the indices shifted
    afterwards: clouds are independent, so this is its result on the whole batch, without its
    2 * M * max_num_neighbors int64 of padded output for the whole batch at once
    (csrc/cuda/radius_cuda.cu:75-78: 69 GB for 64 clouds x 8192 points with a cap of 8192)."""
    parts = []
    for c in range(clouds):
        e = refc.radius(x[c * nx:(c + 1) * nx], y[c * ny:(c + 1) * ny], None, None, r, max_nn, ignore_same)
        e[0] += c * ny
        e[1] += c * nx
        parts.append(e)
    return torch.cat(parts, dim=1)


def test_radius_graph_full_size_untruncated():
    """64 clouds x 8192 points, r = 0.05, neighbour cap 8192 (nothing is cut), self pairs skipped:
    the edge set of the whole batch, bit for bit."""
    x = _mixture(64, 8192)
    p = _ptr(64, 8192)
    ours = _ours_radius(x, x, p, p, 0.05, 8192, True)
    _same(ours, _reference_radius_per_cloud(x, x, 64, 8192, 8192, 0.05, 8192, True))
    assert ours.shape[1] > 40_000_000


@pytest.mark.parametrize("max_nn", [64, 8192])
def test_radius_bipartite_full_size(max_nn):
    """The queries are a sorted 25 % subset of every cloud (2048 of 8192 rows), all 64 clouds."""
    x = _mixture(64, 8192)
    keep = torch.cat([torch.randperm(8192, generator=torch.Generator().manual_seed(9 + c))[:2048].sort().values + 8192 * c
                      for c in range(64)]).to(DEV)
    y = x[keep].contiguous()
    p, py = _ptr(64, 8192), _ptr(64, 2048)
    _same(_ours_radius(x, y, p, py, 0.05, max_nn, False),
          _reference_radius_per_cloud(x, y, 64, 8192, 2048, 0.05, max_nn, False))


@pytest.mark.parametrize("max_nn", [16, 32])
def test_radius_sparse_hits_full_size(max_nn):
    """8 clouds of 131072 uniform points, 8192 queries each, about 15 hits per query: segments of at least
    2048 * max_num_neighbors points, for which the operator takes the screened scan (cap 16 truncates
    nearly half of the queries, cap 32 almost none)."""
    g = torch.Generator().manual_seed(3)
    x = (100 * torch.rand(8 * 131072, 3, generator=g)).to(DEV)
    y = (100 * torch.rand(8 * 8192, 3, generator=g)).to(DEV)
    px, py = _ptr(8, 131072), _ptr(8, 8192)
    ours = _ours_radius(x, y, px, py, 3.0, max_nn, False)
    _same(ours, refc.radius(x, y, px, py, 3.0, max_nn, False))
    assert ours.shape[1] > 500_000


def test_radius_graph_full_size_truncated():
    """The same 64 clouds with a cap of 64: the surviving hits are the reference's (lowest x rows)."""
    x = _mixture(64, 8192)
    p = _ptr(64, 8192)
    _same(_ours_radius(x, x, p, p, 0.05, 64, True), refc.radius(x, x, p, p, 0.05, 64, True))


# ---- 16-bit inputs: the reference instantiates knn for c10::Half and radius for c10::Half and
# c10::BFloat16; this library rounds every operation the same way ----

@pytest.mark.parametrize("dim", [1, 3, 8, 19, 64])
@pytest.mark.parametrize("cosine", [False, True])
def test_knn_half(dim, cosine):
    g = torch.Generator().manual_seed(500 + dim)
    x = torch.randn(3000, dim, generator=g).to(DEV).half()
    y = torch.randn(500, dim, generator=g).to(DEV).half()
    px = torch.tensor([0, 1200, 1200, 3000], device=DEV)
    py = torch.tensor([0, 200, 260, 500], device=DEV)
    for k in (1, 9, 40):
        _same(_ours_knn(x, y, px, py, k, cosine), refc.knn(x, y, px, py, k, cosine))
    big = (x * 100).half()  # squared distances overflow fp16
    _same(_ours_knn(big, big, px, px, 6, cosine), refc.knn(big, big, px, px, 6, cosine))


@pytest.mark.parametrize("dtype", [torch.half, torch.bfloat16])
@pytest.mark.parametrize("dim", [1, 3, 8, 19])
def test_radius_16bit(dtype, dim):
    g = torch.Generator().manual_seed(600 + dim)
    x = torch.rand(5000, dim, generator=g).to(DEV).to(dtype)
    y = torch.rand(900, dim, generator=g).to(DEV).to(dtype)
    px = torch.tensor([0, 2000, 5000], device=DEV)
    py = torch.tensor([0, 400, 900], device=DEV)
    r = 0.02 if dim == 1 else (0.2 if dim == 3 else 0.42 * dim ** 0.5)
    for max_nn in (5, 64, 5000):
        _same(_ours_radius(x, y, px, py, r, max_nn, False), refc.radius(x, y, px, py, r, max_nn, False))
    _same(_ours_radius(x, x, px, px, r, 32, True), refc.radius(x, x, px, px, r, 32, True))

"""The Morton-ordered kNN path for fp32 points of up to 8 features (csrc/spatial.cu, csrc/knn_spatial.cuh):
its ordering pass, and bit-exact equality of its results with the plain exact kernel (selected by
withholding the workspace) and with the oracle, on the inputs where a re-ordered, screened scan could
go wrong: ties and duplicates, data far from the origin, non-finite values, empty and uneven segments,
every feature count, both selection widths."""
import numpy as np
import pytest
import torch

from oracle import neighbor_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _cabi():
    from pytorch_cluster_b200 import cabi

    return cabi


def _ptr(sizes):
    return torch.tensor(np.concatenate([[0], np.cumsum(sizes)]), dtype=torch.long, device=DEV)


def _both(x, y, k, px=None, py=None, hint=0):
    c = _cabi()
    fast = c.knn_padded(x, y, k, px, py, workspace=True, max_segment_rows=hint)
    plain = c.knn_padded(x, y, k, px, py, workspace=False)
    assert fast[2] == plain[2], (fast[2], plain[2])
    assert torch.equal(fast[1], plain[1])
    assert torch.equal(fast[0], plain[0])
    return fast


# up to 16384 rows: one thread block; up to 2^19: bucket sort; above: exchange passes through global memory
@pytest.mark.parametrize("rows", [1, 7, 300, 1024, 1500, 4096, 16384, 16385, 40000, 200001, 524288, 600001])
def test_morton_order_one_segment(rows):
    g = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, 3, generator=g).to(DEV)
    order, keys, first = _cabi().morton_order(x)
    order, keys, first = order.cpu(), keys.cpu().long() & 0xffffffff, first.cpu()
    padded = (rows + 255) // 256 * 256
    assert first.tolist() == [0, padded]
    assert torch.equal(torch.sort(order[:rows].long()).values, torch.arange(rows))
    assert bool((order[rows:padded] == -1).all()) and bool((keys[rows:padded] == 0xffffffff).all())
    k = keys[:rows]
    assert bool((k[1:] >= k[:-1]).all())
    same = k[1:] == k[:-1]
    assert not bool((order[1:rows][same] < order[:rows - 1][same]).any())  # equal keys: by row


@pytest.mark.parametrize("dim", [1, 2, 3, 5, 8])
def test_morton_order_mixed_segments(dim):
    sizes = [3000, 0, 17000, 1, 1024, 70000, 16384, 500]
    g = torch.Generator().manual_seed(dim)
    x = torch.rand(sum(sizes), dim, generator=g).to(DEV)
    ptr = _ptr(sizes)
    for hint in (0, 70000):
        order, keys, first = _cabi().morton_order(x, ptr, hint)
        order, keys, first = order.cpu(), keys.cpu().long() & 0xffffffff, first.cpu().tolist()
        lo = 0
        for b, n in enumerate(sizes):
            assert first[b] % 256 == 0 and first[b + 1] - first[b] == (n + 255) // 256 * 256
            o, k = order[first[b]:first[b] + n], keys[first[b]:first[b] + n]
            assert torch.equal(torch.sort(o.long()).values, torch.arange(lo, lo + n))
            assert n < 2 or bool((k[1:] >= k[:-1]).all())
            lo += n


def test_spatial_knn_uneven_and_empty_segments():
    g = torch.Generator().manual_seed(0)
    sizes_x, sizes_y = [3000, 0, 5000, 1500, 20000], [100, 50, 0, 700, 3000]
    x = torch.randn(sum(sizes_x), 3, generator=g).to(DEV)
    y = torch.randn(sum(sizes_y), 3, generator=g).to(DEV)
    px, py = _ptr(sizes_x), _ptr(sizes_y)
    for k in (1, 16, 32, 33, 64):
        padded, counts, valid = _both(x, y, k, px, py)
        want = orc.knn(x.cpu().numpy(), y.cpu().numpy(), k, px.cpu().numpy(), py.cpu().numpy())
        got = padded[:, padded[1] >= 0].cpu().numpy()
        assert np.array_equal(got, want)
    _both(x, y, 16, px, py, hint=20000)


@pytest.mark.parametrize("dim", [1, 2, 3, 4, 5, 6, 7, 8])
def test_spatial_knn_feature_counts(dim):
    g = torch.Generator().manual_seed(50 + dim)
    x = torch.randn(6000, dim, generator=g).to(DEV)
    y = torch.randn(500, dim, generator=g).to(DEV)
    _both(x, y, 9)
    _both(x, x, 40)


def test_spatial_knn_ties_and_duplicates():
    g = torch.Generator().manual_seed(7)
    lattice = torch.randint(0, 6, (8192, 3), generator=g).float().to(DEV)  # many equal distances
    p = _ptr([4096, 4096])
    for k in (5, 21, 64):
        _both(lattice, lattice, k, p, p)
    same = torch.ones(4096, 3, device=DEV)  # every distance is zero: the lowest rows win
    padded, _, _ = _both(same, same[:100].contiguous(), 8)
    assert torch.equal(padded[1].view(100, 8), torch.arange(8, device=DEV).expand(100, 8))
    few = torch.rand(4096, 3, generator=g).to(DEV)
    few[::2] = few[0]  # half of the rows are one point
    _both(few, few, 21)


def test_spatial_knn_far_from_the_origin_and_extreme_values():
    g = torch.Generator().manual_seed(9)
    base = torch.rand(4096, 3, generator=g)
    for offset in (1e4, 1e6, -3e7):
        x = (base + offset).to(DEV)  # spacing of a few float ulps at the largest offsets
        _both(x, x, 8)
    x = torch.randn(4096, 3, generator=g)
    x[5, 0] = float("inf")
    x[9, 1] = float("nan")
    x[100] = 1e20
    x[200] = -1e20
    x = x.to(DEV)
    _both(x, x, 8)
    huge = (torch.randn(4096, 3, generator=g) * 1e18).to(DEV)  # squared distances overflow or exceed 1e10
    _both(huge, huge, 4)
    tiny = (torch.randn(4096, 3, generator=g) * 1e-30).to(DEV)  # squared distances underflow to zero
    _both(tiny, tiny, 4)
    wide = torch.randn(4096, 3, generator=g)
    wide[:, 0] *= 1e6  # one long axis: the box is far from a cube
    _both(wide.to(DEV), wide.to(DEV), 12)


def test_spatial_knn_fewer_points_than_k_and_single_segment_queries():
    g = torch.Generator().manual_seed(11)
    sizes_x, sizes_y = [5, 4000, 12000], [300, 300, 0]
    x = torch.rand(sum(sizes_x), 2, generator=g).to(DEV)
    y = torch.rand(sum(sizes_y), 2, generator=g).to(DEV)
    padded, counts, valid = _both(x, y, 16, _ptr(sizes_x), _ptr(sizes_y))
    assert bool((counts[:300] == 5).all()) and valid == 300 * 5 + 300 * 16


def test_spatial_knn_graph_in_one_kernel():
    c = _cabi()
    g = torch.Generator().manual_seed(13)
    sizes = [4096, 5000, 30000, 2048]
    x = torch.randn(sum(sizes), 3, generator=g).to(DEV)
    ptr = _ptr(sizes)
    for s2t in (True, False):
        fast, odd_fast = c.knn_graph(x, 20, ptr, s2t, workspace=True, max_segment_rows=30000)
        plain, odd_plain = c.knn_graph(x, 20, ptr, s2t, workspace=False)
        assert odd_fast == 0 and odd_plain == 0 and torch.equal(fast, plain)
    dup = x.clone()
    dup[:30] = dup[0]  # 30 copies of one point: some rows are pushed out of their own lists
    fast, odd_fast = c.knn_graph(dup, 20, ptr, True, workspace=True)
    plain, odd_plain = c.knn_graph(dup, 20, ptr, True, workspace=False)
    assert odd_fast == odd_plain and odd_fast > 0


def test_spatial_path_through_the_python_api():
    import pytorch_cluster_b200 as pc

    g = torch.Generator().manual_seed(17)
    sizes = [6000, 3000, 9000]
    x = torch.randn(sum(sizes), 3, generator=g)
    batch = torch.cat([torch.full((s,), i) for i, s in enumerate(sizes)])
    y, by = x[::7].contiguous(), batch[::7].contiguous()
    got = pc.knn(x.to(DEV), y.to(DEV), 12, batch.to(DEV), by.to(DEV)).cpu().numpy()
    assert np.array_equal(got, orc.knn_api(x.numpy(), y.numpy(), 12, batch.numpy(), by.numpy()))
    for flow in ("source_to_target", "target_to_source"):
        got = pc.knn_graph(x.to(DEV), 10, batch.to(DEV), flow=flow).cpu().numpy()
        assert np.array_equal(got, orc.knn_graph_api(x.numpy(), 10, batch.numpy(), flow=flow))
    assert torch.ops.torch_cluster.batch_info(batch.to(DEV)) == [3, 9000]
    assert torch.ops.torch_cluster.batch_info(torch.tensor([0, 0, 3, 3, 3, 7], device=DEV)) == [8, 3]


def test_large_segments_with_duplicates_and_outliers():
    """Segments above one sort block go through the bucket sort (sampled splitters): equal keys in bulk (half of a
    cloud is one point), and a bounding box blown up by a few far outliers so that nearly all points share a cell."""
    g = torch.Generator().manual_seed(23)
    x = torch.rand(120000, 3, generator=g)
    x[:60000] = x[0]
    x[-3:] = torch.tensor([[1e6, 0., 0.], [0., -1e6, 0.], [0., 0., 1e6]])
    x = x.to(DEV)
    order, keys, first = _cabi().morton_order(x)
    order, keys = order.cpu(), keys.cpu().long() & 0xffffffff
    assert torch.equal(torch.sort(order[:120000].long()).values, torch.arange(120000))
    k = keys[:120000]
    assert bool((k[1:] >= k[:-1]).all())
    y = x[::97].contiguous()
    _both(x, y, 16)
    ptr_x, ptr_y = _ptr([70000, 50000]), _ptr([700, y.shape[0] - 700])
    _both(x, y, 8, ptr_x, ptr_y, hint=70000)


def test_overlapping_segments_are_refused_not_overrun():
    """Segment pointers that are no partition of the rows (sizes adding up to more than the rows) do not fit the
    sorted copies: the ordering pass leaves its layout empty and the call is flagged, as a bounded wait that ran
    out would be — nothing is written out of bounds, and the operator raises."""
    g = torch.Generator().manual_seed(29)
    x = torch.rand(6000, 3, generator=g).to(DEV)
    y = torch.rand(300, 3, generator=g).to(DEV)
    px = torch.tensor([0, 3000, 2000, 6000], device=DEV)  # the third segment starts inside the first
    py = torch.tensor([0, 100, 200, 300], device=DEV)
    with pytest.raises(RuntimeError, match="overlap"):
        torch.ops.torch_cluster.knn(x, y, px, py, 8, False, 1)
    with pytest.raises(RuntimeError, match="overlap"):
        torch.ops.torch_cluster.knn_graph_edges(x, px, 8, False, True, False, 0)
    # the plain kernels take such pointers as the reference does
    _cabi().knn_padded(x, y, 8, px, py, workspace=False)
    # and the next regular call is unaffected
    _both(x, y, 8)

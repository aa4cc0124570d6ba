"""The screened radius scan for fp32 points of up to 8 features (csrc/radius_screen.cuh): bit-exact equality of
its edges with the plain exact kernel (selected by withholding the workspace) and with the oracle, on the inputs
where a screened scan could go wrong: hits in bulk (caps below and above the parked rows), truncation, the skipped own row, uneven / empty / tile-straddling segments, data far from the origin, non-finite
values, every feature count."""
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


def _both(x, y, r, px=None, py=None, max_nn=32, ignore=False):
    c = _cabi()
    fast = c.radius(x, y, r, px, py, max_nn, ignore, screen=True)
    plain = c.radius(x, y, r, px, py, max_nn, ignore, one_pass=False)
    assert fast.shape == plain.shape, (fast.shape, plain.shape)
    assert torch.equal(fast, plain)
    return fast


@pytest.mark.parametrize("dim", [1, 2, 3, 4, 5, 6, 7, 8])
def test_feature_counts(dim):
    g = torch.Generator().manual_seed(dim)
    x = torch.rand(6000, dim, generator=g).to(DEV)
    y = torch.rand(700, dim, generator=g).to(DEV)
    r = 0.5 * (40.0 / 6000) ** (1.0 / dim)  # a few dozen hits per query
    got = _both(x, y, r, max_nn=64)
    want = orc.radius(x.cpu().numpy(), y.cpu().numpy(), r, None, None, 64)
    assert np.array_equal(got.cpu().numpy(), want)
    _both(x, x, r, max_nn=16, ignore=True)


@pytest.mark.parametrize("max_nn", [1, 5, 32, 64, 300, 8192])
def test_caps_and_bulk_hits(max_nn):
    g = torch.Generator().manual_seed(max_nn)
    x = torch.rand(8192, 3, generator=g).to(DEV)
    for r in (0.03, 0.12, 0.5):  # about 1, 60 and 3000 hits per query
        for ignore in (False, True):
            _both(x, x, r, max_nn=max_nn, ignore=ignore)
    y = torch.rand(333, 3, generator=g).to(DEV)
    got = _both(x, y, 0.12, max_nn=max_nn)
    want = orc.radius(x.cpu().numpy(), y.cpu().numpy(), 0.12, None, None, max_nn)
    assert np.array_equal(got.cpu().numpy(), want)


def test_uneven_empty_and_straddling_segments():
    g = torch.Generator().manual_seed(3)
    sizes_x = [3000, 0, 5000, 1500, 700, 9000]
    sizes_y = [100, 50, 0, 7, 3000, 20]  # thread blocks of 64 queries straddle up to four segments
    x = torch.rand(sum(sizes_x), 3, generator=g).to(DEV)
    y = torch.rand(sum(sizes_y), 3, generator=g).to(DEV)
    px, py = _ptr(sizes_x), _ptr(sizes_y)
    for max_nn in (4, 64, 1000):
        got = _both(x, y, 0.1, px, py, max_nn)
        want = orc.radius(x.cpu().numpy(), y.cpu().numpy(), 0.1, px.cpu().numpy(), py.cpu().numpy(), max_nn)
        assert np.array_equal(got.cpu().numpy(), want)
    sizes = [2048, 4096, 1024, 5000]
    x = torch.rand(sum(sizes), 2, generator=g).to(DEV)
    p = _ptr(sizes)
    _both(x, x, 0.05, p, p, 32, ignore=True)


def test_far_from_the_origin_duplicates_and_extreme_values():
    g = torch.Generator().manual_seed(5)
    base = torch.rand(4096, 3, generator=g)
    for offset in (1e4, 1e6, -3e7):
        x = (base + offset).to(DEV)  # spacing of a few float ulps at the largest offsets
        _both(x, x, 0.1 if offset == 1e4 else 4.0, max_nn=64, ignore=True)
    same = torch.ones(4096, 3, device=DEV)  # every distance is zero
    out = _both(same, same[:100].contiguous(), 0.5, max_nn=8)
    assert torch.equal(out[1].view(100, 8), torch.arange(8, device=DEV).expand(100, 8))
    assert _both(same, same, 0.0, max_nn=8).shape[1] == 0  # the comparison is strict
    x = torch.rand(4096, 3, generator=g)
    x[5, 0] = float("inf")
    x[9, 1] = float("nan")
    x[100] = 1e20
    x = x.to(DEV)
    _both(x, x, 0.1, max_nn=64)  # non-finite centred norms: the segment is searched without the screen
    y = torch.rand(300, 3, generator=g)
    y[3, 2] = float("nan")
    y[4, 0] = float("-inf")
    y[5] = 1e25
    _both(base.to(DEV), y.to(DEV), 0.1, max_nn=64)
    _both(base.to(DEV), base.to(DEV), 1e20, max_nn=50)  # r * r overflows: every pair is a hit
    tiny = (torch.randn(4096, 3, generator=g) * 1e-30).to(DEV)  # squared distances underflow to zero
    _both(tiny, tiny, 1e-25, max_nn=20, ignore=True)
    first_bad = base.clone()
    first_bad[0, 0] = float("nan")  # the centre of the layout is the segment's first point
    _both(first_bad.to(DEV), base.to(DEV), 0.1, max_nn=64)


def test_through_the_operators():
    import pytorch_cluster_b200 as pc

    g = torch.Generator().manual_seed(7)
    sizes = [6000, 3000, 9000]
    x = torch.rand(sum(sizes), 3, generator=g)
    batch = torch.cat([torch.full((s,), i) for i, s in enumerate(sizes)])
    for flow in ("source_to_target", "target_to_source"):
        for max_nn in (16, 500):
            got = pc.radius_graph(x.to(DEV), 0.08, batch.to(DEV), loop=False, max_num_neighbors=max_nn, flow=flow)
            want = orc.radius_graph_api(x.numpy(), 0.08, batch.numpy(), False, max_nn, flow)
            assert np.array_equal(got.cpu().numpy(), want)
    y, by = x[::5].contiguous(), batch[::5].contiguous()
    got = pc.radius(x.to(DEV), y.to(DEV), 0.1, batch.to(DEV), by.to(DEV), max_num_neighbors=40)
    assert np.array_equal(got.cpu().numpy(), orc.radius_api(x.numpy(), y.numpy(), 0.1, batch.numpy(), by.numpy(), 40))
    # segments of at least 2048 * max_num_neighbors points: the operator itself takes the screened scan
    big = torch.rand(70000, 3, generator=g).to(DEV)
    pb = _ptr([34000, 36000])
    for same in (False, True):
        got = torch.ops.torch_cluster.radius(big, big, pb, pb, 0.03, 16, 1, same)
        assert torch.equal(got, _cabi().radius(big, big, 0.03, pb, pb, 16, same, one_pass=False))
    # a slice of the queries of one cloud: the pair skipped is the one with equal global rows
    cloud = big[:40000].contiguous()
    whole = torch.ops.torch_cluster.radius_part(cloud, cloud, None, None, 0.03, 16, True, 0, False)
    part = torch.ops.torch_cluster.radius_part(cloud, cloud[2000:5000].contiguous(), None, None, 0.03, 16, True, 2000,
                                               True)
    keep = (whole[0] >= 2000) & (whole[0] < 5000)
    want = whole[:, keep].flip(0).clone()
    want[1] -= 2000
    assert torch.equal(part, want)


def test_overlapping_segments_are_refused_not_overrun():
    """Segments of x that overlap so far that their chunk arrays would not fit the workspace: the layout is left empty
    and the status word says so; nothing is written out of bounds."""
    g = torch.Generator().manual_seed(11)
    x = torch.rand(6000, 3, generator=g).to(DEV)
    y = torch.rand(300, 3, generator=g).to(DEV)
    px = torch.tensor([0, 6000, 0, 6000], device=DEV)  # the whole set twice
    py = torch.tensor([0, 100, 200, 300], device=DEV)
    with pytest.raises(RuntimeError, match="overlap"):
        _cabi().radius(x, y, 0.1, px, py, 16, False, screen=True)
    plain = _cabi().radius(x, y, 0.1, px, py, 16, False, one_pass=False)  # the plain scan takes them as the reference does
    assert plain.shape[1] > 0
    _both(x, y, 0.1, max_nn=16)

"""GPU parity through the C ABI: the sm_100a kernels against the CPU oracle, bit for bit
(index work, so the bar is exact equality — including the order inside each query)."""
import numpy as np
import pytest
import torch

from oracle import neighbor_oracle as orc

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DT = {"f32": torch.float32, "f64": torch.float64}


def _segments(sizes):
    return torch.tensor(np.concatenate([[0], np.cumsum(sizes)]), dtype=torch.long)


def _data(seed, n, m, dim, dtype, scale=1.0, grid=None):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, dim, generator=g, dtype=dtype) * scale
    y = torch.randn(m, dim, generator=g, dtype=dtype) * scale
    if grid:  # snap to a coarse grid: many exactly equal distances
        x, y = torch.round(x * grid) / grid, torch.round(y * grid) / grid
    return x, y


def _check_knn(x, y, k, px=None, py=None, cosine=False):
    from pytorch_cluster_b200 import cabi as _cabi

    dx, dy = x.to(DEV), y.to(DEV)
    dpx = None if px is None else px.to(DEV)
    dpy = None if py is None else py.to(DEV)
    padded, counts, nvalid = _cabi.knn_padded(dx, dy, k, dpx, dpy, cosine)
    torch.cuda.synchronize()
    # the same without the optional workspace: the kernels that screen or use tensor cores need it,
    # so this exercises the plain exact kernels
    plain, plain_counts, plain_valid = _cabi.knn_padded(dx, dy, k, dpx, dpy, cosine, workspace=False)
    assert torch.equal(plain, padded) and torch.equal(plain_counts, counts) and plain_valid == nvalid
    want_col, _ = orc.knn_padded(x.numpy(), y.numpy(), k, None if px is None else px.numpy(),
                                 None if py is None else py.numpy(), cosine=cosine)
    m = y.shape[0]
    got = padded.cpu().numpy()
    assert np.array_equal(got[0].reshape(m, k), np.repeat(np.arange(m), k).reshape(m, k))
    got_col = got[1].reshape(m, k)
    bad = np.nonzero((got_col != want_col).any(axis=1))[0]
    assert bad.size == 0, (f"{bad.size} of {m} queries differ; first {bad[:5]}: got {got_col[bad[:3]]} "
                           f"want {want_col[bad[:3]]}")
    want_counts = (want_col >= 0).sum(1)
    assert np.array_equal(counts.cpu().numpy(), want_counts)
    assert nvalid == int(want_counts.sum())
    # compacted form
    e = _cabi.knn(dx, dy, k, dpx, dpy, cosine).cpu().numpy()
    want = orc.knn(x.numpy(), y.numpy(), k, None if px is None else px.numpy(),
                   None if py is None else py.numpy(), cosine=cosine)
    assert np.array_equal(e, want)


@pytest.mark.parametrize("dt", ["f32", "f64"])
@pytest.mark.parametrize("dim", [1, 2, 3, 4, 5, 6, 7, 8])
def test_knn_lowd_single_segment(dim, dt):
    x, y = _data(dim, 1500, 300, dim, DT[dt])
    _check_knn(x, y, 16)


@pytest.mark.parametrize("dt", ["f32", "f64"])
@pytest.mark.parametrize("k", [1, 2, 17, 21, 32, 33, 64, 65, 100])
def test_knn_lowd_all_k_ranges(k, dt):
    x, y = _data(100 + k, 2100, 130, 3, DT[dt])
    _check_knn(x, y, k)


@pytest.mark.parametrize("dt", ["f32", "f64"])
def test_knn_lowd_uneven_and_empty_segments(dt):
    sx = [300, 0, 17, 650, 5, 1, 2049, 0]
    sy = [40, 3, 0, 200, 31, 7, 65, 0]
    px, py = _segments(sx), _segments(sy)
    x, y = _data(7, sum(sx), sum(sy), 3, DT[dt])
    _check_knn(x, y, 9, px, py)      # segments with fewer than k points -> -1 slots, compaction
    _check_knn(x, y, 40, px, py)


@pytest.mark.parametrize("dt", ["f32", "f64"])
def test_knn_lowd_many_tiny_segments(dt):
    g = torch.Generator().manual_seed(5)
    sx = torch.randint(0, 12, (300,), generator=g).tolist()
    sy = torch.randint(0, 6, (300,), generator=g).tolist()
    x, y = _data(8, sum(sx), sum(sy), 2, DT[dt])
    _check_knn(x, y, 4, _segments(sx), _segments(sy))


@pytest.mark.parametrize("dt", ["f32", "f64"])
def test_knn_lowd_ties_keep_lower_index(dt):
    # coarse grid => lots of exactly equal distances, incl. exact duplicates of points
    x, y = _data(9, 3000, 200, 3, DT[dt], grid=4)
    _check_knn(x, y, 21)
    x2 = torch.cat([x[:500], x[:500]])  # duplicates
    _check_knn(x2, y, 32)


def test_knn_lowd_nan_and_huge_distances_are_skipped():
    x, y = _data(10, 700, 64, 3, torch.float32)
    x[5] = float("nan")
    x[17, 1] = float("inf")
    x[100:140] *= 1e6        # squared distance >= 1e10: never selected (initial bound 1e10)
    y[3, 0] = float("nan")   # a query that can select nothing
    _check_knn(x, y, 16)
    sx = [20, 680]
    _check_knn(x, y, 16, _segments(sx), _segments([10, 54]))


@pytest.mark.parametrize("dt", ["f32", "f64"])
def test_knn_lowd_long_segment_large_coordinates(dt):
    g = torch.Generator().manual_seed(11)
    x = (100 * torch.rand(40000, 3, generator=g)).to(DT[dt])
    y = (100 * torch.rand(257, 3, generator=g)).to(DT[dt])
    _check_knn(x, y, 32)


@pytest.mark.parametrize("dt", ["f32", "f64"])
@pytest.mark.parametrize("dim", [9, 16, 17, 33, 64, 100])
def test_knn_general_dim(dim, dt):
    x, y = _data(20 + dim, 900, 150, dim, DT[dt])
    _check_knn(x, y, 12)


@pytest.mark.parametrize("dt", ["f32", "f64"])
def test_knn_general_dim_batched_k_ranges(dt):
    sx, sy = [400, 0, 300, 37], [90, 4, 110, 9]
    x, y = _data(31, sum(sx), sum(sy), 24, DT[dt])
    for k in (5, 40, 100):
        _check_knn(x, y, k, _segments(sx), _segments(sy))


@pytest.mark.parametrize("dt", ["f32", "f64"])
@pytest.mark.parametrize("dim", [2, 3, 16, 64])
def test_knn_cosine(dim, dt):
    sx, sy = [500, 300], [100, 80]
    x, y = _data(40 + dim, sum(sx), sum(sy), dim, DT[dt])
    _check_knn(x, y, 10, cosine=True)
    _check_knn(x, y, 21, _segments(sx), _segments(sy), cosine=True)


def test_knn_cosine_zero_rows():
    x, y = _data(50, 400, 50, 8, torch.float32)
    x[7] = 0  # zero norm: distance is NaN and never selected
    y[2] = 0
    _check_knn(x, y, 6, cosine=True)


# ---- tensor-core candidate path (fp32, 32 <= D <= 128, D % 8 == 0, k <= 32, long segments) ---------------

@pytest.mark.parametrize("cosine", [False, True])
@pytest.mark.parametrize("dim,k", [(64, 21), (32, 32), (128, 8), (40, 1)])
def test_knn_tensor_path_equals_oracle(dim, k, cosine):
    sx, sy = [2048, 1500, 3000], [700, 300, 1029]
    x, y = _data(200 + dim, sum(sx), sum(sy), dim, torch.float32)
    _check_knn(x, y, k, _segments(sx), _segments(sy), cosine=cosine)


def test_knn_tensor_path_short_and_empty_segments():
    # some segments are far too short for k group minima: those queries are searched exhaustively
    sx, sy = [4000, 5, 0, 3000, 40, 2500], [300, 7, 3, 0, 50, 260]
    x, y = _data(301, sum(sx), sum(sy), 64, torch.float32)
    _check_knn(x, y, 16, _segments(sx), _segments(sy))
    _check_knn(x, y, 16, _segments(sx), _segments(sy), cosine=True)


def test_knn_tensor_path_ties_and_scale():
    # coarse grid => many exactly equal distances; large offsets => big |x| next to small distances
    x, y = _data(302, 6000, 500, 64, torch.float32, grid=2)
    _check_knn(x, y, 21)
    x2, y2 = _data(303, 5000, 300, 64, torch.float32)
    _check_knn(x2 + 50.0, y2 + 50.0, 21)
    _check_knn(torch.cat([x2[:2500], x2[:2500]]), y2, 20)   # exact duplicates


def test_knn_tensor_path_config4_slice():
    # four clouds of the EdgeConv configuration: 2048 points, 64 features, k = 20 (+1)
    g = torch.Generator().manual_seed(4)
    x = torch.randn(4 * 2048, 64, generator=g)
    ptr = torch.arange(0, 4 * 2048 + 1, 2048)
    _check_knn(x, x, 21, ptr, ptr)
    _check_knn(x, x, 21, ptr, ptr, cosine=True)


# ---- radius ---------------------------------------------------------------------------------------

def _check_radius(x, y, r, px=None, py=None, max_nn=32, ignore=False):
    from pytorch_cluster_b200 import cabi as _cabi

    dx, dy = x.to(DEV), y.to(DEV)
    dpx = None if px is None else px.to(DEV)
    dpy = None if py is None else py.to(DEV)
    got = _cabi.radius(dx, dy, r, dpx, dpy, max_nn, ignore).cpu().numpy()
    # the same through count + second scan (no one-pass scratch)
    two = _cabi.radius(dx, dy, r, dpx, dpy, max_nn, ignore, one_pass=False).cpu().numpy()
    assert np.array_equal(got, two)
    want = orc.radius(x.numpy(), y.numpy(), r, None if px is None else px.numpy(),
                      None if py is None else py.numpy(), max_nn, ignore)
    assert got.shape == want.shape, (got.shape, want.shape)
    assert np.array_equal(got, want)
    return got.shape[1]


@pytest.mark.parametrize("dt", ["f32", "f64"])
@pytest.mark.parametrize("dim", [1, 2, 3, 4, 5, 6, 7, 8])
def test_radius_lowd(dim, dt):
    g = torch.Generator().manual_seed(60 + dim)
    x = torch.rand(3000, dim, generator=g, dtype=DT[dt])
    y = torch.rand(400, dim, generator=g, dtype=DT[dt])
    r = 0.5 * (0.02 ** (1.0 / dim)) * (dim ** 0.5)
    e = _check_radius(x, y, r, max_nn=100000)
    assert e > 0


@pytest.mark.parametrize("dt", ["f32", "f64"])
@pytest.mark.parametrize("max_nn", [1, 8, 64, 100000])
def test_radius_truncation_keeps_first_hits(max_nn, dt):
    g = torch.Generator().manual_seed(70)
    x = torch.rand(5000, 3, generator=g, dtype=DT[dt])
    _check_radius(x, x[:700].clone(), 0.2, max_nn=max_nn)
    _check_radius(x, x.clone(), 0.1, max_nn=max_nn, ignore=True)   # radius_graph without self loops


@pytest.mark.parametrize("dt", ["f32", "f64"])
def test_radius_uneven_segments_and_same_index(dt):
    sx = [300, 0, 900, 12, 2100]
    sy = [100, 5, 0, 60, 500]
    g = torch.Generator().manual_seed(71)
    x = torch.rand(sum(sx), 3, generator=g, dtype=DT[dt])
    y = torch.rand(sum(sy), 3, generator=g, dtype=DT[dt])
    for ignore in (False, True):
        _check_radius(x, y, 0.2, _segments(sx), _segments(sy), max_nn=100000, ignore=ignore)
        _check_radius(x, y, 0.2, _segments(sx), _segments(sy), max_nn=5, ignore=ignore)


def test_radius_boundary_is_strict():
    # points at distance exactly r are not neighbours (test/test_radius.py:37-39 relies on it)
    x = torch.tensor([[0.0, 0.0], [3.0, 4.0], [5.0, 0.0], [4.9999995, 0.0]])
    y = torch.tensor([[0.0, 0.0]])
    from pytorch_cluster_b200 import cabi as _cabi

    got = _cabi.radius(x.to(DEV), y.to(DEV), 5.0, max_num_neighbors=10).cpu()
    assert got.t().tolist() == [[0, 0], [0, 3]]


@pytest.mark.parametrize("dt", ["f32", "f64"])
@pytest.mark.parametrize("dim", [9, 16, 40])
def test_radius_general_dim(dim, dt):
    g = torch.Generator().manual_seed(80 + dim)
    x = torch.rand(1200, dim, generator=g, dtype=DT[dt])
    y = torch.rand(300, dim, generator=g, dtype=DT[dt])
    r = 0.33 * dim ** 0.5
    e = _check_radius(x, y, r, max_nn=100000)
    assert e > 0
    _check_radius(x, y, r, max_nn=3)
    sx, sy = [700, 500], [100, 200]
    _check_radius(x, y, r, _segments(sx), _segments(sy), max_nn=100000, ignore=True)


# ---- small passes ----------------------------------------------------------------------------------

def test_segment_ptr_matches_bucketize():
    from pytorch_cluster_b200 import cabi as _cabi

    g = torch.Generator().manual_seed(90)
    for n, b in [(1, 1), (50, 9), (100000, 64), (5000, 4000)]:
        batch = torch.sort(torch.randint(0, b, (n,), generator=g)).values
        want = torch.bucketize(torch.arange(b + 1), batch)
        got = _cabi.segment_ptr(batch.to(DEV), b).cpu()
        assert torch.equal(got, want)
        assert got.tolist() == orc.segment_ptr(batch.numpy(), b).tolist()


@pytest.mark.parametrize("m", [1, 31, 2048, 2049, 1000003])
def test_exclusive_scan(m):
    from pytorch_cluster_b200 import cabi as _cabi

    g = torch.Generator().manual_seed(m)
    counts = torch.randint(0, 1000, (m,), generator=g, dtype=torch.int32)
    got = _cabi.exclusive_scan(counts.to(DEV)).cpu()
    want = torch.zeros(m + 1, dtype=torch.long)
    want[1:] = torch.cumsum(counts.long(), 0)
    assert torch.equal(got, want)


def test_argument_errors():
    from pytorch_cluster_b200 import _native

    lib = _native.cabi()
    x = torch.rand(10, 3, device=DEV)
    out = torch.empty(2, 10 * 101, dtype=torch.long, device=DEV)
    cnt = torch.empty(10, dtype=torch.int32, device=DEV)
    nv = torch.empty(1, dtype=torch.long, device=DEV)
    st = lib.b200c_knn(x.data_ptr(), x.data_ptr(), None, None, 1, 10, 10, 3, 101, 0, 0, out.data_ptr(),
                       cnt.data_ptr(), nv.data_ptr(), 0, None, 0, None)
    assert st == 1 and b"smaller than or equal to 100" in lib.b200c_last_error()


# ---- 16-bit inputs: every operation rounded to fp16 / bf16, as the reference's c10::Half /
# c10::BFloat16 instantiations compute (csrc/cuda/knn_cuda.cu:125, csrc/cuda/radius_cuda.cu:84-85) ----

T16 = {"f16": torch.float16, "bf16": torch.bfloat16}


def _check_knn16(x, y, k, kind, px=None, py=None, cosine=False):
    from pytorch_cluster_b200 import cabi as _cabi

    dx, dy = x.to(DEV), y.to(DEV)
    dpx = None if px is None else px.to(DEV)
    dpy = None if py is None else py.to(DEV)
    padded, counts, nvalid = _cabi.knn_padded(dx, dy, k, dpx, dpy, cosine)
    want_col, _ = orc.knn_padded(x.float().numpy(), y.float().numpy(), k, None if px is None else px.numpy(),
                                 None if py is None else py.numpy(), cosine=cosine, round16=kind)
    m = y.shape[0]
    got_col = padded.cpu().numpy()[1].reshape(m, k)
    bad = np.nonzero((got_col != want_col).any(axis=1))[0]
    assert bad.size == 0, (f"{bad.size} of {m} queries differ; first {bad[:5]}: got {got_col[bad[:3]]} "
                           f"want {want_col[bad[:3]]}")
    assert nvalid == int((want_col >= 0).sum())
    e = _cabi.knn(dx, dy, k, dpx, dpy, cosine).cpu().numpy()
    assert np.array_equal(e, orc.knn(x.float().numpy(), y.float().numpy(), k, None if px is None else px.numpy(),
                                     None if py is None else py.numpy(), cosine=cosine, round16=kind))


@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("dim", [1, 2, 3, 5, 8, 13, 16, 40])
def test_knn_16bit(dim, kind):
    x, y = _data(300 + dim, 1800, 260, dim, torch.float32)
    x, y = x.to(T16[kind]), y.to(T16[kind])
    _check_knn16(x, y, 12, kind)
    sx, sy = [500, 0, 9, 1291], [100, 10, 50, 100]
    _check_knn16(x, y, 33, kind, _segments(sx), _segments(sy))   # a segment with fewer than k points


@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("dim", [3, 24])
def test_knn_16bit_cosine(dim, kind):
    x, y = _data(330 + dim, 1500, 200, dim, torch.float32)
    x, y = x.to(T16[kind]), y.to(T16[kind])
    x[5] = 0  # a zero row: 0 / 0 = NaN, never selected
    _check_knn16(x, y, 10, kind, cosine=True)


def test_knn_16bit_overflow_and_large_k():
    """fp16 distances overflow to +inf beyond 65504: such points are never selected
    (`inf < inf` is false; the initial bound 1e10 narrows to +inf)."""
    x, y = _data(77, 900, 64, 3, torch.float32, scale=120.0)
    _check_knn16(x.half(), y.half(), 100, "f16")


def _check_radius16(x, y, r, kind, px=None, py=None, max_nn=32, ignore_same=False):
    from pytorch_cluster_b200 import cabi as _cabi

    dx, dy = x.to(DEV), y.to(DEV)
    dpx = None if px is None else px.to(DEV)
    dpy = None if py is None else py.to(DEV)
    e = _cabi.radius(dx, dy, r, dpx, dpy, max_nn, ignore_same).cpu().numpy()
    want = orc.radius(x.float().numpy(), y.float().numpy(), r, None if px is None else px.numpy(),
                      None if py is None else py.numpy(), max_nn, ignore_same, round16=kind)
    assert e.shape == want.shape, (e.shape, want.shape)
    assert np.array_equal(e, want)


@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("dim", [1, 3, 8, 20])
def test_radius_16bit(dim, kind):
    g = torch.Generator().manual_seed(400 + dim)
    x = torch.rand(2500, dim, generator=g).to(T16[kind])
    y = torch.rand(600, dim, generator=g).to(T16[kind])
    r = 0.02 if dim == 1 else (0.2 if dim == 3 else 0.45 * dim ** 0.5)
    _check_radius16(x, y, r, kind, max_nn=10000)
    _check_radius16(x, y, r, kind, max_nn=7)
    sx, sy = [1000, 0, 1500], [200, 100, 300]
    _check_radius16(x, y, r, kind, _segments(sx), _segments(sy), max_nn=40)
    _check_radius16(x, x, r, kind, max_nn=25, ignore_same=True)


# ---- knn_graph in one kernel (b200c_knn_graph) --------------------------------------------------------

@pytest.mark.parametrize("dt", ["f32", "f64"])
@pytest.mark.parametrize("s2t", [True, False])
@pytest.mark.parametrize("k", [1, 6, 20, 31, 32, 63, 99])
def test_knn_graph_one_kernel(k, s2t, dt):
    from pytorch_cluster_b200 import cabi as _cabi

    sizes = [700, 150, 1300]
    x, _ = _data(40 + k, sum(sizes), 1, 3, DT[dt])
    ptr = _segments(sizes)
    got, irregular = _cabi.knn_graph(x.to(DEV), k, ptr.to(DEV), s2t)
    assert irregular == 0
    batch = np.repeat(np.arange(3), sizes)
    want = orc.knn_graph_api(x.numpy(), k, batch, loop=False, flow="source_to_target" if s2t else "target_to_source")
    assert np.array_equal(got.cpu().numpy(), want)


def test_knn_graph_one_kernel_reports_irregular_queries():
    """Segments with fewer than k + 1 points, and rows pushed out of their own list by duplicates,
    are counted (and left to the general path), the rest is still written."""
    from pytorch_cluster_b200 import cabi as _cabi

    sizes = [5, 400]
    x, _ = _data(3, sum(sizes), 1, 2, torch.float32)
    got, irregular = _cabi.knn_graph(x.to(DEV), 8, _segments(sizes).to(DEV), True)
    assert irregular == 5
    want = orc.knn_graph_api(x.numpy(), 8, np.repeat(np.arange(2), sizes), loop=False)
    keep = want[1] >= 5  # edges of the regular segment
    assert np.array_equal(got.cpu().numpy()[:, 5 * 8:], want[:, keep])
    # 12 copies of one point, k = 4: a copy with a high index is not among its own 5 nearest
    x = torch.zeros(12, 3)
    _, irregular = _cabi.knn_graph(x.to(DEV), 4, None, True)
    assert irregular == 12 - 5


def test_knn_graph_one_kernel_unsupported_shapes():
    from pytorch_cluster_b200 import _native, cabi as _cabi

    x = torch.randn(100, 9).to(DEV)
    with pytest.raises(RuntimeError):
        _cabi.knn_graph(x, 4)
    assert "8 features" in _native.cabi().b200c_last_error().decode()


# ---- radius through the bit matrix of hits (b200c_radius_count_masks / _fill_masks) --------------------

@pytest.mark.parametrize("dt", ["f32", "f64"])
@pytest.mark.parametrize("dim", [1, 2, 3, 4, 7, 8])
def test_radius_masks_equal_count_and_fill(dim, dt):
    from pytorch_cluster_b200 import cabi as _cabi

    g = torch.Generator().manual_seed(500 + dim)
    sx, sy = [3000, 0, 1, 2500, 900], [700, 5, 0, 1100, 64]
    x = torch.rand(sum(sx), dim, generator=g, dtype=DT[dt])
    y = torch.rand(sum(sy), dim, generator=g, dtype=DT[dt])
    px, py = _segments(sx), _segments(sy)
    r = 0.01 if dim == 1 else (0.1 if dim <= 3 else 0.45)
    for max_nn, ignore in ((100000, False), (300, False), (5, True)):
        got = _cabi.radius_masks(x.to(DEV), y.to(DEV), r, px.to(DEV), py.to(DEV), max_nn, ignore).cpu().numpy()
        want = orc.radius(x.numpy(), y.numpy(), r, px.numpy(), py.numpy(), max_nn, ignore)
        assert got.shape == want.shape and np.array_equal(got, want)
    got = _cabi.radius_masks(x.to(DEV), x.to(DEV), r, None, None, 4000, True).cpu().numpy()
    assert np.array_equal(got, orc.radius(x.numpy(), x.numpy(), r, None, None, 4000, True))


def test_radius_masks_workspace_rules():
    from pytorch_cluster_b200 import _native

    lib = _native.cabi()
    hp = torch.tensor([0, 2000, 5000])
    # 3-D fp32: chunks of 1024 points = 32 words; 2000 points -> 2 chunks, 3000 -> 3
    words = 2000 * 2 * 32 + 3000 * 3 * 32
    assert lib.b200c_radius_mask_workspace_bytes(hp.data_ptr(), hp.data_ptr(), 2, 5000, 5000, 3, 0) == 256 + words * 4
    assert lib.b200c_radius_mask_workspace_bytes(hp.data_ptr(), hp.data_ptr(), 2, 5000, 5000, 9, 0) == 0
    assert lib.b200c_radius_mask_workspace_bytes(None, None, 1, 100, 50, 3, 0) == 256 + 50 * 32 * 4


# ---- large row counts ---------------------------------------------------------------------------------------

def test_knn_and_radius_on_16m_points():
    """16.7 M points in two segments (row numbers beyond 2^24, byte offsets beyond 2^27), k = 100:
    a sample of the queries against the oracle, and size-independent properties for all of them."""
    from pytorch_cluster_b200 import cabi as _cabi

    g = torch.Generator().manual_seed(99)
    n, m = 1 << 24, 2048
    x = torch.rand(n, 3, generator=g)
    y = torch.rand(m, 3, generator=g)
    px = torch.tensor([0, 5_000_000, n])
    py = torch.tensor([0, 1000, m])
    dx, dy, dpx, dpy = x.to(DEV), y.to(DEV), px.to(DEV), py.to(DEV)
    padded, counts, nvalid = _cabi.knn_padded(dx, dy, 100, dpx, dpy)
    assert nvalid == m * 100 and int(counts.min()) == 100
    col = padded[1].view(m, 100)
    lo = torch.where(torch.arange(m, device=DEV) < 1000, 0, 5_000_000)
    hi = torch.where(torch.arange(m, device=DEV) < 1000, 5_000_000, n)
    assert bool(((col >= lo[:, None]) & (col < hi[:, None])).all())          # neighbours stay in the segment
    d = ((dx[col.reshape(-1)] - dy.repeat_interleave(100, 0)) ** 2).sum(1).view(m, 100)
    assert bool((d[:, 1:] >= d[:, :-1] - 1e-9).all())                        # ascending distances
    sample = torch.cat([torch.arange(0, 16), torch.arange(1000, 1016)])
    ys = y[sample].contiguous()
    pys = torch.tensor([0, 16, 32])
    want, _ = orc.knn_padded(x.numpy(), ys.numpy(), 100, px.numpy(), pys.numpy())
    assert np.array_equal(col[sample.to(DEV)].cpu().numpy(), want)
    e = _cabi.radius(dx, dy, 0.004, dpx, dpy, 64, False).cpu().numpy()
    rows = np.isin(e[0], sample.numpy())
    want = orc.radius(x.numpy(), ys.numpy(), 0.004, px.numpy(), pys.numpy(), 64, False)
    remap = {int(s): i for i, s in enumerate(sample.tolist())}
    got = np.stack([np.array([remap[int(r)] for r in e[0][rows]], dtype=np.int64), e[1][rows]])
    assert np.array_equal(got, want)

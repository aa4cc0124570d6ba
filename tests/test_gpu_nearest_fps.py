"""GPU parity of ``nearest`` and ``fps``: the C ABI against the CPU oracle (exact index equality),
the reference's known-answer tests through the public API, and — when built — the reference's own
CUDA kernels compiled for sm_100a (csrc/cuda/nearest_cuda.cu, csrc/cuda/fps_cuda.cu)."""
import numpy as np
import pytest
import torch

from oracle import neighbor_oracle as orc
from oracle import reference_cuda as refc

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DT = {"f32": torch.float32, "f64": torch.float64, "f16": torch.float16, "bf16": torch.bfloat16}
SQ8 = [[-1, -1], [-1, 1], [1, 1], [1, -1], [-2, -2], [-2, 2], [2, 2], [2, -2]]
needs_ref = pytest.mark.skipif(not refc.available(), reason="oracle/_ref/ref_cluster_cuda.so not built")


def _ptr(sizes):
    return torch.tensor(np.concatenate([[0], np.cumsum(sizes)]), dtype=torch.long)


def _np(t):
    return t.float().numpy() if t.dtype in (torch.float16, torch.bfloat16) else t.numpy()


def _kind(dt):
    return dt if dt in ("f16", "bf16") else None


def _out_ptr(ptr, ratio, dtype):
    deg = ptr[1:] - ptr[:-1]
    cnt = (deg.to(dtype) * torch.as_tensor(ratio, dtype=dtype)).ceil().long().cumsum(0)
    return torch.cat([torch.zeros(1, dtype=torch.long), cnt])


# ---- nearest ----------------------------------------------------------------------------------------

@pytest.mark.parametrize("dt", ["f32", "f64", "f16", "bf16"])
@pytest.mark.parametrize("dim", [1, 2, 3, 8, 19])
def test_nearest_cabi(dim, dt):
    from pytorch_cluster_b200 import cabi

    g = torch.Generator().manual_seed(700 + dim)
    sx, sy = [900, 0, 40, 2100], [70, 0, 1, 1500]
    x = torch.randn(sum(sx), dim, generator=g).to(DT[dt])
    y = torch.randn(sum(sy), dim, generator=g).to(DT[dt])
    px, py = _ptr(sx), _ptr(sy)
    got = cabi.nearest(x.to(DEV), y.to(DEV), px.to(DEV), py.to(DEV)).cpu().numpy()
    want = orc.nearest(_np(x), _np(y), px.numpy(), py.numpy(), round16=_kind(dt))
    assert np.array_equal(got, want)
    got = cabi.nearest(x.to(DEV), y.to(DEV)).cpu().numpy()
    assert np.array_equal(got, orc.nearest(_np(x), _np(y), round16=_kind(dt)))


@pytest.mark.parametrize("dt", ["f32", "f16"])
def test_nearest_ties_follow_the_reference_order(dt):
    """Lattice points in segments longer than 1024 rows: many exactly equal minima."""
    from pytorch_cluster_b200 import cabi

    g = torch.Generator().manual_seed(9)
    x = torch.randint(0, 3, (500, 2), generator=g).to(DT[dt])
    y = torch.randint(0, 3, (2 * 2600, 2), generator=g).to(DT[dt])
    px, py = _ptr([250, 250]), _ptr([2600, 2600])
    got = cabi.nearest(x.to(DEV), y.to(DEV), px.to(DEV), py.to(DEV)).cpu().numpy()
    want = orc.nearest(_np(x), _np(y), px.numpy(), py.numpy(), round16=_kind(dt))
    assert np.array_equal(got, want)
    if refc.available():
        ref = refc.nearest(x.to(DEV), y.to(DEV), px.to(DEV), py.to(DEV)).cpu().numpy()
        assert np.array_equal(got, ref)


def test_nearest_nothing_admissible():
    from pytorch_cluster_b200 import cabi

    x = torch.zeros(5, 2)
    y = torch.full((9, 2), float("inf"))
    assert cabi.nearest(x.to(DEV), y.to(DEV)).tolist() == [0] * 5
    y = torch.full((9, 2), float("nan"))
    assert cabi.nearest(x.to(DEV), y.to(DEV)).tolist() == [0] * 5


@pytest.mark.parametrize("dtype", [torch.half, torch.float, torch.double])
def test_nearest_api_reference_known_answers(dtype):
    """test/test_nearest.py:11-66."""
    from pytorch_cluster_b200 import nearest

    x = torch.tensor(SQ8, dtype=dtype, device=DEV)
    y = torch.tensor([[-1, 0], [1, 0], [-2, 0], [2, 0]], dtype=dtype, device=DEV)
    L = lambda v: torch.tensor(v, device=DEV)  # noqa: E731
    assert nearest(x, y, L([0, 0, 0, 0, 1, 1, 1, 1]), L([0, 0, 1, 1])).tolist() == [0, 0, 1, 1, 2, 2, 3, 3]
    assert nearest(x, y).tolist() == [0, 0, 1, 1, 2, 2, 3, 3]
    assert torch.jit.script(nearest)(x, y).tolist() == [0, 0, 1, 1, 2, 2, 3, 3]
    with pytest.raises(ValueError):
        nearest(x, y, L([0, 0, 0, 0, 1, 1, 1, 1]), L([0, 0, 0, 0]))
    with pytest.raises(ValueError):
        nearest(x, y, L([0, 0, 0, 0, 1, 1, 1, 1]), None)
    with pytest.raises(ValueError):
        nearest(x, y, L([0, 0, 1, 1, 2, 2, 3, 3]), L([0, 1, 3, 3]))
    with pytest.raises(ValueError):
        nearest(x[:7], y, L([0, 0, 1, 0, 0, 0, 0]), L([0, 0, 1, 1]))
    with pytest.raises(ValueError):
        nearest(x, y, L([0, 0, 0, 0, 1, 1, 1, 1]), L([0, 0, 1, 0]))


@needs_ref
@pytest.mark.parametrize("dtype", [torch.half, torch.float, torch.double])
@pytest.mark.parametrize("dim", [1, 3, 16])
def test_nearest_equals_reference_cuda(dim, dtype):
    from pytorch_cluster_b200 import nearest

    g = torch.Generator().manual_seed(800 + dim)
    x = torch.randn(20000, dim, generator=g).to(DEV, dtype)
    y = torch.randn(3000, dim, generator=g).to(DEV, dtype)
    bx = torch.arange(4, device=DEV).repeat_interleave(5000)
    by = torch.tensor([0] * 100 + [1] * 1400 + [2] * 1000 + [3] * 500, device=DEV)
    px = torch.tensor([0, 5000, 10000, 15000, 20000], device=DEV)
    py = torch.tensor([0, 100, 1500, 2500, 3000], device=DEV)
    assert torch.equal(nearest(x, y, bx, by), refc.nearest(x, y, px, py))


# ---- farthest point sampling --------------------------------------------------------------------------

@pytest.mark.parametrize("dt", ["f32", "f64", "f16", "bf16"])
@pytest.mark.parametrize("dim", [1, 3, 7])
def test_fps_cabi(dim, dt):
    from pytorch_cluster_b200 import cabi

    g = torch.Generator().manual_seed(900 + dim)
    sizes = [1500, 0, 3, 1, 4097]
    x = torch.randn(sum(sizes), dim, generator=g).to(DT[dt])
    ptr = _ptr(sizes)
    rdt = torch.float32 if dt in ("f16", "bf16") else DT[dt]
    for ratio in (0.5, 0.07, 1.0):
        out_ptr = _out_ptr(ptr, ratio, rdt)
        got = cabi.fps(x.to(DEV), ptr.to(DEV), out_ptr.to(DEV)).cpu().numpy()
        want = orc.fps(_np(x), ptr.numpy(), out_ptr.numpy(), round16=_kind(dt))
        assert np.array_equal(got, want)
    # explicit start offsets
    start = torch.tensor([7, 0, 2, 0, 4000])
    out_ptr = _out_ptr(ptr, 0.25, rdt)
    got = cabi.fps(x.to(DEV), ptr.to(DEV), out_ptr.to(DEV), start.to(DEV)).cpu().numpy()
    assert np.array_equal(got, orc.fps(_np(x), ptr.numpy(), out_ptr.numpy(), start.numpy(), round16=_kind(dt)))


def test_fps_segment_in_shared_memory():
    """10000 three-dimensional fp32 points: too many for the register-resident path (8192), few
    enough for the shared-memory one; beside it segments of 1, 2 and 8192 points, ratio 1."""
    from pytorch_cluster_b200 import cabi

    g = torch.Generator().manual_seed(14)
    sizes = [10000, 1, 2, 8192]
    x = torch.randn(sum(sizes), 3, generator=g)
    ptr = _ptr(sizes)
    for out_ptr in (torch.tensor([0, 500, 501, 503, 903]), torch.tensor([0, 1, 2, 3, 4])):
        got = cabi.fps(x.to(DEV), ptr.to(DEV), out_ptr.to(DEV)).cpu().numpy()
        assert np.array_equal(got, orc.fps(x.numpy(), ptr.numpy(), out_ptr.numpy()))


@pytest.mark.parametrize("dt", ["f32", "f64"])
def test_fps_segment_larger_than_shared_memory(dt):
    """30000 three-dimensional points do not fit on chip: the kernel runs that segment from
    global memory; the small segment beside it stays in shared memory."""
    from pytorch_cluster_b200 import cabi

    g = torch.Generator().manual_seed(12)
    x = torch.rand(30000 + 500, 3, generator=g).to(DT[dt])
    ptr = _ptr([30000, 500])
    out_ptr = torch.tensor([0, 300, 400])
    got = cabi.fps(x.to(DEV), ptr.to(DEV), out_ptr.to(DEV)).cpu().numpy()
    assert np.array_equal(got, orc.fps(x.numpy(), ptr.numpy(), out_ptr.numpy()))


def test_fps_ties_follow_the_reference_order():
    from pytorch_cluster_b200 import cabi

    g = torch.Generator().manual_seed(13)
    x = torch.randint(0, 4, (2000, 2), generator=g).float()            # lattice: equal distances everywhere
    x = torch.cat([x, torch.randint(0, 2, (700, 2), generator=g).float() * 1000.0])  # beyond the 5e4 cap
    ptr, out_ptr = _ptr([2000, 700]), torch.tensor([0, 40, 60])
    got = cabi.fps(x.to(DEV), ptr.to(DEV), out_ptr.to(DEV)).cpu().numpy()
    assert np.array_equal(got, orc.fps(x.numpy(), ptr.numpy(), out_ptr.numpy()))
    if refc.available():
        ref = refc.fps(x.to(DEV), ptr.to(DEV), torch.tensor([0.02, 20 / 700 - 1e-4], device=DEV), False)
        assert ref.numel() == got.size and np.array_equal(got, ref.cpu().numpy())


@pytest.mark.parametrize("dtype", [torch.half, torch.float, torch.double])
def test_fps_api_reference_known_answers(dtype):
    """test/test_fps.py:16-62."""
    from pytorch_cluster_b200 import fps

    x = torch.tensor(SQ8, dtype=dtype, device=DEV)
    batch = torch.tensor([0, 0, 0, 0, 1, 1, 1, 1], device=DEV)
    ptr_list = [0, 4, 8]
    ptr = torch.tensor(ptr_list, device=DEV)
    assert fps(x, batch, random_start=False).tolist() == [0, 2, 4, 6]
    assert fps(x, batch, ratio=0.5, random_start=False).tolist() == [0, 2, 4, 6]
    assert fps(x, batch, ratio=torch.tensor(0.5, device=DEV), random_start=False).tolist() == [0, 2, 4, 6]
    assert fps(x, ptr=ptr_list, ratio=0.5, random_start=False).tolist() == [0, 2, 4, 6]
    assert fps(x, ptr=ptr, ratio=0.5, random_start=False).tolist() == [0, 2, 4, 6]
    assert fps(x, batch, ratio=torch.tensor([0.5, 0.5], device=DEV), random_start=False).tolist() == [0, 2, 4, 6]
    assert fps(x, random_start=False).sort()[0].tolist() == [0, 5, 6, 7]
    assert fps(x, ratio=0.5, random_start=False).sort()[0].tolist() == [0, 5, 6, 7]
    assert fps(x, ratio=torch.tensor([0.5], device=DEV), random_start=False).sort()[0].tolist() == [0, 5, 6, 7]


def test_fps_api_scripted_and_random_start():
    """test/test_fps.py:10-13, 65-74."""
    from pytorch_cluster_b200 import fps

    @torch.jit.script
    def fps2(x: torch.Tensor, ratio: torch.Tensor) -> torch.Tensor:
        return fps(x, None, ratio, False)

    x = torch.tensor(SQ8, dtype=torch.float, device=DEV)
    assert fps2(x, torch.tensor([0.5], device=DEV)).sort()[0].tolist() == [0, 5, 6, 7]
    n = 1024
    pos = torch.randn(2 * n, 3, device=DEV)
    batch = torch.cat([torch.zeros(n, dtype=torch.long), torch.ones(n, dtype=torch.long)]).to(DEV)
    idx = fps(pos, batch, ratio=0.5)
    assert idx.numel() == n and int(idx.min()) >= 0 and int(idx.max()) < 2 * n
    assert int(idx[: n // 2].max()) < n <= int(idx[n // 2:].min())
    assert idx.unique().numel() == n  # distinct points


@needs_ref
@pytest.mark.parametrize("dtype", [torch.half, torch.float, torch.double])
def test_fps_equals_reference_cuda(dtype):
    from pytorch_cluster_b200 import fps

    g = torch.Generator().manual_seed(41)
    x = torch.randn(6 * 4096, 3, generator=g).to(DEV, dtype)
    ptr = torch.arange(7, device=DEV) * 4096
    for ratio in (0.25, 0.01):
        r = torch.tensor(ratio, dtype=dtype, device=DEV)
        assert torch.equal(fps(x, ptr=ptr, ratio=r, random_start=False), refc.fps(x, ptr, r, False))
    xl = torch.rand(40000, 3, generator=g).to(DEV, dtype)   # one segment larger than shared memory
    pl = torch.tensor([0, 40000], device=DEV)
    r = torch.tensor(0.005, dtype=dtype, device=DEV)
    assert torch.equal(fps(xl, ptr=pl, ratio=r, random_start=False), refc.fps(xl, pl, r, False))


# ---- one large segment on many SMs (b200c_fps_large_segment) ------------------------------------------

@pytest.mark.parametrize("n,dim", [(8193, 3), (20000, 3), (131072, 3), (300000, 2), (9000, 7)])
def test_fps_large_segment_cabi(n, dim):
    from pytorch_cluster_b200 import cabi

    g = torch.Generator().manual_seed(1000 + dim)
    pad = 37  # the segment does not start at row 0
    x = torch.rand(pad + n, dim, generator=g)
    count = 200
    got, status = cabi.fps_large_segment(x.to(DEV), pad, n, count, start_offset=5)
    assert status == 0
    want = orc.fps(x.numpy(), [0, pad, pad + n], [0, 0, count], np.array([0, 5]))
    assert np.array_equal(got.cpu().numpy(), want)


def test_fps_large_segment_ties():
    """Lattice points: many equal maxima across the thread blocks."""
    from pytorch_cluster_b200 import cabi

    g = torch.Generator().manual_seed(17)
    x = torch.randint(0, 6, (40000, 3), generator=g).float()
    got, status = cabi.fps_large_segment(x.to(DEV), 0, 40000, 150)
    assert status == 0
    assert np.array_equal(got.cpu().numpy(), orc.fps(x.numpy(), [0, 40000], [0, 150]))


def test_fps_api_mixes_small_and_large_segments():
    from pytorch_cluster_b200 import fps

    g = torch.Generator().manual_seed(18)
    sizes = [3000, 50000, 8192, 1, 9000]
    x = torch.rand(sum(sizes), 3, generator=g)
    ptr = _ptr(sizes)
    ratio = torch.tensor([0.05, 0.004, 0.01, 1.0, 0.02])
    got = fps(x.to(DEV), ptr=ptr.to(DEV), ratio=ratio.to(DEV), random_start=False).cpu().numpy()
    out_ptr = torch.cat([torch.zeros(1, dtype=torch.long),
                         ((ptr[1:] - ptr[:-1]).float() * ratio).ceil().long().cumsum(0)])
    assert np.array_equal(got, orc.fps(x.numpy(), ptr.numpy(), out_ptr.numpy()))
    idx = fps(x.to(DEV), ptr=ptr.to(DEV), ratio=0.01)  # random start: valid, distinct, per segment
    assert idx.unique().numel() == idx.numel()
    if refc.available():
        r = torch.tensor(0.003, device=DEV)
        big = torch.rand(100000, 3, generator=g).to(DEV)
        bp = torch.tensor([0, 100000], device=DEV)
        assert torch.equal(fps(big, ptr=bp, ratio=r, random_start=False), refc.fps(big, bp, r, False))


def test_fps_api_segment_beyond_the_many_sm_kernel_next_to_a_mid_size_one():
    """One call holding a segment the many-SM kernel takes (more than 8192 points) and one larger than
    all SMs together hold: the second runs from global memory in a call of its own, and a list of
    boundaries gives the same samples as a tensor."""
    from pytorch_cluster_b200 import _native, fps

    cap = _native.cabi().b200c_fps_large_segment_max_points(3, 0)
    assert cap >= 8192
    sizes = [10000, cap + 1, 300]
    g = torch.Generator().manual_seed(19)
    x = torch.rand(sum(sizes), 3, generator=g)
    ptr = _ptr(sizes)
    ratio = torch.tensor([0.001, 4.0 / (cap + 1) - 1e-9, 0.01])
    got = fps(x.to(DEV), ptr=ptr.to(DEV), ratio=ratio.to(DEV), random_start=False).cpu().numpy()
    out_ptr = torch.cat([torch.zeros(1, dtype=torch.long),
                         ((ptr[1:] - ptr[:-1]).float() * ratio).ceil().long().cumsum(0)])
    assert np.array_equal(got, orc.fps(x.numpy(), ptr.numpy(), out_ptr.numpy()))
    same = fps(x.to(DEV), ptr=ptr.tolist(), ratio=ratio.to(DEV), random_start=False).cpu().numpy()
    assert np.array_equal(same, got)

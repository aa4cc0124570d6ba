"""Benchmark of the neighbour-graph path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference|reference-cuda] [--no-extra]
    python bench.py --only NAME [--steps K]     (one workload through the C ABI, for profilers)

Headline workload (``knn_graph_batched``): 32 clouds x 4096 points, 3-D fp32 ~ N(0,1), sorted
batch vector, k = 20, loop = False — synthetic, seeded.  One step = one ``knn_graph`` call over
the whole batch.  Printed: ONE JSON line with
  value       queries/s with inputs resident in HBM (CUDA events, L2 flushed between steps)
  e2e         the same result from pinned host buffers to a pinned host buffer
              (``knn_graph_host``): upload of x, search and download of edge_index inside the
              timed region, overlapped across 8 groups of clouds, one stream each
  roofline    of the dominant kernel (knn_spatial_kernel, FP32-pipe bound): 8 flop per
              (query, point) pair / its own duration, CUDA events recorded around that kernel on its
              stream (b200c_profile_knn_scan); beside the nominal FP32 peak the rate a pure-FFMA
              kernel reaches in the same run
  cpu_baseline  the reference's own CPU path (oracle/_ref: kd-tree search, single thread)
  extra       the other configurations (single cloud, large bipartite kNN, 64-D feature kNN with and
              without cosine, radius_graph with and without truncation, its passes in GB/s)
  strong      (N > 1) fixed total work sharded over the ranks, checked against the single-GPU result

``--impl reference`` times the reference's CPU implementation on the same workload instead;
``--impl reference-cuda`` the reference's own CUDA kernels (oracle/_ref, compiled for sm_100a)
beside this library's on the same device tensors.
With N > 1 (torchrun) every rank runs the headline workload on its own clouds (weak scaling, no
data-path collective); the time is the max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FP32_LANES_PER_SM = 128
# ncu, one launch of knn_spatial_kernel on the headline workload (profiles/): dram__bytes_read.sum +
# dram__bytes_write.sum; the sorted copy is read once, most of the output still sits in L2 at the end
KNN_SCAN_DRAM_BYTES = 6353920 + 443648
L2_FLUSH_BYTES = 256 << 20
WORKLOAD = "knn_graph_batched: 32 clouds x 4096 points, 3-D fp32 N(0,1), k=20, loop=False"
# identical in both arms; the L2 remark concerns the GPU arm, the reference arm works from host memory
CONFIG = {"workload": WORKLOAD, "per_gpu": True, "l2": "GPU arm: 256 MiB buffer rewritten between timed steps"}


# ---- workloads -----------------------------------------------------------------------------------

def make_knn_graph_batched(seed=2, clouds=32, points=4096):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(clouds * points, 3, generator=g)
    batch = torch.arange(clouds).repeat_interleave(points)
    return dict(x=x, batch=batch, k=20, clouds=clouds, points=points, queries=clouds * points,
                pairs=clouds * points * points)


def make_knn_bipartite(seed=3, clouds=8, nx=131072, ny=8192):
    g = torch.Generator().manual_seed(seed)
    x = 100 * torch.rand(clouds * nx, 3, generator=g)
    y = 100 * torch.rand(clouds * ny, 3, generator=g)
    return dict(x=x, y=y, batch_x=torch.arange(clouds).repeat_interleave(nx),
                batch_y=torch.arange(clouds).repeat_interleave(ny), k=32, queries=clouds * ny,
                pairs=clouds * nx * ny)


def make_radius_mixture(seed=5, clouds=64, points=8192):
    g = torch.Generator().manual_seed(seed)
    n = clouds * points
    centres = torch.rand(clouds, 32, 3, generator=g)
    pick = torch.randint(0, 32, (clouds, points), generator=g)
    x = torch.gather(centres, 1, pick.unsqueeze(-1).expand(-1, -1, 3)) + 0.02 * torch.randn(clouds, points, 3, generator=g)
    bg = torch.rand(clouds, points, generator=g) < 0.2
    x[bg] = torch.rand(int(bg.sum()), 3, generator=g)
    one_below = float(torch.nextafter(torch.tensor(1.0), torch.tensor(0.0)))
    x = x.clamp_(0, one_below).reshape(n, 3).contiguous()
    return dict(x=x, batch=torch.arange(clouds).repeat_interleave(points), r=0.05, queries=n,
                pairs=clouds * points * points)


# ---- helpers ---------------------------------------------------------------------------------------

class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                 parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def timed_steps(fn, steps, warmup, flush):
    """CUDA-event time of `steps` calls of fn(), L2 flushed (outside the timed span) before each."""
    for _ in range(warmup):
        flush.fill_(1)
        fn()
    torch.cuda.synchronize()
    total_ms = 0.0
    for _ in range(steps):
        flush.fill_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        total_ms += a.elapsed_time(b)
    return total_ms


def max_over_ranks(ms, world):
    if world == 1:
        return ms
    import torch.distributed as dist

    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def load_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f)
    except OSError:
        return {}


def fp32_peak_tf(props, peaks):
    sm_max = peaks.get("sm_max_mhz") or 1965.0
    return props.multi_processor_count * FP32_LANES_PER_SM * 2 * sm_max * 1e6 / 1e12


def scan_kernel_ms(cabi, fn, reps=5):
    """Average duration of the kNN scan kernel alone inside `fn` (CUDA events around that kernel)."""
    from pytorch_cluster_b200 import _native

    lib = _native.cabi()
    lib.b200c_profile_knn_scan(1)
    total = 0.0
    try:
        fn()
        for _ in range(reps):
            fn()
            total += lib.b200c_profile_knn_scan_ms()
    finally:
        lib.b200c_profile_knn_scan(0)
    return total / reps


def measured_fp32_tf(dev):
    """TFLOP/s of a kernel of independent FFMA chains over the whole device (about a millisecond)."""
    import ctypes

    from pytorch_cluster_b200 import _native

    lib = _native.cabi()
    scratch = torch.zeros(1, device=dev)
    flops = ctypes.c_double(0.0)
    stream = torch.cuda.current_stream().cuda_stream
    iters = 40000
    _native.check(lib.b200c_probe_fp32(iters, scratch.data_ptr(), ctypes.byref(flops), stream))
    best = 0.0
    for _ in range(3):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        _native.check(lib.b200c_probe_fp32(iters, scratch.data_ptr(), ctypes.byref(flops), stream))
        b.record()
        b.synchronize()
        best = max(best, flops.value / (a.elapsed_time(b) * 1e-3) / 1e12)
    return best


def radius_passes(cabi, x, ptr, r, max_nn, ms_of, peaks):
    """The passes of one radius_graph call through the C ABI: the scan that counts (and parks the hits
    or their bits), and the HBM-bound pass that writes the edges, with its bytes per second against the
    measured copy bandwidth.  Algorithmic bytes of the write pass: 16 per edge written, 4 per count and 8
    per offset read, plus what it reads per edge (4-byte parked hits, or the hit bits)."""
    from pytorch_cluster_b200 import _native

    lib = _native.cabi()
    n, dim = x.shape
    nseg = ptr.numel() - 1
    dt = _native.B200C_F32
    stream = torch.cuda.current_stream().cuda_stream
    counts = torch.empty(n, dtype=torch.int32, device=x.device)
    hbm = (peaks.get("hbm_gbs") or 6650.0)
    # the operator's rule for the screened scan: segments of at least 2048 * max_nn points
    screen_bytes = (lib.b200c_radius_screen_workspace_bytes(n, n, dim, max_nn, dt, nseg)
                    if n // nseg >= 2048 * max_nn else 0)
    if screen_bytes > 0 or max_nn <= 256:
        # the screened scan parks the hits (any cap); without it the plain one-pass mode does for small caps
        nbytes = max(screen_bytes, lib.b200c_radius_workspace_bytes(n, n, dim, max_nn, dt))
        ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=x.device)
        count = lambda: _native.check(lib.b200c_radius_count(x.data_ptr(), x.data_ptr(), ptr.data_ptr(), ptr.data_ptr(),
                                                             nseg, n, n, dim, float(r), max_nn, 1, dt, counts.data_ptr(),
                                                             ws.data_ptr(), nbytes, stream))
        count()
        offsets = cabi.exclusive_scan(counts)
        total = int(offsets[-1].item())
        out = torch.empty(2, total, dtype=torch.long, device=x.device)
        fill = lambda: _native.check(lib.b200c_radius_fill(x.data_ptr(), x.data_ptr(), ptr.data_ptr(), ptr.data_ptr(), nseg,
                                                           n, n, dim, float(r), max_nn, 1, dt, counts.data_ptr(),
                                                           offsets.data_ptr(), total, out.data_ptr(), ws.data_ptr(), nbytes,
                                                           stream))
        read_per_edge, kernel = 4, "radius_direct_compact_kernel"
        if screen_bytes > 0 and max_nn > 256:
            kernel += " + radius_screen_kernel for queries beyond the parked rows (none here)"
        extra_read = 0
    else:
        hp = ptr.cpu()
        nbytes = lib.b200c_radius_mask_workspace_bytes(hp.data_ptr(), hp.data_ptr(), nseg, n, n, dim, dt)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
        count = lambda: _native.check(lib.b200c_radius_count_masks(x.data_ptr(), x.data_ptr(), ptr.data_ptr(),
                                                                   ptr.data_ptr(), hp.data_ptr(), hp.data_ptr(), nseg, n, n,
                                                                   dim, float(r), max_nn, 1, dt, counts.data_ptr(),
                                                                   ws.data_ptr(), nbytes, stream))
        count()
        offsets = cabi.exclusive_scan(counts)
        total = int(offsets[-1].item())
        out = torch.empty(2, total, dtype=torch.long, device=x.device)
        fill = lambda: _native.check(lib.b200c_radius_fill_masks(ptr.data_ptr(), ptr.data_ptr(), nseg, n, n, dim, dt,
                                                                 counts.data_ptr(), offsets.data_ptr(), total, out.data_ptr(),
                                                                 ws.data_ptr(), stream))
        read_per_edge, kernel = 0, "radius_mask_fill_kernel"
        extra_read = nbytes
    t_count, t_fill = ms_of(count), ms_of(fill)
    fill_bytes = 16 * total + 12 * n + read_per_edge * total + extra_read
    return {"count_scan_ms": t_count, "write_pass_ms": t_fill, "write_pass_kernel": kernel,
            "write_pass_bytes": fill_bytes, "write_pass_gbs": fill_bytes / (t_fill * 1e-3) / 1e9,
            "write_pass_frac_of_measured_hbm": fill_bytes / (t_fill * 1e-3) / 1e9 / hbm}


def extra_workloads(pc, cabi, dev, flush, peak_tf, world, rank, peaks):
    """The other configurations, a few repetitions each: kernel time through the C ABI and call time
    through the public API, with the rates they imply."""
    reps, warm = 5, 2
    out = {}

    def ms_of(fn):
        return timed_steps(fn, reps, warm, flush) / reps

    # one cloud of 1024 points, k = 16
    g = torch.Generator().manual_seed(1)
    x1 = torch.rand(1024, 3, generator=g).to(dev)
    t = ms_of(lambda: pc.knn_graph(x1, 16))
    out["knn_graph_1024x3_k16"] = {"api_ms": t, "queries_per_s": 1024 / (t * 1e-3)}

    # the headline workload with `batch_size` given: the call then makes one host read (the edge count of the
    # fused tail) instead of two (the batch vector's summary first)
    wb = make_knn_graph_batched()
    xb, bb = wb["x"].to(dev), wb["batch"].to(dev)
    t = ms_of(lambda: pc.knn_graph(xb, wb["k"], bb, batch_size=32))
    out["knn_graph_32x4096x3_k20_batch_size_given"] = {"api_ms": t, "queries_per_s": xb.shape[0] / (t * 1e-3)}
    del xb, bb

    # large bipartite kNN: 8 clouds x (131072 points, 8192 queries), k = 32
    w = make_knn_bipartite()
    x, y = w["x"].to(dev), w["y"].to(dev)
    bx, by = w["batch_x"].to(dev), w["batch_y"].to(dev)
    px, py = torch.ops.torch_cluster.segment_ptr(bx, 8), torch.ops.torch_cluster.segment_ptr(by, 8)
    tk = ms_of(lambda: cabi.knn_padded_nosync(x, y, 32, px, py, max_segment_rows=131072))
    tscan = scan_kernel_ms(cabi, lambda: cabi.knn_padded_nosync(x, y, 32, px, py, max_segment_rows=131072))
    ta = ms_of(lambda: pc.knn(x, y, 32, bx, by))
    out["knn_bipartite_8x131072x8192_k32"] = {
        "kernels_ms": tk, "scan_kernel_ms": tscan, "api_ms": ta, "queries_per_s": w["queries"] / (ta * 1e-3),
        "fp32_frac": 8.0 * w["pairs"] / (tk * 1e-3) / 1e12 / peak_tf,
        "fp32_frac_scan_kernel": 8.0 * w["pairs"] / (tscan * 1e-3) / 1e12 / peak_tf}
    # the same clouds as a fixed-radius search with sparse hits (about 15 per query, cap 32): segments of
    # 131072 >= 2048 * 32 points, so the operator takes the screened scan; beside it the plain scan
    tr = ms_of(lambda: pc.radius(x, y, 3.0, bx, by, max_num_neighbors=32))
    edges = int(pc.radius(x, y, 3.0, bx, by, max_num_neighbors=32).shape[1])
    tplain = ms_of(lambda: cabi.radius(x, y, 3.0, px, py, 32))
    out["radius_bipartite_8x131072x8192_r3_max32"] = {
        "api_ms": tr, "edges": edges, "edges_per_s": edges / (tr * 1e-3),
        "fp32_frac": 8.0 * w["pairs"] / (tr * 1e-3) / 1e12 / peak_tf,
        "plain_scan_call_ms": tplain, "fp32_frac_plain_scan": 8.0 * w["pairs"] / (tplain * 1e-3) / 1e12 / peak_tf}
    del x, y

    # feature-space kNN: 16 clouds x 2048 points x 64 features, k = 20
    g = torch.Generator().manual_seed(4)
    xf = torch.randn(32768, 64, generator=g).to(dev)
    bf = torch.arange(16).repeat_interleave(2048).to(dev)
    pf = torch.ops.torch_cluster.segment_ptr(bf, 16)
    for cosine in (False, True):
        tk = ms_of(lambda: cabi.knn_padded_nosync(xf, xf, 21, pf, pf, cosine))
        ta = ms_of(lambda: pc.knn_graph(xf, 20, bf, cosine=cosine))
        out["knn_graph_16x2048x64_k20_cosine" if cosine else "knn_graph_16x2048x64_k20"] = {
            "kernel_ms": tk, "api_ms": ta, "queries_per_s": 32768 / (ta * 1e-3)}

    # radius_graph on a clustered density: 64 clouds x 8192 points, r = 0.05
    w = make_radius_mixture()
    xr, br = w["x"].to(dev), w["batch"].to(dev)
    pr = torch.ops.torch_cluster.segment_ptr(br, 64)
    for max_nn in (64, 8192):
        e = pc.radius_graph(xr, w["r"], br, max_num_neighbors=max_nn)
        ta = ms_of(lambda: pc.radius_graph(xr, w["r"], br, max_num_neighbors=max_nn))
        rec = {"api_ms": ta, "edges": int(e.shape[1]), "edges_per_s": e.shape[1] / (ta * 1e-3),
               "fp32_frac": 8.0 * w["pairs"] / (ta * 1e-3) / 1e12 / peak_tf}
        rec.update(radius_passes(cabi, xr, pr, w["r"], max_nn, ms_of, peaks))
        out[f"radius_graph_64x8192x3_r0.05_max{max_nn}"] = rec

    # the operators either side of the path: farthest point sampling (25 % of every cloud, first
    # point first), then assignment of every point to its nearest sample
    t = ms_of(lambda: pc.fps(xr, br, ratio=0.25, random_start=False, batch_size=64))
    samples = pc.fps(xr, br, ratio=0.25, random_start=False, batch_size=64)
    out["fps_64x8192x3_ratio0.25"] = {"api_ms": t, "samples": int(samples.numel()),
                                      "samples_per_s": samples.numel() / (t * 1e-3)}
    # one large cloud: 1024 samples of 1 M points, spread over the SMs of the device
    g = torch.Generator().manual_seed(6)
    xl = torch.rand(1 << 20, 3, generator=g).to(dev)
    pl = torch.tensor([0, 1 << 20], device=dev)
    t = ms_of(lambda: pc.fps(xl, ptr=pl, ratio=1024 / (1 << 20) - 1e-9, random_start=False))
    out["fps_1x1048576x3_1024_samples"] = {"api_ms": t, "us_per_step": t * 1e3 / 1024}
    del xl
    ys, bs = xr[samples].contiguous(), br[samples].contiguous()
    t = ms_of(lambda: pc.nearest(xr, ys, br, bs))
    out["nearest_64x8192_to_2048x3"] = {"api_ms": t, "rows_per_s": xr.shape[0] / (t * 1e-3),
                                        "fp32_frac": 8.0 * 64 * 8192 * 2048 / (t * 1e-3) / 1e12 / peak_tf}
    return out


def strong_scaling(pc, dev, flush, world, rank):
    """Fixed total work split over the ranks (replicated inputs, segments sharded): the large bipartite
    kNN, radius_graph with both neighbour caps and the bipartite radius search.  Per workload: the
    single-GPU call on this rank (`ms_1gpu`), the sharded call with every rank keeping its own slice
    (`ms_sharded`) and with the global edge_index assembled on every rank (`ms_assembled`); times are
    the max over ranks.  Before timing, the assembled result is checked to equal the single-GPU
    result on every rank."""
    import torch.distributed as dist

    reps, warm = 5, 2
    out = {}

    def ms_of(fn):
        return max_over_ranks(timed_steps(fn, reps, warm, flush) / reps, world)

    def record(name, single, sharded, units, unit_name, gather_bytes):
        want = single()
        got = sharded(True)
        same = torch.tensor([int(torch.equal(want, got))], device=dev)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        assert int(same.item()) == 1, f"{name}: the assembled sharded result differs from the single-GPU result"
        units_n = units(want)
        del got
        t1 = ms_of(single)
        ts = ms_of(lambda: sharded(False))
        ta = ms_of(lambda: sharded(True))
        out[name] = {"ms_1gpu": t1, "ms_sharded": ts, "ms_assembled": ta, "speedup_sharded": t1 / ts,
                     "speedup_assembled": t1 / ta, unit_name + "_per_s_sharded": units_n / (ts * 1e-3),
                     unit_name + "_per_s_assembled": units_n / (ta * 1e-3),
                     "assembly": {"collective": "one all-gather of the padded [2, width] slices (NCCL) + copies into place",
                                  "bytes_received_per_rank": gather_bytes(want) * (world - 1) // world,
                                  "ms": ta - ts}}

    w = make_knn_bipartite()
    x, y = w["x"].to(dev), w["y"].to(dev)
    bx, by = w["batch_x"].to(dev), w["batch_y"].to(dev)
    plan = pc.make_plan(x.size(0), y.size(0), bx, by, 8, world)
    record("knn_bipartite_8x131072x8192_k32", lambda: pc.knn(x, y, 32, bx, by, batch_size=8),
           lambda asm: pc.knn_sharded(x, y, 32, bx, by, batch_size=8, plan=plan, assemble=asm),
           lambda e: w["queries"], "queries", lambda e: e.numel() * 8)
    del x, y

    w = make_radius_mixture()
    xr, br = w["x"].to(dev), w["batch"].to(dev)
    plan = pc.make_plan(xr.size(0), xr.size(0), br, br, 64, world)
    for max_nn in (64, 8192):
        record(f"radius_graph_64x8192x3_r0.05_max{max_nn}",
               lambda: pc.radius_graph(xr, w["r"], br, max_num_neighbors=max_nn, batch_size=64),
               lambda asm: pc.radius_graph_sharded(xr, w["r"], br, max_num_neighbors=max_nn, batch_size=64, plan=plan,
                                                   assemble=asm),
               lambda e: e.shape[1], "edges", lambda e: e.numel() * 8)
    g = torch.Generator().manual_seed(9)
    keep = torch.cat([torch.randperm(8192, generator=g)[:2048].sort().values + 8192 * c for c in range(64)]).to(dev)
    ys, bs = xr[keep].contiguous(), br[keep].contiguous()
    plan = pc.make_plan(xr.size(0), ys.size(0), br, bs, 64, world)
    record("radius_bipartite_64x8192_to_2048_r0.05_max64",
           lambda: pc.radius(xr, ys, w["r"], br, bs, max_num_neighbors=64, batch_size=64),
           lambda asm: pc.radius_sharded(xr, ys, w["r"], br, bs, max_num_neighbors=64, batch_size=64, plan=plan,
                                         assemble=asm),
           lambda e: e.shape[1], "edges", lambda e: e.numel() * 8)
    return out


# ---- reference arm (CPU) ------------------------------------------------------------------------------

def reference_knn_graph_cpu(x, k, batch, clouds):
    """The reference's knn_graph on CPU tensors (torch_cluster/knn.py:131-144) over its compiled
    CPU operator (oracle/_ref)."""
    from oracle import reference_cpu as rc

    ptr = torch.bucketize(torch.arange(clouds + 1), batch)
    e = rc.knn(x, x, ptr, ptr, k + 1, num_workers=os.cpu_count() or 1)
    row, col = e[1], e[0]
    mask = row != col
    return torch.stack([row[mask], col[mask]], dim=0)


def run_reference(args, rank, world):
    if rank != 0:
        return
    from oracle import reference_cpu as rc

    w = make_knn_graph_batched()
    if not rc.available():
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref (reference CPU path) is not built"}))
        return
    # The reference's kd-tree path takes about 13 ms per cloud on one core.  A step is a bounded sample of
    # the workload — the first c of its 32 clouds, the same c every step — with c chosen so that the K
    # timed steps end within about a minute; with K <= 140 every step is the whole workload.
    clouds = max(1, min(w["clouds"], int(60.0 / (max(1, args.steps) * 0.0135))))
    rows = clouds * w["points"]
    xs, bs = w["x"][:rows].contiguous(), w["batch"][:rows].contiguous()
    for _ in range(max(1, min(args.warmup, 2))):
        reference_knn_graph_cpu(xs, w["k"], bs, clouds)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        reference_knn_graph_cpu(xs, w["k"], bs, clouds)
    dt = time.perf_counter() - t0
    steps = args.steps
    value = rows * steps / dt
    line = {
        "impl": "reference", "metric": "knn_graph queries/s", "value": value, "unit": "queries/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup, "ms_per_step": dt / steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": CONFIG,
        "cpu_baseline": {"value": value, "unit": "queries/s", "cores": 1, "kind": "reference",
                         "sample": f"{clouds} of the 32 clouds per step ({rows} queries); the reference's CPU path "
                                   "ignores num_workers (csrc/cpu/knn_cpu.cpp:10), so it runs on one core"},
        "e2e": {"value": value, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---- the reference's CUDA kernels beside this library (same GPU, same tensors) ---------------------------------

def run_reference_cuda(args):
    """Operator-level time (CUDA events, whole operator call incl. its compaction) of the reference's CUDA
    path, compiled unmodified for sm_100a (oracle/_ref), and of this library on the same device tensors at
    the sizes of the benchmark's workloads; results are checked to be identical first.  One JSON line."""
    from oracle import reference_cuda as refc

    if not refc.available():
        print(json.dumps({"impl": "reference-cuda", "unavailable": "oracle/_ref/ref_cluster_cuda.so is not built"}))
        return
    import pytorch_cluster_b200  # noqa: F401

    dev = torch.device("cuda", 0)
    ops = torch.ops.torch_cluster
    rep = {}

    def ms(fn, reps):
        fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    def both(name, ref_fn, our_fn, ref_reps=3):
        assert torch.equal(our_fn(), ref_fn()), name
        rep[name] = {"reference_cuda_ms": round(ms(ref_fn, ref_reps), 4), "this_library_ms": round(ms(our_fn, 5), 4)}
        rep[name]["ratio"] = round(rep[name]["reference_cuda_ms"] / rep[name]["this_library_ms"], 2)

    def ptr(clouds, per):
        return torch.arange(clouds + 1, device=dev) * per

    w = make_knn_graph_batched()
    x, p = w["x"].to(dev), ptr(32, 4096)
    both("knn_32x4096x3_k21", lambda: refc.knn(x, x, p, p, 21), lambda: ops.knn_hinted(x, x, p, p, 21, False, 4096))
    w = make_knn_bipartite()
    xb, yb, pxb, pyb = w["x"].to(dev), w["y"].to(dev), ptr(8, 131072), ptr(8, 8192)
    both("knn_8x131072x8192x3_k32", lambda: refc.knn(xb, yb, pxb, pyb, 32),
         lambda: ops.knn_hinted(xb, yb, pxb, pyb, 32, False, 131072), 1)
    del xb, yb
    xf = torch.randn(32768, 64, generator=torch.Generator().manual_seed(4)).to(dev)
    pf = ptr(16, 2048)
    for cosine in (False, True):
        both(f"knn_16x2048x64_k21_cosine{int(cosine)}", lambda: refc.knn(xf, xf, pf, pf, 21, cosine),
             lambda: ops.knn(xf, xf, pf, pf, 21, cosine, 1))
    xr, pr = make_radius_mixture()["x"].to(dev), ptr(64, 8192)
    both("radius_64x8192x3_r0.05_max64", lambda: refc.radius(xr, xr, pr, pr, 0.05, 64, True),
         lambda: ops.radius(xr, xr, pr, pr, 0.05, 64, 1, True))
    # a cap of 8192 on all 64 clouds would make the reference allocate 2 x 34 GB of padded output: 8 clouds
    xs, ps = xr[: 8 * 8192].contiguous(), ptr(8, 8192)
    both("radius_8x8192x3_r0.05_max8192", lambda: refc.radius(xs, xs, ps, ps, 0.05, 8192, True),
         lambda: ops.radius(xs, xs, ps, ps, 0.05, 8192, 1, True))
    ys, pys = torch.cat([xr[c * 8192: c * 8192 + 2048] for c in range(64)]).contiguous(), ptr(64, 2048)
    both("nearest_64x8192_to_2048x3", lambda: refc.nearest(xr, ys, pr, pys), lambda: ops.nearest(xr, ys, pr, pys))
    ratio = torch.tensor(0.25, device=dev)
    both("fps_64x8192x3_ratio0.25", lambda: refc.fps(xr, pr, ratio, False), lambda: ops.fps(xr, pr, ratio, False), 1)
    xl = torch.rand(1 << 20, 3, generator=torch.Generator().manual_seed(6)).to(dev)
    pl, rl = torch.tensor([0, 1 << 20], device=dev), torch.tensor(1024 / (1 << 20) - 1e-9, device=dev)
    both("fps_1x1048576x3_1024_samples", lambda: refc.fps(xl, pl, rl, False), lambda: ops.fps(xl, pl, rl, False), 1)
    print(json.dumps({"impl": "reference-cuda", "unit": "ms per operator call", "workloads": rep}))


# ---- single workloads for profilers --------------------------------------------------------------------------

def run_only(args):
    """`--only NAME`: K launches of one workload's kernels through the C ABI, nothing else (small
    enough for an ncu capture).  Prints nothing but a completion line."""
    import pytorch_cluster_b200  # noqa: F401  (registers the operators)
    from pytorch_cluster_b200 import cabi

    dev = torch.device("cuda", 0)
    seg = torch.ops.torch_cluster.segment_ptr
    name, steps = args.only, max(1, args.steps)
    if name == "knn_graph_batched":            # the headline kernel: 32 x 4096 x 3, k = 20 (+1)
        w = make_knn_graph_batched()
        x, ptr = w["x"].to(dev), seg(w["batch"].to(dev), 32)
        fn = lambda: cabi.knn_padded_nosync(x, x, 21, ptr, ptr, max_segment_rows=4096)
    elif name == "knn_bipartite_small":        # 2 of the 8 clouds of the large bipartite search
        w = make_knn_bipartite(clouds=2)
        x, y = w["x"].to(dev), w["y"].to(dev)
        px, py = seg(w["batch_x"].to(dev), 2), seg(w["batch_y"].to(dev), 2)
        fn = lambda: cabi.knn_padded_nosync(x, y, 32, px, py, max_segment_rows=131072)
    elif name == "knn_features":               # 16 x 2048 x 64, k = 20 (+1): tensor-core candidates + re-rank
        g = torch.Generator().manual_seed(4)
        x = torch.randn(32768, 64, generator=g).to(dev)
        ptr = torch.arange(0, 32768 + 1, 2048, device=dev)
        fn = lambda: cabi.knn_padded_nosync(x, x, 21, ptr, ptr, args.cosine)
    elif name == "radius_sparse_small":        # 2 clouds of the large bipartite set, about 15 hits per query: screened scan
        w = make_knn_bipartite(clouds=2)
        x, y = w["x"].to(dev), w["y"].to(dev)
        px, py = seg(w["batch_x"].to(dev), 2), seg(w["batch_y"].to(dev), 2)
        fn = lambda: cabi.radius(x, y, 3.0, px, py, 32, False, screen=True)
    elif name in ("radius_mixture_small_screen", "radius_mixture_small_screen_large_cap"):
        w = make_radius_mixture(clouds=16)     # 16 of the 64 clouds, the screened scan
        x, ptr = w["x"].to(dev), seg(w["batch"].to(dev), 16)
        max_nn = 8192 if name.endswith("large_cap") else 64
        fn = lambda: cabi.radius(x, x, w["r"], ptr, ptr, max_nn, True, screen=True)
    elif name in ("radius_mixture_small", "radius_mixture_small_two_scans", "radius_mixture_small_masks"):
        w = make_radius_mixture(clouds=16)     # 16 of the 64 clouds
        x, ptr = w["x"].to(dev), seg(w["batch"].to(dev), 16)
        if name.endswith("masks"):             # large cap: count scan + bit matrix, edges from the bits
            fn = lambda: cabi.radius_masks(x, x, w["r"], ptr, ptr, 8192, True)
        else:
            max_nn = 8192 if name.endswith("two_scans") else 64
            fn = lambda: cabi.radius(x, x, w["r"], ptr, ptr, max_nn, True)
    elif name == "knn_graph_one_kernel":       # the headline call's kernel in its graph-output mode
        w = make_knn_graph_batched()
        x, ptr = w["x"].to(dev), seg(w["batch"].to(dev), 32)
        fn = lambda: cabi.knn_graph_nosync(x, 20, ptr, True, True, 4096)
    elif name in ("fps_small", "nearest_small"):  # 16 of the 64 clouds; 25 % samples, then assignment
        w = make_radius_mixture(clouds=16)
        x, ptr = w["x"].to(dev), seg(w["batch"].to(dev), 16)
        out_ptr = torch.arange(17, device=dev) * 2048
        samples = cabi.fps(x, ptr, out_ptr)
        if name == "fps_small":
            fn = lambda: cabi.fps(x, ptr, out_ptr)
        else:
            y = x[samples].contiguous()
            fn = lambda: cabi.nearest(x, y, ptr, out_ptr)
    else:
        raise SystemExit(f"unknown workload {name}")
    for _ in range(steps):
        fn()
    torch.cuda.synchronize()
    print(f"done: {name} x {steps}")


# ---- our arm ------------------------------------------------------------------------------------------------

def run_ours(args, rank, world, local_rank):
    import pytorch_cluster_b200 as pc
    from pytorch_cluster_b200 import cabi as _cabi

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)
    peaks = load_peaks()
    props = torch.cuda.get_device_properties(dev)

    # every rank works on its own clouds (different seed), same shapes: weak scaling
    w = make_knn_graph_batched(seed=2 + 1000 * rank)
    x, batch, k = w["x"].to(dev), w["batch"].to(dev), w["k"]
    hx, hb = w["x"].pin_memory(), w["batch"].pin_memory()

    def step_resident():
        return pc.knn_graph(x, k, batch)

    out_pinned = torch.empty(2, w["queries"] * k, dtype=torch.long).pin_memory()

    def step_e2e():
        # host buffers in, host buffer out: uploads, search and downloads of groups of clouds overlap
        pc.knn_graph_host(hx, k, hb, device=dev, out=out_pinned)

    e0 = step_resident()
    edges = e0.shape[1]
    assert edges == w["queries"] * k

    if world > 1:
        import torch.distributed as dist

        dist.barrier()
    torch.cuda.synchronize()
    ptr = torch.ops.torch_cluster.segment_ptr(batch, w["clouds"])
    with ClockSampler(local_rank) as clocks:
        ms = timed_steps(step_resident, args.steps, args.warmup, flush)
        torch.cuda.synchronize()
        ms = max_over_ranks(ms, world)
        if world > 1:
            dist.barrier()
        ms_e2e = max_over_ranks(timed_steps(step_e2e, args.steps, args.warmup, flush), world)
        # the kernels of one call through the C ABI (ordering passes + scan), and the scan kernel alone
        ksteps = min(args.steps, 200)
        graph_call = lambda: _cabi.knn_graph_nosync(x, k, ptr, True, True, w["points"])
        ms_kernels = max_over_ranks(timed_steps(graph_call, ksteps, args.warmup, flush) / ksteps, world)
        ms_scan = max_over_ranks(scan_kernel_ms(_cabi, graph_call, reps=min(ksteps, 50)), world)
        fp32_measured = measured_fp32_tf(dev)
        extra = {} if args.no_extra else extra_workloads(pc, _cabi, dev, flush, fp32_peak_tf(props, load_peaks()),
                                                         world, rank, peaks)
        strong = strong_scaling(pc, dev, flush, world, rank) if (world > 1 and not args.no_extra) else None

    if rank != 0:
        return
    total_queries = w["queries"] * world
    sm_max = peaks.get("sm_max_mhz") or 1965.0
    fp32_peak = fp32_peak_tf(props, peaks)
    flops = 8.0 * w["pairs"]
    achieved = flops / (ms_scan * 1e-3) / 1e12
    line = {
        "metric": "knn_graph queries/s", "value": total_queries * args.steps / (ms * 1e-3), "unit": "queries/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": CONFIG,
        "e2e": {"value": total_queries * args.steps / (ms_e2e * 1e-3), "unit": "queries/s",
                # the points and the per-group segment pointers go up (the batch vector is only read on the
                # host), the edge rows and one flag per group come down
                "h2d_bytes_per_step": hx.numel() * 4 + (w["clouds"] + 8) * 8,
                "d2h_bytes_per_step": 2 * edges * 8 + 8 * 4},
        # per knn_graph call: batch_info, segment_ptr, the layout and sort kernels of the ordering pass and
        # the scan kernel, which writes the final edge rows itself
        "gpu_launches": 5 * args.steps,
        "clocks": clocks.summary(),
        "roofline": {"bound": "fp32", "kernel": "knn_spatial_kernel<3,32,rolled>", "achieved": achieved,
                     "peak": fp32_peak, "unit": "TFLOP/s", "frac": achieved / fp32_peak,
                     "peak_source": f"nominal: {props.multi_processor_count} SMs x 128 lanes x 2 flop x "
                                    f"{sm_max:.0f} MHz (MEASURED_PEAKS.json holds no fp32 figure); frac uses it",
                     "peak_measured_ffma": fp32_measured, "frac_of_measured_ffma": achieved / fp32_measured,
                     "flops_per_launch": flops, "ms_per_launch": ms_scan,
                     "ms_all_kernels_of_the_call": ms_kernels,
                     "frac_all_kernels_of_the_call": flops / (ms_kernels * 1e-3) / 1e12 / fp32_peak,
                     "traffic": KNN_SCAN_DRAM_BYTES},
        "extra": extra,
    }
    if strong is not None:
        line["strong"] = strong
    if not args.no_cpu_baseline:
        from oracle import reference_cpu as rc

        if rc.available():
            base = make_knn_graph_batched()
            t0 = time.perf_counter()
            reference_knn_graph_cpu(base["x"], base["k"], base["batch"], base["clouds"])
            dt = time.perf_counter() - t0
            line["cpu_baseline"] = {"value": base["queries"] / dt, "unit": "queries/s", "cores": 1,
                                    "kind": "reference",
                                    "sample": "one pass over the full workload (reference kd-tree path, which "
                                              "ignores num_workers)"}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-cuda"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true")
    ap.add_argument("--only", default=None, help="run one named workload through the C ABI (for profilers)")
    ap.add_argument("--cosine", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.only:
        run_only(args)
        return
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.impl == "reference-cuda":
        if rank == 0:
            run_reference_cuda(args)
        return
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist

            dist.destroy_process_group()


if __name__ == "__main__":
    main()

"""Generates ``tests/golden/reference_cpu_cases.npz`` by running the REFERENCE.

The reference's own Python entry points (``torch_cluster/knn.py``,
``torch_cluster/radius.py``) are executed by path on CPU tensors; the operators
they call (``torch.ops.torch_cluster.knn`` / ``radius``) are bound for this one
process to the reference's compiled CPU path (``oracle/_ref``, i.e. the
unmodified ``csrc/cpu/knn_cpu.cpp`` / ``radius_cpu.cpp``).  Inputs come from
fixed seeds and are stored next to the outputs, so the fixtures can be used
where the reference checkout does not exist.

Run from the repository root, where the reference checkout is available:
    python tests/golden/make_golden.py [--reference DIR]

What the stored outputs pin: edge *sets* for kNN (ties are broken by kd-tree
visit order on CPU, so order inside a query is not pinned) and for radius
without truncation; for truncated radius only the per-query degree is pinned
by the CPU path (it keeps hits in tree order, ``csrc/cpu/radius_cpu.cpp:99-107``),
so those cases also store the untruncated edge set.
"""
from __future__ import annotations

import argparse
import importlib.util
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_cpu_cases.npz")


def bind_reference_ops():
    from oracle import reference_cpu as rc

    rc.load()
    lib = torch.library.Library("torch_cluster", "DEF")
    lib.define("knn(Tensor x, Tensor y, Tensor? ptr_x, Tensor? ptr_y, int k, bool cosine, "
               "int num_workers) -> Tensor")
    lib.define("radius(Tensor x, Tensor y, Tensor? ptr_x, Tensor? ptr_y, float r, "
               "int max_num_neighbors, int num_workers, bool ignore_same_index) -> Tensor")

    def knn(x, y, ptr_x, ptr_y, k, cosine, num_workers):
        assert not cosine, "the reference has no cosine path on CPU (csrc/knn.cpp:33-34)"
        return torch.ops.ref_cluster.knn_cpu(x, y, ptr_x, ptr_y, k, num_workers)

    def radius(x, y, ptr_x, ptr_y, r, max_num_neighbors, num_workers, ignore_same_index):
        return torch.ops.ref_cluster.radius_cpu(x, y, ptr_x, ptr_y, r, max_num_neighbors,
                                                num_workers, ignore_same_index)

    lib.impl("knn", knn, "CompositeExplicitAutograd")
    lib.impl("radius", radius, "CompositeExplicitAutograd")
    return lib


def load_by_path(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def uneven_batch(g, sizes):
    return torch.cat([torch.full((s,), i, dtype=torch.long) for i, s in enumerate(sizes)])


def main():
    from oracle import build_ref

    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=build_ref.default_reference_dir())
    a = ap.parse_args()
    keep = bind_reference_ops()  # noqa: F841  (keeps the registration alive)
    ref_knn = load_by_path("ref_knn_py", os.path.join(a.reference, "torch_cluster", "knn.py"))
    ref_rad = load_by_path("ref_radius_py", os.path.join(a.reference, "torch_cluster", "radius.py"))

    out = {}
    names = []

    def put(name, kind, tensors, args, result, extra=None):
        names.append(name)
        out[f"{name}/kind"] = np.array(kind)
        for key, t in tensors.items():
            if t is not None:
                out[f"{name}/{key}"] = t.numpy()
        out[f"{name}/args"] = np.array(repr(args))
        out[f"{name}/edge_index"] = result.numpy()
        for key, t in (extra or {}).items():
            out[f"{name}/{key}"] = t.numpy()

    g = torch.Generator().manual_seed(20240611)

    # ---- knn(x, y, k, batch_x, batch_y) -------------------------------------------------
    for name, n, m, d, k, dtype, sizes_x, sizes_y in [
        ("knn_d3_single", 1000, 300, 3, 16, torch.float32, None, None),
        ("knn_d2_single", 700, 700, 2, 7, torch.float32, None, None),
        ("knn_d1_single", 257, 64, 1, 5, torch.float32, None, None),
        ("knn_d3_uneven", None, None, 3, 9, torch.float32, [300, 0, 17, 650, 5], [40, 3, 0, 200, 31]),
        ("knn_d3_f64", 900, 500, 3, 21, torch.float64, None, None),
        ("knn_d8_uneven", None, None, 8, 33, torch.float32, [500, 40, 260], [100, 100, 57]),
        ("knn_d5_k100", 600, 50, 5, 100, torch.float32, None, None),
        ("knn_d16_single", 512, 128, 16, 10, torch.float32, None, None),
        ("knn_d64_batched", None, None, 64, 21, torch.float32, [400, 300], [90, 110]),
        ("knn_d64_f64", 300, 40, 64, 12, torch.float64, None, None),
    ]:
        if sizes_x is not None:
            bx, by = uneven_batch(g, sizes_x), uneven_batch(g, sizes_y)
            n, m = bx.numel(), by.numel()
        else:
            bx = by = None
        x = torch.randn(n, d, generator=g, dtype=dtype)
        y = torch.randn(m, d, generator=g, dtype=dtype)
        bs = None if sizes_x is None else len(sizes_x)
        e = ref_knn.knn(x, y, k, bx, by, batch_size=bs)
        put(name, "knn", dict(x=x, y=y, batch_x=bx, batch_y=by), dict(k=k, batch_size=bs), e)

    # ---- knn_graph ------------------------------------------------------------------------
    for name, sizes, d, k, loop, flow, dtype in [
        ("knn_graph_cfg1_like", [1024], 3, 16, False, "source_to_target", torch.float32),
        ("knn_graph_loop_t2s", [333, 500], 3, 6, True, "target_to_source", torch.float32),
        ("knn_graph_small_segments", [5, 3, 9, 1, 30], 3, 4, False, "source_to_target", torch.float32),
        ("knn_graph_f64", [400, 400], 3, 20, False, "source_to_target", torch.float64),
    ]:
        b = uneven_batch(g, sizes) if len(sizes) > 1 else None
        x = torch.rand(sum(sizes), d, generator=g, dtype=dtype)
        e = ref_knn.knn_graph(x, k, b, loop=loop, flow=flow)
        put(name, "knn_graph", dict(x=x, batch=b), dict(k=k, loop=loop, flow=flow), e)

    # ---- radius / radius_graph ------------------------------------------------------------
    for name, sizes_x, sizes_y, d, r, max_nn, dtype in [
        ("radius_d3_single", [1500], [400], 3, 0.12, 4000, torch.float32),
        ("radius_d3_uneven", [300, 0, 900, 12], [100, 5, 0, 60], 3, 0.2, 4000, torch.float32),
        ("radius_d2_f64", [800], [800], 2, 0.05, 4000, torch.float64),
        ("radius_d8", [600, 600], [64, 64], 8, 0.9, 4000, torch.float32),
        ("radius_d3_truncated", [2000], [500], 3, 0.25, 8, torch.float32),
    ]:
        multi = len(sizes_x) > 1
        bx = uneven_batch(g, sizes_x) if multi else None
        by = uneven_batch(g, sizes_y) if multi else None
        x = torch.rand(sum(sizes_x), d, generator=g, dtype=dtype)
        y = torch.rand(sum(sizes_y), d, generator=g, dtype=dtype)
        bs = len(sizes_x) if multi else None
        e = ref_rad.radius(x, y, r, bx, by, max_num_neighbors=max_nn, batch_size=bs)
        extra = None
        if max_nn < 100:
            extra = dict(untruncated=ref_rad.radius(x, y, r, bx, by, max_num_neighbors=1 << 20,
                                                    batch_size=bs))
        put(name, "radius", dict(x=x, y=y, batch_x=bx, batch_y=by),
            dict(r=r, max_num_neighbors=max_nn, batch_size=bs), e, extra)

    for name, sizes, d, r, max_nn, loop, flow, dtype in [
        ("radius_graph_mixture", [1024, 1024], 3, 0.05, 4000, False, "source_to_target", torch.float32),
        ("radius_graph_loop_t2s", [700], 3, 0.15, 4000, True, "target_to_source", torch.float32),
        ("radius_graph_f64", [500, 20, 500], 3, 0.1, 4000, False, "source_to_target", torch.float64),
        ("radius_graph_truncated", [1500], 3, 0.3, 16, False, "source_to_target", torch.float32),
    ]:
        b = uneven_batch(g, sizes) if len(sizes) > 1 else None
        n = sum(sizes)
        if name == "radius_graph_mixture":
            # clustered density: 8 Gaussian blobs (sigma 0.02) plus 20 % uniform background
            centres = torch.rand(8, 3, generator=g)
            pick = torch.randint(0, 8, (n,), generator=g)
            x = centres[pick] + 0.02 * torch.randn(n, 3, generator=g)
            bg = torch.rand(n, generator=g) < 0.2
            x[bg] = torch.rand(int(bg.sum()), 3, generator=g)
            x = x.clamp_(0, float(np.nextafter(np.float32(1), np.float32(0)))).to(dtype)
        else:
            x = torch.rand(n, d, generator=g, dtype=dtype)
        e = ref_rad.radius_graph(x, r, b, loop=loop, max_num_neighbors=max_nn, flow=flow)
        extra = None
        if max_nn < 100:
            extra = dict(untruncated=ref_rad.radius_graph(x, r, b, loop=loop, max_num_neighbors=1 << 20,
                                                          flow=flow))
        put(name, "radius_graph", dict(x=x, batch=b),
            dict(r=r, max_num_neighbors=max_nn, loop=loop, flow=flow), e, extra)

    out["names"] = np.array(names)
    np.savez_compressed(OUT, **out)
    print(f"wrote {OUT}: {len(names)} cases, {os.path.getsize(OUT) / 1024:.0f} KiB")


if __name__ == "__main__":
    main()

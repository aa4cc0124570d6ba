"""Loader for the reference's own CPU path compiled into ``oracle/_ref`` (test
infrastructure; also the timed CPU baseline).  Built by ``oracle/build_ref.py``.

``knn`` / ``radius`` call ``ref_cluster::knn_cpu`` / ``ref_cluster::radius_cpu``,
i.e. the unmodified ``csrc/cpu/knn_cpu.cpp`` / ``csrc/cpu/radius_cpu.cpp`` of the
reference (kd-tree search through the vendored nanoflann).
"""
from __future__ import annotations

import os

import torch

from . import build_ref as _b

_loaded = False


def available() -> bool:
    return os.path.exists(_b.OUT)


def load() -> None:
    global _loaded
    if not _loaded:
        if not available():
            raise RuntimeError("oracle/_ref is not built; run `python oracle/build_ref.py`")
        torch.ops.load_library(_b.OUT)
        _loaded = True


def knn(x, y, ptr_x, ptr_y, k, num_workers=1):
    load()
    return torch.ops.ref_cluster.knn_cpu(x, y, ptr_x, ptr_y, k, num_workers)


def radius(x, y, ptr_x, ptr_y, r, max_num_neighbors, num_workers=1, ignore_same_index=False):
    load()
    return torch.ops.ref_cluster.radius_cpu(x, y, ptr_x, ptr_y, r, max_num_neighbors,
                                            num_workers, ignore_same_index)


def fps(src, ptr, ratio, random_start=False):
    load()
    return torch.ops.ref_cluster.fps_cpu(src, ptr, ratio, random_start)

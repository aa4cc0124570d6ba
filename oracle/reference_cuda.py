"""Loader for the reference's own CUDA kernels compiled for sm_100a into ``oracle/_ref``
(test infrastructure: a second parity checker on the GPU and the timed "kernel to beat").
Built by ``oracle/build_ref.py``; never loaded by the product.

``knn`` / ``radius`` call ``ref_cluster_cuda::knn_cuda`` / ``ref_cluster_cuda::radius_cuda``, i.e.
the unmodified ``csrc/cuda/knn_cuda.cu`` / ``csrc/cuda/radius_cuda.cu`` of the reference.
"""
from __future__ import annotations

import os

import torch

from . import build_ref as _b

_loaded = False


def available() -> bool:
    return os.path.exists(_b.OUT_CUDA)


def load() -> None:
    global _loaded
    if not _loaded:
        if not available():
            raise RuntimeError("oracle/_ref/ref_cluster_cuda.so is not built; run `python oracle/build_ref.py`")
        torch.ops.load_library(_b.OUT_CUDA)
        _loaded = True


def knn(x, y, ptr_x, ptr_y, k, cosine=False):
    load()
    return torch.ops.ref_cluster_cuda.knn_cuda(x, y, ptr_x, ptr_y, k, cosine)


def radius(x, y, ptr_x, ptr_y, r, max_num_neighbors, ignore_same_index=False):
    load()
    return torch.ops.ref_cluster_cuda.radius_cuda(x, y, ptr_x, ptr_y, r, max_num_neighbors, ignore_same_index)


def nearest(x, y, ptr_x, ptr_y):
    load()
    return torch.ops.ref_cluster_cuda.nearest_cuda(x, y, ptr_x, ptr_y)


def fps(src, ptr, ratio, random_start=False):
    load()
    return torch.ops.ref_cluster_cuda.fps_cuda(src, ptr, ratio, random_start)

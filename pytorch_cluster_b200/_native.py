"""Loads the two in-tree native libraries and fails loudly when they are missing.

``libb200cluster.so`` (C ABI, sm_100a kernels) is loaded through ctypes for direct calls;
``_torch_ops.so`` registers ``torch.ops.torch_cluster.{knn,radius,segment_ptr}``.  There is no
fallback: without the built extension, importing the package raises.
"""
from __future__ import annotations

import ctypes
import os

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_CABI = os.path.join(_PKG, "libb200cluster.so")
LIB_OPS = os.path.join(_PKG, "_torch_ops.so")

B200C_OK = 0
B200C_F32, B200C_F64, B200C_F16, B200C_BF16 = 0, 1, 2, 3

_cabi = None


def _missing(path: str) -> ImportError:
    return ImportError(
        f"{os.path.basename(path)} is not built ({path}). Build the extension first: "
        "`python pytorch_cluster_b200/build.py` (or `__graft_entry__.build()`). "
        "This package has no CPU or eager fallback.")


def load_ops() -> None:
    if not os.path.exists(LIB_CABI):
        raise _missing(LIB_CABI)
    if not os.path.exists(LIB_OPS):
        raise _missing(LIB_OPS)
    torch.ops.load_library(LIB_OPS)


def cabi() -> ctypes.CDLL:
    """The C ABI with argument types declared as in ``include/b200_cluster.h``."""
    global _cabi
    if _cabi is not None:
        return _cabi
    if not os.path.exists(LIB_CABI):
        raise _missing(LIB_CABI)
    lib = ctypes.CDLL(LIB_CABI)
    p, i64, i32, dbl, sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_double, ctypes.c_size_t
    lib.b200c_version.restype = i32
    lib.b200c_last_error.restype = ctypes.c_char_p
    lib.b200c_segment_ptr.argtypes = [p, i64, i64, p, p]
    lib.b200c_batch_info.argtypes = [p, i64, p, p]
    lib.b200c_batch_info.restype = i32
    lib.b200c_batch_check.argtypes = [p, i64, p, p]
    lib.b200c_batch_check.restype = i32
    lib.b200c_segment_mismatch.argtypes = [p, p, i64, p, p]
    lib.b200c_segment_mismatch.restype = i32
    lib.b200c_scan_workspace_bytes.argtypes = [i64]
    lib.b200c_scan_workspace_bytes.restype = sz
    lib.b200c_exclusive_scan.argtypes = [p, i64, p, p, sz, p]
    lib.b200c_exclusive_scan_static.argtypes = [p, i64, p, p]
    lib.b200c_knn_workspace_bytes.argtypes = [i64, i64, i64, i64, i32, i32, i64]
    lib.b200c_knn_workspace_bytes.restype = sz
    lib.b200c_knn.argtypes = [p, p, p, p, i64, i64, i64, i64, i64, i32, i32, p, p, p, i64, p, sz, p]
    lib.b200c_morton_order_workspace_bytes.argtypes = [i64, i64, i64]
    lib.b200c_morton_order_workspace_bytes.restype = sz
    lib.b200c_morton_order_rows.argtypes = [i64, i64]
    lib.b200c_morton_order_rows.restype = i64
    lib.b200c_morton_order.argtypes = [p, p, i64, i64, i64, i64, p, p, p, p, sz, p]
    lib.b200c_morton_order.restype = i32
    lib.b200c_profile_knn_scan.argtypes = [i32]
    lib.b200c_profile_knn_scan.restype = i32
    lib.b200c_profile_knn_scan_ms.argtypes = []
    lib.b200c_profile_knn_scan_ms.restype = ctypes.c_float
    lib.b200c_probe_fp32.argtypes = [i64, p, ctypes.POINTER(ctypes.c_double), p]
    lib.b200c_probe_fp32.restype = i32
    lib.b200c_knn_compact.argtypes = [p, p, p, i64, i64, i64, p, p]
    lib.b200c_knn_graph_tail_count.argtypes = [p, p, i64, i64, i32, p, p]
    lib.b200c_knn_graph_tail_write.argtypes = [p, p, p, i64, i64, i32, i32, i64, p, p]
    lib.b200c_radius_workspace_bytes.argtypes = [i64, i64, i64, i64, i32]
    lib.b200c_radius_workspace_bytes.restype = sz
    lib.b200c_radius_screen_workspace_bytes.argtypes = [i64, i64, i64, i64, i32, i64]
    lib.b200c_radius_screen_workspace_bytes.restype = sz
    lib.b200c_radius_count.argtypes = [p, p, p, p, i64, i64, i64, i64, dbl, i64, i32, i32, p, p, sz, p]
    lib.b200c_radius_fill.argtypes = [p, p, p, p, i64, i64, i64, i64, dbl, i64, i32, i32, p, p, i64, p, p, sz, p]
    lib.b200c_radius_count_part.argtypes = [p, p, p, p, i64, i64, i64, i64, dbl, i64, i32, i64, i32, p, p, sz, p]
    lib.b200c_radius_count_part.restype = i32
    lib.b200c_radius_fill_part.argtypes = [p, p, p, p, i64, i64, i64, i64, dbl, i64, i32, i64, i32, i32, p, p, i64, p, p,
                                           sz, p]
    lib.b200c_radius_fill_part.restype = i32
    lib.b200c_radius_count_masks_part.argtypes = [p, p, p, p, p, p, i64, i64, i64, i64, dbl, i64, i32, i64, i32, p, p,
                                                  sz, p]
    lib.b200c_radius_count_masks_part.restype = i32
    lib.b200c_radius_fill_masks_part.argtypes = [p, p, i64, i64, i64, i64, i32, i32, p, p, i64, p, p, p]
    lib.b200c_radius_fill_masks_part.restype = i32
    lib.b200c_knn_graph_workspace_bytes.argtypes = [i64, i64, i64, i32, i64]
    lib.b200c_knn_graph_workspace_bytes.restype = sz
    lib.b200c_knn_graph.argtypes = [p, p, i64, i64, i64, i64, i32, i32, p, p, i64, p, sz, p]
    lib.b200c_knn_graph.restype = i32
    lib.b200c_knn_graph_part.argtypes = [p, p, i64, i64, i64, i64, i32, i32, i64, p, i64, p, i64, p, sz, p]
    lib.b200c_knn_graph_part.restype = i32
    lib.b200c_knn_graph_cosine_workspace_bytes.argtypes = [i64, i64, i64, i64]
    lib.b200c_knn_graph_cosine_workspace_bytes.restype = sz
    lib.b200c_knn_graph_cosine.argtypes = [p, p, i64, i64, i64, i64, i32, p, p, p, sz, p]
    lib.b200c_knn_graph_cosine.restype = i32
    lib.b200c_radius_mask_workspace_bytes.argtypes = [p, p, i64, i64, i64, i64, i32]
    lib.b200c_radius_mask_workspace_bytes.restype = sz
    lib.b200c_radius_count_masks.argtypes = [p, p, p, p, p, p, i64, i64, i64, i64, dbl, i64, i32, i32, p, p, sz, p]
    lib.b200c_radius_count_masks.restype = i32
    lib.b200c_radius_fill_masks.argtypes = [p, p, i64, i64, i64, i64, i32, p, p, i64, p, p, p]
    lib.b200c_radius_fill_masks.restype = i32
    lib.b200c_nearest_workspace_bytes.argtypes = [i64, i64, i64, i32]
    lib.b200c_nearest_workspace_bytes.restype = sz
    lib.b200c_nearest.argtypes = [p, p, p, p, i64, i64, i64, i64, i32, p, p, sz, p]
    lib.b200c_nearest.restype = i32
    lib.b200c_fps_workspace_bytes.argtypes = [i64, i64, i32]
    lib.b200c_fps_workspace_bytes.restype = sz
    lib.b200c_fps.argtypes = [p, p, p, p, i64, i64, i64, i32, p, p, sz, p]
    lib.b200c_fps.restype = i32
    lib.b200c_fps_up_to.argtypes = [p, p, p, p, i64, i64, i64, i32, i64, p, p, sz, p]
    lib.b200c_fps_up_to.restype = i32
    lib.b200c_fps_large_segment_max_points.argtypes = [i64, i32]
    lib.b200c_fps_large_segment_max_points.restype = i64
    lib.b200c_fps_large_segment_workspace_bytes.argtypes = []
    lib.b200c_fps_large_segment_workspace_bytes.restype = sz
    lib.b200c_fps_large_segment.argtypes = [p, i64, i64, i64, i64, i64, i32, p, p, sz, p, p]
    lib.b200c_fps_large_segment.restype = i32
    for name in ("b200c_segment_ptr", "b200c_exclusive_scan", "b200c_exclusive_scan_static", "b200c_knn", "b200c_knn_compact", "b200c_knn_graph_tail_count", "b200c_knn_graph_tail_write",
                 "b200c_radius_count", "b200c_radius_fill"):
        getattr(lib, name).restype = i32
    _cabi = lib
    return lib


def check(status: int) -> None:
    if status != B200C_OK:
        raise RuntimeError(f"b200_cluster status {status}: {cabi().b200c_last_error().decode()}")

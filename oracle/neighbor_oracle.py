"""numpy/ctypes front end of ``neighbor_oracle.c`` (test infrastructure only).

All functions take and return numpy arrays and mirror the reference's operator
results: ``knn`` / ``radius`` return an ``int64 [2, E]`` array whose row 0 is the
query (y) index and row 1 the point (x) index, ordered as the reference's CUDA
operators order them (csrc/cuda/knn_cuda.cu:80-83,133-134;
csrc/cuda/radius_cuda.cu:34-36,94-95).
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

from . import build as _build

_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = _build.OUT if os.path.exists(_build.OUT) and not os.path.exists(_build.SRC) else _build.build()
        _lib = ctypes.CDLL(path)
        i64, p, dbl, i32 = ctypes.c_int64, ctypes.c_void_p, ctypes.c_double, ctypes.c_int
        _lib.oracle_segment_ptr.argtypes = [p, i64, i64, p]
        _lib.oracle_segment_ptr.restype = None
        for sfx in ("f32", "f64"):
            f = getattr(_lib, f"oracle_knn_{sfx}")
            f.argtypes = [p, p, p, p, i64, i64, i64, i64, i64, i32, i32, p, p]
            f.restype = i64
            f = getattr(_lib, f"oracle_radius_{sfx}")
            f.argtypes = [p, p, p, p, i64, i64, i64, i64, dbl, i64, i32, i32, p, p, p]
            f.restype = i64
        for sfx in ("f32", "f64"):
            f = getattr(_lib, f"oracle_nearest_{sfx}")
            f.argtypes = [p, p, p, p, i64, i64, i64, i32, p]
            f.restype = None
            f = getattr(_lib, f"oracle_fps_{sfx}")
            f.argtypes = [p, p, p, p, i64, i64, i32, p, p]
            f.restype = None
        _lib.oracle_knn_r16.argtypes = [p, p, p, p, i64, i64, i64, i64, i64, i32, i32, p, p]
        _lib.oracle_knn_r16.restype = i64
        _lib.oracle_radius_r16.argtypes = [p, p, p, p, i64, i64, i64, i64, dbl, i64, i32, i32, p, p, p]
        _lib.oracle_radius_r16.restype = i64
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def segment_ptr(batch: np.ndarray, num_segments: int) -> np.ndarray:
    """``torch.bucketize(arange(B+1), batch)`` (torch_cluster/knn.py:77-79)."""
    batch = np.ascontiguousarray(batch, dtype=np.int64)
    out = np.empty(num_segments + 1, dtype=np.int64)
    lib().oracle_segment_ptr(_ptr(batch), batch.size, num_segments, _ptr(out))
    return out


def _prep(x, y, ptr_x, ptr_y):
    x = np.ascontiguousarray(x)
    y = np.ascontiguousarray(y, dtype=x.dtype)
    assert x.dtype in (np.float32, np.float64) and x.ndim == 2 and y.ndim == 2
    assert x.shape[1] == y.shape[1]
    if ptr_x is None:
        ptr_x = np.array([0, x.shape[0]], dtype=np.int64)
    if ptr_y is None:
        ptr_y = np.array([0, y.shape[0]], dtype=np.int64)
    ptr_x = np.ascontiguousarray(ptr_x, dtype=np.int64)
    ptr_y = np.ascontiguousarray(ptr_y, dtype=np.int64)
    assert ptr_x.size == ptr_y.size
    sfx = "f32" if x.dtype == np.float32 else "f64"
    return x, y, ptr_x, ptr_y, sfx


_KIND16 = {"f16": 1, "bf16": 2}


def _fn(name, sfx, x, fused, round16):
    """-> (C function, value of its policy argument).  ``round16`` ("f16" / "bf16") selects the
    restatement for 16-bit inputs; x, y are then float32 arrays of 16-bit-representable values."""
    if round16 is None:
        return getattr(lib(), f"oracle_{name}_{sfx}"), int(fused)
    assert x.dtype == np.float32
    return getattr(lib(), f"oracle_{name}_r16"), _KIND16[round16]


def knn_padded(x, y, k, ptr_x=None, ptr_y=None, cosine=False, fused=True, round16=None):
    """Per-query best lists: ``(col [M,k] int64 with -1 padding, dist [M,k])``."""
    x, y, ptr_x, ptr_y, sfx = _prep(x, y, ptr_x, ptr_y)
    m = y.shape[0]
    col = np.empty((m, k), dtype=np.int64)
    dist = np.empty((m, k), dtype=x.dtype)
    f, policy = _fn("knn", sfx, x, fused, round16)
    f(_ptr(x), _ptr(y), _ptr(ptr_x), _ptr(ptr_y), ptr_x.size - 1, x.shape[0], m,
      x.shape[1], k, int(cosine), policy, _ptr(col), _ptr(dist))
    return col, dist


def knn(x, y, k, ptr_x=None, ptr_y=None, cosine=False, fused=True, round16=None) -> np.ndarray:
    col, _ = knn_padded(x, y, k, ptr_x, ptr_y, cosine, fused, round16)
    row = np.repeat(np.arange(col.shape[0], dtype=np.int64), k).reshape(col.shape)
    mask = col != -1
    return np.stack([row[mask], col[mask]])


def radius(x, y, r, ptr_x=None, ptr_y=None, max_num_neighbors=32,
           ignore_same_index=False, fused=True, round16=None) -> np.ndarray:
    x, y, ptr_x, ptr_y, sfx = _prep(x, y, ptr_x, ptr_y)
    m = y.shape[0]
    f, policy = _fn("radius", sfx, x, fused, round16)
    counts = np.empty(m, dtype=np.int64)
    args = (_ptr(x), _ptr(y), _ptr(ptr_x), _ptr(ptr_y), ptr_x.size - 1, x.shape[0], m,
            x.shape[1], float(r), int(max_num_neighbors), int(ignore_same_index), policy)
    total = f(*args, _ptr(counts), None, None)
    offsets = np.zeros(m + 1, dtype=np.int64)
    np.cumsum(counts, out=offsets[1:])
    col = np.empty(total, dtype=np.int64)
    f(*args, None, _ptr(offsets), _ptr(col))
    row = np.repeat(np.arange(m, dtype=np.int64), counts)
    return np.stack([row, col])


def nearest(x, y, ptr_x=None, ptr_y=None, round16=None) -> np.ndarray:
    """out[i] = nearest row of y for row i of x (csrc/cuda/nearest_cuda.cu)."""
    x, y, ptr_x, ptr_y, sfx = _prep(x, y, ptr_x, ptr_y)
    out = np.empty(x.shape[0], dtype=np.int64)
    policy = 0 if round16 is None else _KIND16[round16]
    assert policy == 0 or x.dtype == np.float32
    getattr(lib(), f"oracle_nearest_{sfx}")(_ptr(x), _ptr(y), _ptr(ptr_x), _ptr(ptr_y), ptr_x.size - 1,
                                            x.shape[0], x.shape[1], policy, _ptr(out))
    return out


def fps(src, ptr, out_ptr, start=None, round16=None) -> np.ndarray:
    """Sample indices for given per-segment output boundaries (csrc/cuda/fps_cuda.cu:9-68)."""
    src = np.ascontiguousarray(src)
    assert src.dtype in (np.float32, np.float64) and src.ndim == 2
    ptr = np.ascontiguousarray(ptr, dtype=np.int64)
    out_ptr = np.ascontiguousarray(out_ptr, dtype=np.int64)
    start = None if start is None else np.ascontiguousarray(start, dtype=np.int64)
    out = np.zeros(int(out_ptr[-1]), dtype=np.int64)
    dist = np.empty(src.shape[0], dtype=src.dtype)
    policy = 0 if round16 is None else _KIND16[round16]
    assert policy == 0 or src.dtype == np.float32
    sfx = "f32" if src.dtype == np.float32 else "f64"
    getattr(lib(), f"oracle_fps_{sfx}")(_ptr(src), _ptr(ptr), _ptr(out_ptr), _ptr(start), ptr.size - 1,
                                        src.shape[1], policy, _ptr(dist), _ptr(out))
    return out


# ---- the Python-level functions of the reference, restated over the oracle ----

def _ptrs_from_batch(n, m, batch_x, batch_y, batch_size):
    """torch_cluster/knn.py:62-79: B from the batch maxima unless given; pointers
    only when B > 1."""
    if batch_size is None:
        batch_size = 1
        if batch_x is not None:
            assert n == batch_x.size
            batch_size = int(batch_x.max()) + 1
        if batch_y is not None:
            assert m == batch_y.size
            batch_size = max(batch_size, int(batch_y.max()) + 1)
    assert batch_size > 0
    if batch_size > 1:
        assert batch_x is not None and batch_y is not None
        return segment_ptr(batch_x, batch_size), segment_ptr(batch_y, batch_size)
    return None, None


def knn_api(x, y, k, batch_x=None, batch_y=None, cosine=False, batch_size=None, fused=True):
    """torch_cluster/knn.py:6-82."""
    x, y = np.asarray(x), np.asarray(y)
    if x.size == 0 or y.size == 0:
        return np.empty((2, 0), dtype=np.int64)
    x = x.reshape(-1, 1) if x.ndim == 1 else x
    y = y.reshape(-1, 1) if y.ndim == 1 else y
    px, py = _ptrs_from_batch(x.shape[0], y.shape[0], batch_x, batch_y, batch_size)
    return knn(x, y, k, px, py, cosine, fused)


def knn_graph_api(x, k, batch=None, loop=False, flow="source_to_target", cosine=False,
                  batch_size=None, fused=True):
    """torch_cluster/knn.py:85-144 (k+1 search, flow swap, row != col mask)."""
    assert flow in ("source_to_target", "target_to_source")
    e = knn_api(x, x, k if loop else k + 1, batch, batch, cosine, batch_size, fused)
    row, col = (e[1], e[0]) if flow == "source_to_target" else (e[0], e[1])
    if not loop:
        mask = row != col
        row, col = row[mask], col[mask]
    return np.stack([row, col])


def radius_api(x, y, r, batch_x=None, batch_y=None, max_num_neighbors=32, batch_size=None,
               ignore_same_index=False, fused=True):
    """torch_cluster/radius.py:6-88."""
    x, y = np.asarray(x), np.asarray(y)
    if x.size == 0 or y.size == 0:
        return np.empty((2, 0), dtype=np.int64)
    x = x.reshape(-1, 1) if x.ndim == 1 else x
    y = y.reshape(-1, 1) if y.ndim == 1 else y
    px, py = _ptrs_from_batch(x.shape[0], y.shape[0], batch_x, batch_y, batch_size)
    return radius(x, y, r, px, py, max_num_neighbors, ignore_same_index, fused)


def radius_graph_api(x, r, batch=None, loop=False, max_num_neighbors=32,
                     flow="source_to_target", batch_size=None, fused=True):
    """torch_cluster/radius.py:91-148."""
    assert flow in ("source_to_target", "target_to_source")
    e = radius_api(x, x, r, batch, batch, max_num_neighbors, batch_size, not loop, fused)
    row, col = (e[1], e[0]) if flow == "source_to_target" else (e[0], e[1])
    return np.stack([row, col])

"""Direct calls of the C ABI (include/b200_cluster.h) through ctypes on torch CUDA tensors:
the same entry points the torch operator layer uses, without the operator layer.  Used by the
GPU parity tests and the benchmark's kernel timing."""
from __future__ import annotations

import torch

from . import _native


def _p(t):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _dtype(x):
    return {torch.float32: _native.B200C_F32, torch.float64: _native.B200C_F64,
            torch.float16: _native.B200C_F16, torch.bfloat16: _native.B200C_BF16}[x.dtype]


def segment_ptr(batch, num_segments):
    lib = _native.cabi()
    ptr = torch.empty(num_segments + 1, dtype=torch.long, device=batch.device)
    _native.check(lib.b200c_segment_ptr(_p(batch), batch.numel(), num_segments, _p(ptr), _stream()))
    return ptr


def exclusive_scan(counts):
    lib = _native.cabi()
    m = counts.numel()
    offsets = torch.empty(m + 1, dtype=torch.long, device=counts.device)
    nbytes = lib.b200c_scan_workspace_bytes(m)
    ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=counts.device)
    _native.check(lib.b200c_exclusive_scan(_p(counts), m, _p(offsets), _p(ws), nbytes, _stream()))
    return offsets


def knn_padded_nosync(x, y, k, ptr_x=None, ptr_y=None, cosine=False, workspace=True, max_segment_rows=0):
    """-> (edge_padded int64 [2, m*k], counts int32 [m], num_valid int64 [1]); nothing is read back.
    workspace=False withholds the optional workspace, which selects the kernels that need none."""
    lib = _native.cabi()
    n, m, dim = x.shape[0], y.shape[0], x.shape[1]
    nseg = 1 if ptr_x is None else ptr_x.numel() - 1
    padded = torch.empty(2, m * k, dtype=torch.long, device=x.device)
    counts = torch.empty(m, dtype=torch.int32, device=x.device)
    nvalid = torch.empty(1, dtype=torch.long, device=x.device)
    nbytes = lib.b200c_knn_workspace_bytes(n, m, dim, k, _dtype(x), int(cosine), nseg) if (workspace or cosine or x.element_size() == 2) else 0
    ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=x.device)
    _native.check(lib.b200c_knn(_p(x), _p(y), _p(ptr_x), _p(ptr_y), nseg, n, m, dim, k, _dtype(x),
                                int(cosine), _p(padded), _p(counts), _p(nvalid), max_segment_rows, _p(ws), nbytes,
                                _stream()))
    return padded, counts, nvalid


def knn_padded(x, y, k, ptr_x=None, ptr_y=None, cosine=False, workspace=True, max_segment_rows=0):
    """-> (edge_padded int64 [2, m*k], counts int32 [m], num_valid int)"""
    padded, counts, nvalid = knn_padded_nosync(x, y, k, ptr_x, ptr_y, cosine, workspace, max_segment_rows)
    return padded, counts, int(nvalid.item())


def knn(x, y, k, ptr_x=None, ptr_y=None, cosine=False, workspace=True, max_segment_rows=0):
    """Compacted edge_index through b200c_knn (+ scan + compact when needed)."""
    lib = _native.cabi()
    padded, counts, nvalid = knn_padded(x, y, k, ptr_x, ptr_y, cosine, workspace, max_segment_rows)
    m = y.shape[0]
    if nvalid == m * k:
        return padded
    offsets = exclusive_scan(counts)
    out = torch.empty(2, nvalid, dtype=torch.long, device=x.device)
    _native.check(lib.b200c_knn_compact(_p(padded), _p(counts), _p(offsets), m, k, nvalid, _p(out), _stream()))
    return out


def _radius_workspace(x, m, dim, max_num_neighbors, one_pass):
    lib = _native.cabi()
    nbytes = (lib.b200c_radius_workspace_bytes(x.shape[0], m, dim, max_num_neighbors, _dtype(x))
              if (one_pass or x.element_size() == 2) else 0)
    ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=x.device)
    return ws, nbytes


def radius_counts(x, y, r, ptr_x=None, ptr_y=None, max_num_neighbors=32, ignore_same_index=False, workspace=None):
    """Pass 1.  workspace = (tensor, nbytes) from _radius_workspace, or None for the two-scan mode."""
    lib = _native.cabi()
    n, m, dim = x.shape[0], y.shape[0], x.shape[1]
    nseg = 1 if ptr_x is None else ptr_x.numel() - 1
    counts = torch.empty(m, dtype=torch.int32, device=x.device)
    ws, nbytes = workspace if workspace is not None else (None, 0)
    _native.check(lib.b200c_radius_count(_p(x), _p(y), _p(ptr_x), _p(ptr_y), nseg, n, m, dim, float(r),
                                         max_num_neighbors, int(ignore_same_index), _dtype(x), _p(counts),
                                         _p(ws) if nbytes else None, nbytes, _stream()))
    return counts


def radius(x, y, r, ptr_x=None, ptr_y=None, max_num_neighbors=32, ignore_same_index=False, one_pass=True,
           screen=False):
    """count -> scan -> fill.  one_pass: with the workspace of b200c_radius_workspace_bytes; screen: with that
    of b200c_radius_screen_workspace_bytes (an error where the screened scan does not apply)."""
    lib = _native.cabi()
    n, m, dim = x.shape[0], y.shape[0], x.shape[1]
    nseg = 1 if ptr_x is None else ptr_x.numel() - 1
    if screen:
        nbytes = lib.b200c_radius_screen_workspace_bytes(n, m, dim, max_num_neighbors, _dtype(x), nseg)
        if nbytes == 0:
            raise RuntimeError("screened radius scan not applicable")
        ws = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
    else:
        ws, nbytes = _radius_workspace(x, m, dim, max_num_neighbors, one_pass)
    counts = radius_counts(x, y, r, ptr_x, ptr_y, max_num_neighbors, ignore_same_index, (ws, nbytes))
    offsets = exclusive_scan(counts)
    if screen and int(ws[:8].view(torch.long).item()) != 0:
        raise RuntimeError("the radius scan was abandoned (a bounded wait ran out, or segment pointers that overlap)")
    total = int(offsets[-1].item())
    out = torch.empty(2, total, dtype=torch.long, device=x.device)
    _native.check(lib.b200c_radius_fill(_p(x), _p(y), _p(ptr_x), _p(ptr_y), nseg, n, m, dim, float(r),
                                        max_num_neighbors, int(ignore_same_index), _dtype(x), _p(counts),
                                        _p(offsets), total, _p(out), _p(ws) if nbytes else None, nbytes,
                                        _stream()))
    return out


def nearest(x, y, ptr_x=None, ptr_y=None):
    """-> int64 [n]: for each row of x the nearest row of y of the same segment (b200c_nearest)."""
    lib = _native.cabi()
    n, m, dim = x.shape[0], y.shape[0], x.shape[1]
    nseg = 1 if ptr_x is None else ptr_x.numel() - 1
    out = torch.empty(n, dtype=torch.long, device=x.device)
    nbytes = lib.b200c_nearest_workspace_bytes(n, m, dim, _dtype(x))
    ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=x.device)
    _native.check(lib.b200c_nearest(_p(x), _p(y), _p(ptr_x), _p(ptr_y), nseg, n, m, dim, _dtype(x), _p(out),
                                    _p(ws) if nbytes else None, nbytes, _stream()))
    return out


def fps(src, ptr, out_ptr, start=None):
    """-> int64 [out_ptr[-1]]: farthest point samples per segment (b200c_fps)."""
    lib = _native.cabi()
    n, dim = src.shape[0], src.shape[1]
    total = int(out_ptr[-1].item())
    out = torch.empty(total, dtype=torch.long, device=src.device)
    nbytes = lib.b200c_fps_workspace_bytes(n, dim, _dtype(src))
    ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=src.device)
    _native.check(lib.b200c_fps(_p(src), _p(ptr), _p(out_ptr), _p(start), ptr.numel() - 1, n, dim, _dtype(src),
                                _p(out), _p(ws), nbytes, _stream()))
    return out


def knn_graph_nosync(x, k, ptr=None, source_to_target=True, workspace=True, max_segment_rows=0):
    """-> (edge_index int64 [2, n*k], irregular int32 [1]): b200c_knn_graph, nothing read back."""
    lib = _native.cabi()
    n, dim = x.shape
    nseg = 1 if ptr is None else ptr.numel() - 1
    out = torch.empty(2, n * k, dtype=torch.long, device=x.device)
    irregular = torch.empty(1, dtype=torch.int32, device=x.device)
    nbytes = lib.b200c_knn_graph_workspace_bytes(n, dim, k, _dtype(x), nseg) if workspace else 0
    ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=x.device)
    _native.check(lib.b200c_knn_graph(_p(x), _p(ptr), nseg, n, dim, k, _dtype(x), int(source_to_target), _p(out),
                                      _p(irregular), max_segment_rows, _p(ws) if nbytes else None, nbytes, _stream()))
    return out, irregular


def knn_graph(x, k, ptr=None, source_to_target=True, workspace=True, max_segment_rows=0):
    """-> (edge_index int64 [2, n*k], irregular int): b200c_knn_graph; edge_index is final iff irregular == 0."""
    out, irregular = knn_graph_nosync(x, k, ptr, source_to_target, workspace, max_segment_rows)
    return out, int(irregular.item())


def radius_masks(x, y, r, ptr_x=None, ptr_y=None, max_num_neighbors=32, ignore_same_index=False):
    """Radius search through the bit-matrix entry points (b200c_radius_count_masks / _fill_masks)."""
    lib = _native.cabi()
    n, m, dim = x.shape[0], y.shape[0], x.shape[1]
    nseg = 1 if ptr_x is None else ptr_x.numel() - 1
    hx = None if ptr_x is None else ptr_x.cpu()
    hy = None if ptr_y is None else ptr_y.cpu()
    nbytes = lib.b200c_radius_mask_workspace_bytes(_p(hx), _p(hy), nseg, n, m, dim, _dtype(x))
    if nbytes == 0:
        raise RuntimeError("bit-matrix radius search not applicable")
    ws = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
    counts = torch.empty(m, dtype=torch.int32, device=x.device)
    _native.check(lib.b200c_radius_count_masks(_p(x), _p(y), _p(ptr_x), _p(ptr_y), _p(hx), _p(hy), nseg, n, m, dim,
                                               float(r), max_num_neighbors, int(ignore_same_index), _dtype(x),
                                               _p(counts), _p(ws), nbytes, _stream()))
    offsets = exclusive_scan(counts)
    total = int(offsets[-1].item())
    out = torch.empty(2, total, dtype=torch.long, device=x.device)
    _native.check(lib.b200c_radius_fill_masks(_p(ptr_x), _p(ptr_y), nseg, n, m, dim, _dtype(x), _p(counts), _p(offsets),
                                              total, _p(out), _p(ws), _stream()))
    return out


def fps_large_segment(src, seg_lo, seg_points, count, start_offset=0):
    """-> (int64 [count] samples of one segment, status int): b200c_fps_large_segment."""
    lib = _native.cabi()
    out = torch.empty(count, dtype=torch.long, device=src.device)
    nbytes = lib.b200c_fps_large_segment_workspace_bytes()
    ws = torch.empty(nbytes, dtype=torch.uint8, device=src.device)
    status = torch.zeros(1, dtype=torch.int32, device=src.device)
    _native.check(lib.b200c_fps_large_segment(_p(src), seg_lo, seg_points, start_offset, count, src.shape[1],
                                              _dtype(src), _p(out), _p(ws), nbytes, _p(status), _stream()))
    return out, int(status.item())


def morton_order(x, ptr=None, max_segment_rows=0):
    """-> (order int32 [rows], keys int32 [rows] (bit pattern of uint32), first int64 [B + 1]): b200c_morton_order."""
    lib = _native.cabi()
    n, dim = x.shape
    nseg = 1 if ptr is None else ptr.numel() - 1
    rows = lib.b200c_morton_order_rows(n, nseg)
    order = torch.full((rows,), -2, dtype=torch.int32, device=x.device)
    keys = torch.zeros(rows, dtype=torch.int32, device=x.device)
    first = torch.empty(nseg + 1, dtype=torch.long, device=x.device)
    nbytes = lib.b200c_morton_order_workspace_bytes(n, dim, nseg)
    ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=x.device)
    _native.check(lib.b200c_morton_order(_p(x), _p(ptr), nseg, n, dim, max_segment_rows, _p(order), _p(keys), _p(first),
                                         _p(ws), nbytes, _stream()))
    return order, keys, first

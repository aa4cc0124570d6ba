"""Host-buffer entry point: ``knn_graph`` from pinned host memory to pinned host memory.

The reference's functions take device tensors; a caller whose points and result live on the host
pays the copies around them one after the other.  ``knn_graph_host`` cuts the call into groups of
whole batch segments and runs them on two CUDA streams, so that the upload of group i + 1 and the
download of group i - 1 overlap the search of group i (``b200c_knn_graph_part`` writes each group's
edges, with global row numbers, straight into its slice of the device-side result).  The result
equals ``knn_graph(x.cuda(), k, batch.cuda(), loop=False, flow=flow).cpu()`` exactly.

Covers what the one-kernel route covers (fp32 / fp64, up to 8 features, ``loop=False``, no cosine);
anything else, and any input with irregular queries (segments of fewer than k + 1 points, rows
pushed out of their own list by duplicates), takes the ordinary route through ``knn_graph``.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from . import _native
from .knn import knn_graph
from .sharded import balanced_ranges

_DTYPES = {torch.float32: _native.B200C_F32, torch.float64: _native.B200C_F64}


class _Pipeline:
    """Streams and small pinned buffers reused between calls on a device."""

    def __init__(self, device: torch.device):
        self.streams = [torch.cuda.Stream(device), torch.cuda.Stream(device)]
        self.flags_host: Optional[torch.Tensor] = None
        self.ptrs_host: Optional[torch.Tensor] = None


_pipelines: dict = {}


def _segment_ptr_host(batch: Optional[torch.Tensor], rows: int, batch_size: Optional[int]) -> torch.Tensor:
    if batch is None:
        return torch.tensor([0, rows], dtype=torch.long)
    if batch_size is None:
        batch_size = int(batch[-1]) + 1 if rows > 0 else 1
    return torch.bucketize(torch.arange(batch_size + 1, dtype=torch.long), batch)


def knn_graph_host(x: torch.Tensor, k: int, batch: Optional[torch.Tensor] = None, loop: bool = False,
                   flow: str = 'source_to_target', cosine: bool = False, batch_size: Optional[int] = None,
                   device: Optional[torch.device] = None, out: Optional[torch.Tensor] = None,
                   num_groups: int = 4) -> torch.Tensor:
    """``knn_graph`` for host tensors.  x: [N, D] CPU tensor (pinned for overlap), batch: sorted CPU
    int64 [N] or None.  Returns a pinned CPU int64 [2, E] tensor (``out`` is used when it has the
    right shape)."""
    assert flow in ['source_to_target', 'target_to_source']
    assert not x.is_cuda and (batch is None or not batch.is_cuda)
    device = torch.device('cuda', torch.cuda.current_device()) if device is None else torch.device(device)
    x = x.view(-1, 1) if x.dim() == 1 else x
    x = x.contiguous()
    n, dim = x.shape

    def ordinary() -> torch.Tensor:
        e = knn_graph(x.to(device, non_blocking=True), k, None if batch is None else batch.to(device, non_blocking=True),
                      loop, flow, cosine, 1, batch_size)
        res = out if out is not None and out.shape == e.shape else torch.empty(e.shape, dtype=torch.long).pin_memory()
        res.copy_(e, non_blocking=True)
        torch.cuda.current_stream(device).synchronize()
        return res

    if loop or cosine or dim > 8 or x.dtype not in _DTYPES or n == 0 or k + 1 > 100:
        return ordinary()

    ptr = _segment_ptr_host(batch, n, batch_size)
    sizes = (ptr[1:] - ptr[:-1]).tolist()
    groups: List = [g for g in balanced_ranges([s * s for s in sizes], max(1, min(num_groups, len(sizes)))) if g[1] > g[0]]
    pipe = _pipelines.setdefault(device, _Pipeline(device))
    lib = _native.cabi()
    s2t = int(flow == 'source_to_target')
    total = n * k

    res = out if out is not None and tuple(out.shape) == (2, total) and out.is_pinned() else \
        torch.empty(2, total, dtype=torch.long).pin_memory()
    if pipe.flags_host is None or pipe.flags_host.numel() < len(groups):
        pipe.flags_host = torch.empty(max(8, len(groups)), dtype=torch.int32).pin_memory()
    # every group's own pointers (starting at 0), back to back in one pinned buffer
    count = sum(s1 - s0 + 1 for s0, s1 in groups)
    if pipe.ptrs_host is None or pipe.ptrs_host.numel() < count:
        pipe.ptrs_host = torch.empty(max(1024, count), dtype=torch.long).pin_memory()
    off = 0
    for s0, s1 in groups:
        torch.sub(ptr[s0:s1 + 1], ptr[s0], out=pipe.ptrs_host[off:off + s1 - s0 + 1])
        off += s1 - s0 + 1
    with torch.cuda.device(device):
        x_dev = torch.empty(n, dim, dtype=x.dtype, device=device)
        ptr_dev = torch.empty(count, dtype=torch.long, device=device)
        ptr_dev.copy_(pipe.ptrs_host[:count], non_blocking=True)
        edges_dev = torch.empty(2, total, dtype=torch.long, device=device)
        flags_dev = torch.empty(len(groups), dtype=torch.int32, device=device)
        start = torch.cuda.Event()
        start.record()  # the buffers above, and the copy of the pointers, belong to the current stream
        ptr_off = 0
        for gi, (s0, s1) in enumerate(groups):
            stream = pipe.streams[gi & 1]
            r0, r1 = int(ptr[s0]), int(ptr[s1])
            nseg = s1 - s0
            with torch.cuda.stream(stream):
                stream.wait_event(start)
                x_dev[r0:r1].copy_(x[r0:r1], non_blocking=True)
                local = ptr_dev[ptr_off:ptr_off + nseg + 1]
                _native.check(lib.b200c_knn_graph_part(
                    x_dev[r0:].data_ptr(), local.data_ptr(), nseg, r1 - r0, dim, k, _DTYPES[x.dtype], s2t, r0,
                    edges_dev[0, r0 * k:].data_ptr(), total, flags_dev[gi:].data_ptr(), stream.cuda_stream))
                res[0, r0 * k:r1 * k].copy_(edges_dev[0, r0 * k:r1 * k], non_blocking=True)
                res[1, r0 * k:r1 * k].copy_(edges_dev[1, r0 * k:r1 * k], non_blocking=True)
                pipe.flags_host[gi:gi + 1].copy_(flags_dev[gi:gi + 1], non_blocking=True)
            ptr_off += nseg + 1
        for stream in pipe.streams:
            stream.synchronize()
    if int(pipe.flags_host[:len(groups)].sum()) != 0:
        return ordinary()  # some query does not have the regular shape: the general route handles it
    return res

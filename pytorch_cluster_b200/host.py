"""Host-buffer entry point: ``knn_graph`` from pinned host memory to pinned host memory.

The reference's functions take device tensors; a caller whose points and result live on the host
pays the copies around them one after the other.  ``knn_graph_host`` cuts the call into groups of
whole batch segments, one CUDA stream each, so that the uploads and downloads of the other groups
overlap the search of a group, while the block scheduler keeps the SMs filled across the groups'
kernels (``b200c_knn_graph_part`` writes each group's
edges, with global row numbers, straight into its slice of the device-side result).  The result
equals ``knn_graph(x.cuda(), k, batch.cuda(), loop=False, flow=flow).cpu()`` exactly.

Covers what the one-kernel route covers (fp32 / fp64, up to 8 features, ``loop=False``, no cosine);
anything else, and any input with irregular queries (segments of fewer than k + 1 points, rows
pushed out of their own list by duplicates), takes the ordinary route through ``knn_graph``.
"""
from __future__ import annotations

from typing import Optional

import torch

from .knn import knn_graph

_DTYPES = (torch.float32, torch.float64)


def _segment_ptr_host(batch: Optional[torch.Tensor], rows: int, batch_size: Optional[int]) -> torch.Tensor:
    if batch is None:
        return torch.tensor([0, rows], dtype=torch.long)
    if batch_size is None:
        batch_size = int(batch[-1]) + 1 if rows > 0 else 1
    return torch.bucketize(torch.arange(batch_size + 1, dtype=torch.long), batch)


def knn_graph_host(x: torch.Tensor, k: int, batch: Optional[torch.Tensor] = None, loop: bool = False,
                   flow: str = 'source_to_target', cosine: bool = False, batch_size: Optional[int] = None,
                   device: Optional[torch.device] = None, out: Optional[torch.Tensor] = None,
                   num_groups: int = 8) -> torch.Tensor:
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
    res = out if out is not None and tuple(out.shape) == (2, n * k) and out.is_contiguous() else \
        torch.empty(2, n * k, dtype=torch.long).pin_memory()
    irregular = torch.ops.torch_cluster.knn_graph_host(x, ptr, k, flow == 'source_to_target', res, num_groups,
                                                       device.index if device.index is not None else
                                                       torch.cuda.current_device())
    if irregular != 0:
        return ordinary()  # some query does not have the regular shape: the general route handles it
    return res

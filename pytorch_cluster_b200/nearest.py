"""``nearest`` with the reference's signature (torch_cluster/nearest.py:7-12) on top of
``torch.ops.torch_cluster.nearest``.  CUDA tensors only: the reference's CPU branch (a scipy
vector quantiser, torch_cluster/nearest.py:89-124) has no counterpart here."""
from typing import Optional

import torch


def nearest(
    x: torch.Tensor,
    y: torch.Tensor,
    batch_x: Optional[torch.Tensor] = None,
    batch_y: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    r"""Clusters points in :obj:`x` together which are nearest to a given query point in :obj:`y`:
    returns, for every row of x, the index of the closest row of y of the same example.

    Args, checks and errors follow torch_cluster/nearest.py:44-87: both batch vectors must be
    sorted (``ValueError`` otherwise), and every example that has rows in x must have rows in y.
    """
    x = x.view(-1, 1) if x.dim() == 1 else x
    y = y.view(-1, 1) if y.dim() == 1 else y
    assert x.size(1) == y.size(1)
    if not x.is_cuda:
        raise RuntimeError("x must be CUDA tensor")

    if batch_x is not None and bool((batch_x[1:] - batch_x[:-1] < 0).any()):
        raise ValueError("'batch_x' is not sorted")
    if batch_y is not None and bool((batch_y[1:] - batch_y[:-1] < 0).any()):
        raise ValueError("'batch_y' is not sorted")

    if batch_x is not None:
        assert x.size(0) == batch_x.numel()
        ptr_x = torch.ops.torch_cluster.segment_ptr(batch_x, int(batch_x[-1]) + 1 if batch_x.numel() > 0 else 1)
    else:
        ptr_x = torch.tensor([0, x.size(0)], device=x.device)
    if batch_y is not None:
        assert y.size(0) == batch_y.numel()
        ptr_y = torch.ops.torch_cluster.segment_ptr(batch_y, int(batch_y[-1]) + 1 if batch_y.numel() > 0 else 1)
    else:
        ptr_y = torch.tensor([0, y.size(0)], device=y.device)

    # If an instance in `batch_x` is non-empty, it must be non-empty in `batch_y` as well
    nonempty_ptr_x = (ptr_x[1:] - ptr_x[:-1]) > 0
    nonempty_ptr_y = (ptr_y[1:] - ptr_y[:-1]) > 0
    if not torch.equal(nonempty_ptr_x, nonempty_ptr_y):
        raise ValueError("Some batch indices occur in 'batch_x' that do not occur in 'batch_y'")

    return torch.ops.torch_cluster.nearest(x, y, ptr_x, ptr_y)

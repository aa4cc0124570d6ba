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

    # checks, segment pointers and search in one operator (two host reads: the batch vectors' summaries
    # before the search, the emptiness comparison after it)
    return torch.ops.torch_cluster.nearest_batched(x, y, batch_x, batch_y)

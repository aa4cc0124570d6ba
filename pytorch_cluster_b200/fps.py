"""``fps`` with the reference's signature (torch_cluster/fps.py:33-40) on top of
``torch.ops.torch_cluster.fps``; TorchScript-able through the same overload declarations
(torch_cluster/fps.py:9-30)."""
from typing import List, Optional, Union

import torch
from torch import Tensor


@torch.jit._overload  # noqa
def fps(src, batch, ratio, random_start, batch_size, ptr):  # noqa
    # type: (Tensor, Optional[Tensor], Optional[float], bool, Optional[int], Optional[Tensor]) -> Tensor  # noqa
    pass  # pragma: no cover


@torch.jit._overload  # noqa
def fps(src, batch, ratio, random_start, batch_size, ptr):  # noqa
    # type: (Tensor, Optional[Tensor], Optional[Tensor], bool, Optional[int], Optional[Tensor]) -> Tensor  # noqa
    pass  # pragma: no cover


@torch.jit._overload  # noqa
def fps(src, batch, ratio, random_start, batch_size, ptr):  # noqa
    # type: (Tensor, Optional[Tensor], Optional[float], bool, Optional[int], Optional[List[int]]) -> Tensor  # noqa
    pass  # pragma: no cover


@torch.jit._overload  # noqa
def fps(src, batch, ratio, random_start, batch_size, ptr):  # noqa
    # type: (Tensor, Optional[Tensor], Optional[Tensor], bool, Optional[int], Optional[List[int]]) -> Tensor  # noqa
    pass  # pragma: no cover


def fps(  # noqa
    src: torch.Tensor,
    batch: Optional[Tensor] = None,
    ratio: Optional[Union[Tensor, float]] = None,
    random_start: bool = True,
    batch_size: Optional[int] = None,
    ptr: Optional[Union[Tensor, List[int]]] = None,
):
    r"""Farthest point sampling: iteratively samples the point most distant from the points
    sampled so far, ``ceil(ratio * n)`` points per example (default ratio 0.5).  With
    ``random_start=False`` the first point of every example starts.  Returns the sampled row
    indices, example by example."""
    r: Optional[Tensor] = None
    if ratio is None:
        r = torch.tensor(0.5, dtype=src.dtype, device=src.device)
    elif isinstance(ratio, float):
        r = torch.tensor(ratio, dtype=src.dtype, device=src.device)
    else:
        r = ratio
    assert r is not None

    if ptr is not None:
        if isinstance(ptr, list):
            return torch.ops.torch_cluster.fps(src, torch.tensor(ptr, device=src.device), r, random_start)
        else:
            return torch.ops.torch_cluster.fps(src, ptr, r, random_start)

    if batch is not None:
        assert src.size(0) == batch.numel()
        if batch_size is None:
            batch_size = int(batch.max()) + 1
        # batch need not be sorted here (torch_cluster/fps.py:98-103 counts members), so the
        # boundaries come from a count, not from a bisection
        deg = src.new_zeros(batch_size, dtype=torch.long)
        deg.scatter_add_(0, batch, torch.ones_like(batch))
        ptr_vec = deg.new_zeros(batch_size + 1)
        torch.cumsum(deg, 0, out=ptr_vec[1:])
    else:
        ptr_vec = torch.tensor([0, src.size(0)], device=src.device)

    return torch.ops.torch_cluster.fps(src, ptr_vec, r, random_start)

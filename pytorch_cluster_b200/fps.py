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
            # boundaries known on the host (torch_cluster/fps.py:84-86)
            return torch.ops.torch_cluster.fps_ptr_list(src, ptr, r, random_start)
        return torch.ops.torch_cluster.fps(src, ptr, r, random_start)

    if batch is None:
        return torch.ops.torch_cluster.fps_ptr_list(src, [0, src.size(0)], r, random_start)

    assert src.size(0) == batch.numel()
    # A sorted vector (the usual case) gives its boundaries by bisection, one small kernel; the summary that
    # says so is one kernel and one host read.
    seen: List[int] = torch.ops.torch_cluster.batch_check(batch)
    if seen[2] == 0:
        examples = batch_size if batch_size is not None else seen[0]
        return torch.ops.torch_cluster.fps(src, torch.ops.torch_cluster.segment_ptr(batch, examples), r, random_start)
    num_examples = batch_size if batch_size is not None else int(batch.max()) + 1
    # The example ids need not be sorted for this operator (torch_cluster/fps.py:98-103 counts
    # members instead of bisecting), so the boundaries are the running sum of a histogram.
    members = torch.bincount(batch, minlength=num_examples)
    boundaries = torch.nn.functional.pad(members.cumsum(0), [1, 0])
    return torch.ops.torch_cluster.fps(src, boundaries, r, random_start)

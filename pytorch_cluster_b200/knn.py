"""``knn`` / ``knn_graph`` with the reference's signatures (torch_cluster/knn.py:6-15, 85-94),
TorchScript-able, on top of ``torch.ops.torch_cluster.knn``."""
from typing import List, Optional, Tuple

import torch


def _batch_info(rows: int, batch: Optional[torch.Tensor]) -> List[int]:
    # [number of segments, rows of the largest one].  `batch` is sorted (a documented precondition,
    # torch_cluster/knn.py:27), so its largest id is its last entry; one small kernel finds both
    # numbers and they cross to the host together (the reference reads batch.max()).
    if batch is None:
        return [1, rows]
    assert rows == batch.numel()
    return torch.ops.torch_cluster.batch_info(batch)


def _segment_ptrs(x: torch.Tensor, y: torch.Tensor, batch_x: Optional[torch.Tensor],
                  batch_y: Optional[torch.Tensor],
                  batch_size: Optional[int]) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor], int]:
    """Segment boundaries of x and y rows (torch_cluster/knn.py:62-79): B is inferred from the
    batch vectors unless given, and pointers are only built for B > 1.  Third result: an upper bound
    of any segment's row count, 0 when it is not known (B was given)."""
    num_segments = 1
    max_rows = 0
    if batch_size is None:
        info_x = _batch_info(x.size(0), batch_x)
        info_y = _batch_info(y.size(0), batch_y)
        num_segments = max(info_x[0], info_y[0])
        max_rows = max(info_x[1], info_y[1])
    else:
        num_segments = batch_size
    assert num_segments > 0
    ptr_x: Optional[torch.Tensor] = None
    ptr_y: Optional[torch.Tensor] = None
    if num_segments > 1:
        assert batch_x is not None
        assert batch_y is not None
        ptr_x = torch.ops.torch_cluster.segment_ptr(batch_x, num_segments)
        ptr_y = torch.ops.torch_cluster.segment_ptr(batch_y, num_segments)
    return ptr_x, ptr_y, max_rows


def _graph_ptr(x: torch.Tensor, batch: Optional[torch.Tensor],
               batch_size: Optional[int]) -> Tuple[Optional[torch.Tensor], int]:
    """Segment boundaries when x is searched in itself: one pointer vector serves both sides.
    Second result: an upper bound of any segment's row count, 0 when it is not known."""
    num_segments = 1
    max_rows = 0
    if batch_size is None:
        info = _batch_info(x.size(0), batch)
        num_segments = info[0]
        max_rows = info[1]
    else:
        num_segments = batch_size
    assert num_segments > 0
    ptr: Optional[torch.Tensor] = None
    if num_segments > 1:
        assert batch is not None
        ptr = torch.ops.torch_cluster.segment_ptr(batch, num_segments)
    return ptr, max_rows


def knn(
    x: torch.Tensor,
    y: torch.Tensor,
    k: int,
    batch_x: Optional[torch.Tensor] = None,
    batch_y: Optional[torch.Tensor] = None,
    cosine: bool = False,
    num_workers: int = 1,
    batch_size: Optional[int] = None,
) -> torch.Tensor:
    r"""For each row of :obj:`y`, the :obj:`k` nearest rows of :obj:`x` (of the same example).

    Arguments as in the reference: :obj:`batch_x` / :obj:`batch_y` are sorted ``int64`` example ids,
    :obj:`cosine` selects the cosine distance, :obj:`num_workers` has no effect on the GPU,
    :obj:`batch_size` skips the inference of the number of examples.  Returns ``int64 [2, E]``:
    row 0 indexes :obj:`y`, row 1 indexes :obj:`x`; per query ascending by (distance, index).
    Inputs must be CUDA tensors.
    """
    if x.numel() == 0 or y.numel() == 0:
        return torch.empty(2, 0, dtype=torch.long, device=x.device)
    if x.dim() == 1:
        x = x.view(-1, 1)
    if y.dim() == 1:
        y = y.view(-1, 1)
    x = x.contiguous()
    y = y.contiguous()
    ptr_x, ptr_y, max_rows = _segment_ptrs(x, y, batch_x, batch_y, batch_size)
    # the operator torch_cluster::knn with one more argument: the largest segment, when known
    return torch.ops.torch_cluster.knn_hinted(x, y, ptr_x, ptr_y, k, cosine, max_rows)


def knn_graph(
    x: torch.Tensor,
    k: int,
    batch: Optional[torch.Tensor] = None,
    loop: bool = False,
    flow: str = 'source_to_target',
    cosine: bool = False,
    num_workers: int = 1,
    batch_size: Optional[int] = None,
) -> torch.Tensor:
    r"""Edges from every node to its :obj:`k` nearest nodes.

    Same result as the reference's composition (torch_cluster/knn.py:131-144): the k (+1 without
    self loops) nearest rows of x for every row of x, oriented by :obj:`flow`, with the
    ``row == col`` entries dropped when :obj:`loop` is false — computed by one operator.
    """
    assert flow in ['source_to_target', 'target_to_source']
    if x.numel() == 0:
        return torch.empty(2, 0, dtype=torch.long, device=x.device)
    if x.dim() == 1:
        x = x.view(-1, 1)
    x = x.contiguous()
    ptr, max_rows = _graph_ptr(x, batch, batch_size)
    # one operator: search, self-match and padding removal, flow orientation (one host sync)
    return torch.ops.torch_cluster.knn_graph_edges(x, ptr, k, loop, flow == 'source_to_target', cosine, max_rows)

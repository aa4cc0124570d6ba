"""Multi-GPU neighbour search: shard by batch segment, assemble the global ``edge_index``.

Every query row (and every batch segment) is independent of all others
(csrc/cuda/knn_cuda.cu:38-52 of the reference: a thread touches only its own query and that
query's segment of x), so the path shards with no collective on the data path itself:

* one process per GPU (``torch.distributed``, NCCL over NVLink); inputs are either already
  replicated on every rank or live on ``src`` and are broadcast first (``broadcast_inputs``);
* the segments are split into ``world_size`` contiguous ranges balanced by the number of
  (query, point) pairs; because batch vectors are sorted, a range of segments is a contiguous
  range of y rows and of x rows, and its result is a contiguous slice of the query-ordered global
  ``edge_index``; a single segment is split by y rows instead, with x kept whole;
* each rank runs the ordinary single-GPU operator on its slice and shifts the indices back;
* the only exchange: an all-gather of the per-rank edge counts, then an all-gather of the edge
  slices (padded to the largest count) — skipped with ``assemble=False`` when the consumer is
  sharded the same way.

The reference has no multi-GPU support; this layer is new.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def balanced_ranges(weights: Sequence[int], parts: int) -> List[Tuple[int, int]]:
    """Split ``range(len(weights))`` into ``parts`` contiguous ranges whose weight sums are as even
    as a greedy prefix cut gets them.  Ranges may be empty; they always tile the whole range."""
    n = len(weights)
    total = float(sum(weights))
    bounds = [0]
    acc = 0.0
    i = 0
    for p in range(1, parts):
        target = total * p / parts
        while i < n and acc + weights[i] / 2.0 <= target:
            acc += weights[i]
            i += 1
        bounds.append(i)
    bounds.append(n)
    return [(bounds[p], bounds[p + 1]) for p in range(parts)]


def _segment_ptr_host(batch: Optional[torch.Tensor], rows: int, num_segments: int) -> List[int]:
    if batch is None:
        return [0, rows]
    arange = torch.arange(num_segments + 1, device=batch.device)
    return torch.bucketize(arange, batch).tolist()  # small: B + 1 values cross to the host


def plan(x_rows: int, y_rows: int, batch_x: Optional[torch.Tensor], batch_y: Optional[torch.Tensor],
         batch_size: Optional[int], world_size: int):
    """-> list over ranks of (x_lo, x_hi, y_lo, y_hi, seg_lo, seg_hi)."""
    if batch_size is None:
        batch_size = 1
        if batch_x is not None:
            batch_size = int(batch_x[-1]) + 1
        if batch_y is not None:
            batch_size = max(batch_size, int(batch_y[-1]) + 1)
    if batch_size > 1:
        assert batch_x is not None and batch_y is not None
        px = _segment_ptr_host(batch_x, x_rows, batch_size)
        py = _segment_ptr_host(batch_y, y_rows, batch_size)
        weights = [(px[b + 1] - px[b]) * (py[b + 1] - py[b]) for b in range(batch_size)]
        out = []
        for s0, s1 in balanced_ranges(weights, world_size):
            out.append((px[s0], px[s1], py[s0], py[s1], s0, s1))
        return out
    # one segment: split the queries, keep x whole
    out = []
    for r in range(world_size):
        lo, hi = y_rows * r // world_size, y_rows * (r + 1) // world_size
        out.append((0, x_rows, lo, hi, 0, 1))
    return out


def _all_gather_edges(local: torch.Tensor, group, world_size: int) -> torch.Tensor:
    """All-gather of int64 [2, E_r] slices with unequal E_r: counts first, then padded slices."""
    count = torch.tensor([local.shape[1]], dtype=torch.long, device=local.device)
    counts = [torch.zeros_like(count) for _ in range(world_size)]
    dist.all_gather(counts, count, group=group)
    counts = [int(c.item()) for c in counts]
    width = max(counts) if counts else 0
    padded = torch.zeros(2, width, dtype=torch.long, device=local.device)
    padded[:, :local.shape[1]] = local
    gathered = [torch.empty_like(padded) for _ in range(world_size)]
    dist.all_gather(gathered, padded.contiguous(), group=group)
    return torch.cat([g[:, :c] for g, c in zip(gathered, counts)], dim=1)


def _run_sharded(local_fn: Callable, x, y, batch_x, batch_y, batch_size, group, assemble, broadcast_inputs, src):
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if broadcast_inputs:
        for t in (x, y, batch_x, batch_y):
            if t is not None:
                dist.broadcast(t, src=src, group=group)
    x = x.view(-1, 1) if x.dim() == 1 else x
    y = y.view(-1, 1) if y.dim() == 1 else y
    ranges = plan(x.size(0), y.size(0), batch_x, batch_y, batch_size, world)
    x_lo, x_hi, y_lo, y_hi, s0, s1 = ranges[rank]
    if y_hi > y_lo and x_hi > x_lo:
        bx = None if batch_x is None else batch_x[x_lo:x_hi] - s0
        by = None if batch_y is None else batch_y[y_lo:y_hi] - s0
        local = local_fn(x[x_lo:x_hi], y[y_lo:y_hi], bx, by, max(s1 - s0, 1))
        local = local + torch.tensor([[y_lo], [x_lo]], dtype=torch.long, device=local.device)
    else:
        local = torch.empty(2, 0, dtype=torch.long, device=x.device)
    if not assemble:
        return local
    return _all_gather_edges(local, group, world)


def knn_sharded(x: torch.Tensor, y: torch.Tensor, k: int, batch_x: Optional[torch.Tensor] = None,
                batch_y: Optional[torch.Tensor] = None, cosine: bool = False, batch_size: Optional[int] = None,
                group=None, assemble: bool = True, broadcast_inputs: bool = False, src: int = 0,
                compute: Optional[Callable] = None) -> torch.Tensor:
    """``knn`` over all ranks of ``group``.  With ``assemble`` every rank returns the same global
    ``[2, E]`` tensor the single-GPU call returns; without it, its own (globally indexed) slice.
    ``compute`` replaces the single-GPU operator (tests inject a CPU checker to exercise the
    plumbing over gloo)."""
    if compute is None:
        from .knn import knn as compute

    def local_fn(xs, ys, bx, by, nseg):
        return compute(xs, ys, k, bx, by, cosine=cosine, batch_size=nseg if bx is not None else None)

    return _run_sharded(local_fn, x, y, batch_x, batch_y, batch_size, group, assemble, broadcast_inputs, src)


def radius_sharded(x: torch.Tensor, y: torch.Tensor, r: float, batch_x: Optional[torch.Tensor] = None,
                   batch_y: Optional[torch.Tensor] = None, max_num_neighbors: int = 32,
                   batch_size: Optional[int] = None, group=None, assemble: bool = True,
                   broadcast_inputs: bool = False, src: int = 0, compute: Optional[Callable] = None) -> torch.Tensor:
    """``radius`` over all ranks of ``group`` (see ``knn_sharded``).  ``ignore_same_index`` is not
    offered here: slicing changes row numbers, so self pairs are removed by the caller
    (``radius_graph_sharded`` does it on global indices)."""
    if compute is None:
        from .radius import radius as compute

    def local_fn(xs, ys, bx, by, nseg):
        return compute(xs, ys, r, bx, by, max_num_neighbors=max_num_neighbors,
                       batch_size=nseg if bx is not None else None)

    return _run_sharded(local_fn, x, y, batch_x, batch_y, batch_size, group, assemble, broadcast_inputs, src)

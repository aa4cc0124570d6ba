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
* each rank runs the single-GPU operators on its slice (segment pointers cut from the global ones,
  no batch vector is re-scanned) and shifts the indices back;
* the only exchange: one all-gather of the per-rank edge counts (one host read), then one
  all-gather of the edge slices (both rows, padded to the largest slice) and the copies into the
  final ``[2, E]`` tensor — skipped with ``assemble=False`` when the consumer is sharded the same way.

The partition (``ShardPlan``) needs the segment sizes on the host: pass ``plan=make_plan(...)`` to
reuse one across calls on the same batch layout (no host synchronisation per call then), or let
each call build it (one device-to-host read of the segment pointers).

``knn_graph_sharded`` / ``radius_graph_sharded`` are the graph forms: a rank's slice of a batched
cloud set is searched in itself, so ``row != col`` and ``ignore_same_index`` keep their meaning
after the shift; for a single cloud the queries are split and ``radius`` is told the slice's first
row (``query_index_base``) so that the skipped pair is the one with equal *global* row numbers
(csrc/cuda/radius_cuda.cu:33).

The reference has no multi-GPU support; this layer is new.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

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


def plan(x_rows: int, y_rows: int, batch_x: Optional[torch.Tensor], batch_y: Optional[torch.Tensor],
         batch_size: Optional[int], world_size: int):
    """-> list over ranks of (x_lo, x_hi, y_lo, y_hi, seg_lo, seg_hi)."""
    return make_plan(x_rows, y_rows, batch_x, batch_y, batch_size, world_size).ranges


class ShardPlan:
    """The partition of one batch layout over ``world_size`` ranks.

    ``ranges[r] = (x_lo, x_hi, y_lo, y_hi, seg_lo, seg_hi)``; ``ptr_x`` / ``ptr_y`` are the global
    segment pointers as host lists (``None`` for a single segment).  ``local_ptrs(rank, device)``
    gives the rank's own pointers, starting at 0, as device tensors (built once, then cached)."""

    def __init__(self, ranges, ptr_x: Optional[List[int]], ptr_y: Optional[List[int]]):
        self.ranges = ranges
        self.ptr_x = ptr_x
        self.ptr_y = ptr_y
        self._local = {}

    def local_ptrs(self, rank: int, device) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
        if self.ptr_x is None:
            return None, None
        key = (rank, str(device))
        if key not in self._local:
            _, _, _, _, s0, s1 = self.ranges[rank]
            px = [v - self.ptr_x[s0] for v in self.ptr_x[s0:s1 + 1]]
            py = [v - self.ptr_y[s0] for v in self.ptr_y[s0:s1 + 1]]
            self._local[key] = (torch.tensor(px, dtype=torch.long, device=device),
                                torch.tensor(py, dtype=torch.long, device=device))
        return self._local[key]

    def max_rows(self, rank: int) -> int:
        """Rows of the rank's largest segment (x or y side); 0 for a single segment (not known here)."""
        if self.ptr_x is None:
            return 0
        _, _, _, _, s0, s1 = self.ranges[rank]
        sizes = [self.ptr_x[b + 1] - self.ptr_x[b] for b in range(s0, s1)]
        sizes += [self.ptr_y[b + 1] - self.ptr_y[b] for b in range(s0, s1)]
        return max(sizes) if sizes else 0


def _host_ptrs(batch_x, batch_y, batch_size):
    """Segment pointers of both sides as host lists: ONE device-to-host transfer."""
    from_op = batch_x.is_cuda
    if from_op:
        seg = torch.ops.torch_cluster.segment_ptr
        both = torch.cat([seg(batch_x, batch_size), seg(batch_y, batch_size)]).tolist()
    else:
        arange = torch.arange(batch_size + 1)
        both = torch.cat([torch.bucketize(arange, batch_x), torch.bucketize(arange, batch_y)]).tolist()
    return both[:batch_size + 1], both[batch_size + 1:]


def make_plan(x_rows: int, y_rows: int, batch_x: Optional[torch.Tensor], batch_y: Optional[torch.Tensor],
              batch_size: Optional[int], world_size: int, ptr_x: Optional[Sequence[int]] = None,
              ptr_y: Optional[Sequence[int]] = None) -> ShardPlan:
    """Partition for ``world_size`` ranks.  With host pointer lists (``ptr_x``, ``ptr_y``) nothing is
    read from the device; otherwise the batch vectors give them (one transfer, plus one element of
    each vector when ``batch_size`` is not given)."""
    if ptr_x is not None:
        assert ptr_y is not None and len(ptr_x) == len(ptr_y) and len(ptr_x) >= 2
        px, py = [int(v) for v in ptr_x], [int(v) for v in ptr_y]
        batch_size = len(px) - 1
    else:
        if batch_size is None:
            batch_size = 1
            if batch_x is not None:
                batch_size = int(batch_x[-1]) + 1
            if batch_y is not None:
                batch_size = max(batch_size, int(batch_y[-1]) + 1)
        px = py = None
        if batch_size > 1:
            assert batch_x is not None and batch_y is not None
            px, py = _host_ptrs(batch_x, batch_y, batch_size)
    if batch_size > 1:
        weights = [(px[b + 1] - px[b]) * (py[b + 1] - py[b]) for b in range(batch_size)]
        ranges = [(px[s0], px[s1], py[s0], py[s1], s0, s1) for s0, s1 in balanced_ranges(weights, world_size)]
        return ShardPlan(ranges, px, py)
    # one segment: split the queries, keep x whole
    ranges = []
    for r in range(world_size):
        lo, hi = y_rows * r // world_size, y_rows * (r + 1) // world_size
        ranges.append((0, x_rows, lo, hi, 0, 1))
    return ShardPlan(ranges, None, None)


class _DeviceOps:
    """The single-GPU operators a rank runs on its slice."""

    @staticmethod
    def knn(x, y, ptr_x, ptr_y, k, cosine, max_rows=0):
        return torch.ops.torch_cluster.knn_hinted(x, y, ptr_x, ptr_y, k, cosine, max_rows)

    @staticmethod
    def knn_graph(x, ptr, k, loop, source_to_target, cosine, max_rows=0):
        return torch.ops.torch_cluster.knn_graph_edges(x, ptr, k, loop, source_to_target, cosine, max_rows)

    @staticmethod
    def radius(x, y, ptr_x, ptr_y, r, max_num_neighbors, ignore_same_index, query_index_base, swap_rows):
        return torch.ops.torch_cluster.radius_part(x, y, ptr_x, ptr_y, r, max_num_neighbors, ignore_same_index,
                                                   query_index_base, swap_rows)


def _gather_edges(local: torch.Tensor, group, world_size: int) -> torch.Tensor:
    """All-gather of int64 [2, E_r] slices into the global [2, E], rank slices side by side in each
    row.  One all-gather of the counts (one host read), then ONE all-gather of the slices, both rows
    together and padded to the largest count, into a staging tensor [world, 2, width], and the copies
    that put every rank's columns at their place (one strided copy when the counts are equal).  A
    single large collective runs at NVLink rate; per-row or per-rank collectives of unequal sizes
    (which NCCL runs as grouped broadcasts) were measured four times slower."""
    device = local.device
    mine = torch.tensor([local.shape[1]], dtype=torch.long, device=device)
    all_counts = torch.empty(world_size, dtype=torch.long, device=device)
    dist.all_gather_into_tensor(all_counts, mine, group=group)
    counts = all_counts.tolist()  # the one host read of the assembly
    total, width = sum(counts), max(counts)
    out = torch.empty(2, total, dtype=torch.long, device=device)
    if total == 0:
        return out
    if local.shape[1] == width:
        padded = local.contiguous()
    else:
        padded = torch.empty(2, width, dtype=torch.long, device=device)
        padded[:, :local.shape[1]] = local
    staging = torch.empty(world_size, 2, width, dtype=torch.long, device=device)
    dist.all_gather_into_tensor(staging.view(-1), padded.view(-1), group=group)
    if min(counts) == width:
        out.view(2, world_size, width).copy_(staging.permute(1, 0, 2))
        return out
    off = 0
    for r, c in enumerate(counts):
        if c:
            out[:, off:off + c] = staging[r, :, :c]
        off += c
    return out


def _setup(x, y, batch_x, batch_y, batch_size, group, broadcast_inputs, src, plan_):
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if broadcast_inputs:
        seen = []  # x may be passed as y, one batch vector for both sides: broadcast each tensor once
        for t in (x, y, batch_x, batch_y):
            if t is not None and not any(t is s for s in seen):
                dist.broadcast(t, src=src, group=group)
                seen.append(t)
    if plan_ is None:
        plan_ = make_plan(x.size(0), y.size(0), batch_x, batch_y, batch_size, world)
    assert len(plan_.ranges) == world, "the plan was made for another world size"
    return world, rank, plan_


def _shift(local: torch.Tensor, row0: int, row1: int) -> torch.Tensor:
    if row0 == 0 and row1 == 0:
        return local
    local[0] += row0
    local[1] += row1
    return local


def _finish(local, group, world, assemble):
    return _gather_edges(local, group, world) if assemble else local


def _as_2d(t):
    return t.view(-1, 1) if t.dim() == 1 else t


def knn_sharded(x: torch.Tensor, y: torch.Tensor, k: int, batch_x: Optional[torch.Tensor] = None,
                batch_y: Optional[torch.Tensor] = None, cosine: bool = False, batch_size: Optional[int] = None,
                group=None, assemble: bool = True, broadcast_inputs: bool = False, src: int = 0,
                plan: Optional[ShardPlan] = None, ops=None) -> torch.Tensor:
    """``knn`` over all ranks of ``group``.  With ``assemble`` every rank returns the same global
    ``[2, E]`` tensor the single-GPU call returns; without it, its own (globally indexed) slice.
    ``ops`` replaces the single-GPU operators (tests inject a CPU checker to exercise the plumbing
    over gloo)."""
    ops = ops or _DeviceOps
    x, y = _as_2d(x), _as_2d(y)
    world, rank, plan = _setup(x, y, batch_x, batch_y, batch_size, group, broadcast_inputs, src, plan)
    x_lo, x_hi, y_lo, y_hi, _, _ = plan.ranges[rank]
    if y_hi > y_lo and x_hi > x_lo:
        px, py = plan.local_ptrs(rank, x.device)
        local = _shift(ops.knn(x[x_lo:x_hi], y[y_lo:y_hi], px, py, k, cosine, plan.max_rows(rank)), y_lo, x_lo)
    else:
        local = torch.empty(2, 0, dtype=torch.long, device=x.device)
    return _finish(local, group, world, assemble)


def radius_sharded(x: torch.Tensor, y: torch.Tensor, r: float, batch_x: Optional[torch.Tensor] = None,
                   batch_y: Optional[torch.Tensor] = None, max_num_neighbors: int = 32,
                   batch_size: Optional[int] = None, group=None, assemble: bool = True,
                   broadcast_inputs: bool = False, src: int = 0, plan: Optional[ShardPlan] = None,
                   ops=None) -> torch.Tensor:
    """``radius`` over all ranks of ``group`` (see ``knn_sharded``).  For a search of a point set in
    itself without self pairs use ``radius_graph_sharded``."""
    ops = ops or _DeviceOps
    x, y = _as_2d(x), _as_2d(y)
    world, rank, plan = _setup(x, y, batch_x, batch_y, batch_size, group, broadcast_inputs, src, plan)
    x_lo, x_hi, y_lo, y_hi, _, _ = plan.ranges[rank]
    if y_hi > y_lo and x_hi > x_lo:
        px, py = plan.local_ptrs(rank, x.device)
        local = _shift(ops.radius(x[x_lo:x_hi], y[y_lo:y_hi], px, py, r, max_num_neighbors, False, 0, False),
                       y_lo, x_lo)
    else:
        local = torch.empty(2, 0, dtype=torch.long, device=x.device)
    return _finish(local, group, world, assemble)


def knn_graph_sharded(x: torch.Tensor, k: int, batch: Optional[torch.Tensor] = None, loop: bool = False,
                      flow: str = 'source_to_target', cosine: bool = False, batch_size: Optional[int] = None,
                      group=None, assemble: bool = True, broadcast_inputs: bool = False, src: int = 0,
                      plan: Optional[ShardPlan] = None, ops=None) -> torch.Tensor:
    """``knn_graph`` over all ranks of ``group``: the result of the single-GPU call
    (torch_cluster/knn.py:85-144), edges ordered by the node that searched."""
    assert flow in ['source_to_target', 'target_to_source']
    ops = ops or _DeviceOps
    x = _as_2d(x)
    s2t = flow == 'source_to_target'
    world, rank, plan = _setup(x, x, batch, batch, batch_size, group, broadcast_inputs, src, plan)
    x_lo, x_hi, y_lo, y_hi, _, _ = plan.ranges[rank]
    if y_hi <= y_lo or x_hi <= x_lo:
        local = torch.empty(2, 0, dtype=torch.long, device=x.device)
    elif plan.ptr_x is not None:
        # whole clouds: the slice is searched in itself, both rows shift by the slice's first row
        ptr, _ = plan.local_ptrs(rank, x.device)
        local = _shift(ops.knn_graph(x[x_lo:x_hi], ptr, k, loop, s2t, cosine, plan.max_rows(rank)), x_lo, x_lo)
    else:
        # one cloud: this rank's rows search all of x; the self match is the one whose shifted
        # query row equals the neighbour (the `row != col` mask of torch_cluster/knn.py:140-142)
        e = ops.knn(x, x[y_lo:y_hi], None, None, k if loop else k + 1, cosine)
        q, nb = e[0] + y_lo, e[1]
        if not loop:
            keep = q != nb
            q, nb = q[keep], nb[keep]
        local = torch.stack([nb, q] if s2t else [q, nb], dim=0)
    return _finish(local, group, world, assemble)


def radius_graph_sharded(x: torch.Tensor, r: float, batch: Optional[torch.Tensor] = None, loop: bool = False,
                         max_num_neighbors: int = 32, flow: str = 'source_to_target',
                         batch_size: Optional[int] = None, group=None, assemble: bool = True,
                         broadcast_inputs: bool = False, src: int = 0, plan: Optional[ShardPlan] = None,
                         ops=None) -> torch.Tensor:
    """``radius_graph`` over all ranks of ``group``: the result of the single-GPU call
    (torch_cluster/radius.py:91-148).  Self pairs are skipped inside the search, before the
    ``max_num_neighbors`` cut, on global row numbers."""
    assert flow in ['source_to_target', 'target_to_source']
    ops = ops or _DeviceOps
    x = _as_2d(x)
    s2t = flow == 'source_to_target'
    world, rank, plan = _setup(x, x, batch, batch, batch_size, group, broadcast_inputs, src, plan)
    x_lo, x_hi, y_lo, y_hi, _, _ = plan.ranges[rank]
    if y_hi <= y_lo or x_hi <= x_lo:
        local = torch.empty(2, 0, dtype=torch.long, device=x.device)
    elif plan.ptr_x is not None:
        ptr, _ = plan.local_ptrs(rank, x.device)
        xs = x[x_lo:x_hi]
        local = _shift(ops.radius(xs, xs, ptr, ptr, r, max_num_neighbors, not loop, 0, s2t), x_lo, x_lo)
    else:
        local = ops.radius(x, x[y_lo:y_hi], None, None, r, max_num_neighbors, not loop, y_lo, s2t)
        local = _shift(local, 0, y_lo) if s2t else _shift(local, y_lo, 0)
    return _finish(local, group, world, assemble)

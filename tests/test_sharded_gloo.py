"""The multi-GPU plumbing (partition by segment, index shifting, counts + padded all-gather)
exercised on CPU with two gloo ranks.  The single-GPU operator is replaced by the CPU oracle here:
what is under test is the host logic around it, not a CPU product path."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import neighbor_oracle as orc
from pytorch_cluster_b200.sharded import balanced_ranges, plan


def _oracle_knn(x, y, k, bx, by, cosine=False, batch_size=None):
    e = orc.knn_api(x.numpy(), y.numpy(), k, None if bx is None else bx.numpy(),
                    None if by is None else by.numpy(), cosine=cosine, batch_size=batch_size)
    return torch.from_numpy(e)


def _oracle_radius(x, y, r, bx, by, max_num_neighbors=32, batch_size=None):
    e = orc.radius_api(x.numpy(), y.numpy(), r, None if bx is None else bx.numpy(),
                       None if by is None else by.numpy(), max_num_neighbors, batch_size)
    return torch.from_numpy(e)


def _inputs():
    g = torch.Generator().manual_seed(7)
    sx, sy = [300, 0, 120, 700, 40], [50, 10, 0, 90, 33]
    bx = torch.cat([torch.full((s,), i) for i, s in enumerate(sx)])
    by = torch.cat([torch.full((s,), i) for i, s in enumerate(sy)])
    return torch.rand(sum(sx), 3, generator=g), torch.rand(sum(sy), 3, generator=g), bx, by


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from pytorch_cluster_b200.sharded import knn_sharded, radius_sharded

        x, y, bx, by = _inputs()
        res = {}
        res["knn"] = knn_sharded(x, y, 6, bx, by, compute=_oracle_knn)
        res["knn_single_segment"] = knn_sharded(x, y, 4, compute=_oracle_knn)
        res["radius"] = radius_sharded(x, y, 0.2, bx, by, max_num_neighbors=7, compute=_oracle_radius)
        res["knn_local"] = knn_sharded(x, y, 6, bx, by, compute=_oracle_knn, assemble=False)
        # inputs living on rank 0 only
        if rank != 0:
            x, y, bx, by = torch.zeros_like(x), torch.zeros_like(y), torch.zeros_like(bx), torch.zeros_like(by)
        res["knn_broadcast"] = knn_sharded(x, y, 6, bx, by, batch_size=5, compute=_oracle_knn, broadcast_inputs=True)
        torch.save(res, os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_balanced_ranges_tile_and_balance():
    assert balanced_ranges([1, 1, 1, 1], 2) == [(0, 2), (2, 4)]
    assert balanced_ranges([10, 1, 1, 1, 1, 10], 2) == [(0, 3), (3, 6)]
    r = balanced_ranges([5], 4)
    assert r[0][0] == 0 and r[-1][1] == 1 and all(a[1] == b[0] for a, b in zip(r, r[1:]))
    r = balanced_ranges([0, 0, 0], 2)
    assert r[0][0] == 0 and r[-1][1] == 3


def test_plan_covers_all_rows():
    x, y, bx, by = _inputs()
    p = plan(x.size(0), y.size(0), bx, by, None, 3)
    assert p[0][0] == 0 and p[0][2] == 0 and p[-1][1] == x.size(0) and p[-1][3] == y.size(0)
    for a, b in zip(p, p[1:]):
        assert a[1] == b[0] and a[3] == b[2] and a[5] == b[4]
    p = plan(100, 10, None, None, None, 4)  # one segment: split y, keep x
    assert [q[:4] for q in p] == [(0, 100, 0, 2), (0, 100, 2, 5), (0, 100, 5, 7), (0, 100, 7, 10)]


def test_two_ranks_assemble_the_single_process_result(tmp_path):
    world, port = 2, 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    x, y, bx, by = _inputs()
    want_knn = _oracle_knn(x, y, 6, bx, by)
    want_single = _oracle_knn(x, y, 4, None, None)
    want_radius = _oracle_radius(x, y, 0.2, bx, by, max_num_neighbors=7)
    parts = []
    for rank in range(world):
        res = torch.load(os.path.join(tmp_path, f"rank{rank}.pt"))
        assert torch.equal(res["knn"], want_knn)
        assert torch.equal(res["knn_single_segment"], want_single)
        assert torch.equal(res["radius"], want_radius)
        assert torch.equal(res["knn_broadcast"], want_knn)
        parts.append(res["knn_local"])
    assert torch.equal(torch.cat(parts, dim=1), want_knn)
    assert all(p.shape[1] > 0 for p in parts)

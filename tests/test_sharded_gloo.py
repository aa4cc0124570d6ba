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


def _np(t):
    return None if t is None else t.numpy()


class OracleOps:
    """The single-GPU operators of the sharded layer, answered by the CPU oracle."""

    @staticmethod
    def knn(x, y, ptr_x, ptr_y, k, cosine, max_rows=0):
        return torch.from_numpy(orc.knn(x.numpy(), y.numpy(), k, _np(ptr_x), _np(ptr_y), cosine))

    @staticmethod
    def knn_graph(x, ptr, k, loop, source_to_target, cosine, max_rows=0):
        e = orc.knn(x.numpy(), x.numpy(), k if loop else k + 1, _np(ptr), _np(ptr), cosine)
        row, col = (e[1], e[0]) if source_to_target else (e[0], e[1])
        if not loop:
            keep = row != col
            row, col = row[keep], col[keep]
        return torch.from_numpy(np.stack([row, col]))

    @staticmethod
    def radius(x, y, ptr_x, ptr_y, r, max_num_neighbors, ignore_same_index, query_index_base, swap_rows):
        if query_index_base == 0:
            e = orc.radius(x.numpy(), y.numpy(), r, _np(ptr_x), _np(ptr_y), max_num_neighbors, ignore_same_index)
        else:
            # the oracle has no index base: take one hit more, drop the pair with equal global row
            # numbers, keep the first max_num_neighbors of the rest (hits come in ascending x order)
            e = orc.radius(x.numpy(), y.numpy(), r, _np(ptr_x), _np(ptr_y), max_num_neighbors + 1, False)
            if ignore_same_index:
                e = e[:, e[0] + query_index_base != e[1]]
            rank_in_query = np.arange(e.shape[1]) - np.searchsorted(e[0], e[0], side="left")
            e = e[:, rank_in_query < max_num_neighbors]
        return torch.from_numpy(e[::-1].copy() if swap_rows else e)


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
        from pytorch_cluster_b200.sharded import (knn_graph_sharded, knn_sharded, make_plan, radius_graph_sharded,
                                                  radius_sharded)

        x, y, bx, by = _inputs()
        o = OracleOps
        res = {}
        res["knn"] = knn_sharded(x, y, 6, bx, by, ops=o)
        res["knn_single_segment"] = knn_sharded(x, y, 4, ops=o)
        res["radius"] = radius_sharded(x, y, 0.2, bx, by, max_num_neighbors=7, ops=o)
        res["knn_local"] = knn_sharded(x, y, 6, bx, by, ops=o, assemble=False)
        # a plan made once from host pointer lists: no batch vector is looked at again
        px = torch.bucketize(torch.arange(6), bx).tolist()
        py = torch.bucketize(torch.arange(6), by).tolist()
        p = make_plan(x.size(0), y.size(0), None, None, None, world, ptr_x=px, ptr_y=py)
        res["knn_planned"] = knn_sharded(x, y, 6, plan=p, ops=o)
        # graph forms: batched clouds (slices searched in themselves), one cloud (queries split)
        for flow in ("source_to_target", "target_to_source"):
            res["knn_graph_" + flow] = knn_graph_sharded(x, 5, bx, flow=flow, ops=o)
            res["radius_graph_" + flow] = radius_graph_sharded(x, 0.15, bx, max_num_neighbors=6, flow=flow, ops=o)
            res["knn_graph_one_" + flow] = knn_graph_sharded(x[:400], 5, flow=flow, ops=o)
            res["radius_graph_one_" + flow] = radius_graph_sharded(x[:400], 0.15, max_num_neighbors=6, flow=flow, ops=o)
        res["knn_graph_loop"] = knn_graph_sharded(x[:400], 5, loop=True, ops=o)
        res["radius_graph_loop"] = radius_graph_sharded(x[:400], 0.15, loop=True, max_num_neighbors=6, ops=o)
        # inputs living on rank 0 only
        if rank != 0:
            x, y, bx, by = torch.zeros_like(x), torch.zeros_like(y), torch.zeros_like(bx), torch.zeros_like(by)
        res["knn_broadcast"] = knn_sharded(x, y, 6, bx, by, batch_size=5, ops=o, broadcast_inputs=True)
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


def test_plan_local_pointers_start_at_zero():
    from pytorch_cluster_b200.sharded import make_plan

    p = make_plan(10, 6, None, None, None, 2, ptr_x=[0, 4, 4, 10], ptr_y=[0, 1, 3, 6])
    for rank in range(2):
        x_lo, x_hi, y_lo, y_hi, s0, s1 = p.ranges[rank]
        px, py = p.local_ptrs(rank, "cpu")
        assert px[0] == 0 and py[0] == 0 and px[-1] == x_hi - x_lo and py[-1] == y_hi - y_lo
        assert px.numel() == s1 - s0 + 1


def test_two_ranks_assemble_the_single_process_result(tmp_path):
    world, port = 2, 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    x, y, bx, by = _inputs()
    want_knn = _oracle_knn(x, y, 6, bx, by)
    want_single = _oracle_knn(x, y, 4, None, None)
    want_radius = _oracle_radius(x, y, 0.2, bx, by, max_num_neighbors=7)
    xn, bn = x.numpy(), bx.numpy()
    parts = []
    for rank in range(world):
        res = torch.load(os.path.join(tmp_path, f"rank{rank}.pt"))
        assert torch.equal(res["knn"], want_knn)
        assert torch.equal(res["knn_single_segment"], want_single)
        assert torch.equal(res["radius"], want_radius)
        assert torch.equal(res["knn_broadcast"], want_knn)
        assert torch.equal(res["knn_planned"], want_knn)
        for flow in ("source_to_target", "target_to_source"):
            assert np.array_equal(res["knn_graph_" + flow].numpy(), orc.knn_graph_api(xn, 5, bn, flow=flow))
            assert np.array_equal(res["radius_graph_" + flow].numpy(),
                                  orc.radius_graph_api(xn, 0.15, bn, max_num_neighbors=6, flow=flow))
            assert np.array_equal(res["knn_graph_one_" + flow].numpy(), orc.knn_graph_api(xn[:400], 5, flow=flow))
            assert np.array_equal(res["radius_graph_one_" + flow].numpy(),
                                  orc.radius_graph_api(xn[:400], 0.15, max_num_neighbors=6, flow=flow))
        assert np.array_equal(res["knn_graph_loop"].numpy(), orc.knn_graph_api(xn[:400], 5, loop=True))
        assert np.array_equal(res["radius_graph_loop"].numpy(),
                              orc.radius_graph_api(xn[:400], 0.15, loop=True, max_num_neighbors=6))
        parts.append(res["knn_local"])
    assert torch.equal(torch.cat(parts, dim=1), want_knn)
    assert all(p.shape[1] > 0 for p in parts)


# ---- failures made on the host: no collective may hang, every rank must come back with an error --------

def _failing_worker(rank, world, port, out_dir, mode):
    import datetime

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    outcome = "ok"
    try:
        from pytorch_cluster_b200.sharded import knn_sharded, make_plan

        x, y, bx, by = _inputs()
        if mode == "raise_before_collective":
            # rank 1's operator raises; it never joins the assembly, rank 0's collective must end by
            # the process-group timeout instead of waiting for ever
            class Broken(OracleOps):
                @staticmethod
                def knn(*a):
                    if rank == 1:
                        raise RuntimeError("injected failure on rank 1")
                    return OracleOps.knn(*a)

            knn_sharded(x, y, 6, bx, by, ops=Broken)
        elif mode == "plan_for_other_world":
            p = make_plan(x.size(0), y.size(0), bx, by, None, world + 1)
            knn_sharded(x, y, 6, bx, by, plan=p, ops=OracleOps)
    except AssertionError as e:
        outcome = "assert: " + str(e)
    except RuntimeError as e:
        outcome = "error: " + str(e)[:80]
    finally:
        with open(os.path.join(out_dir, f"{mode}_{rank}.txt"), "w") as f:
            f.write(outcome)
        try:
            dist.destroy_process_group()
        except Exception:
            pass


@pytest.mark.parametrize("mode", ["raise_before_collective", "plan_for_other_world"])
def test_host_side_failures_end_with_errors_not_hangs(tmp_path, mode):
    world, port = 2, 31500 + os.getpid() % 2000 + (7 if mode.startswith("plan") else 0)
    mp.spawn(_failing_worker, args=(world, port, str(tmp_path), mode), nprocs=world, join=True)
    got = [open(os.path.join(tmp_path, f"{mode}_{r}.txt")).read() for r in range(world)]
    if mode == "raise_before_collective":
        assert got[1].startswith("error: injected failure")
        assert got[0].startswith("error:")  # the collective gave up: timeout or a closed connection
    else:
        assert all(g.startswith("assert: the plan was made for another world size") for g in got)

"""Two NCCL ranks on two GPUs: the sharded calls return the single-GPU result on every rank.
Skipped on boxes with one GPU."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import pytorch_cluster_b200 as pc

        dev = torch.device("cuda", rank)
        g = torch.Generator().manual_seed(3)
        sizes = [3000, 500, 0, 4000, 1200, 2500]
        batch = torch.cat([torch.full((s,), i) for i, s in enumerate(sizes)]).to(dev)
        x = torch.rand(sum(sizes), 3, generator=g).to(dev)
        y = x[::3].contiguous()
        by = batch[::3].contiguous()
        # every check is evaluated (no short circuit): each sharded call is a collective both ranks must enter
        checks = {}
        checks["knn"] = torch.equal(pc.knn(x, y, 16, batch, by), pc.knn_sharded(x, y, 16, batch, by))
        got_knn = pc.knn_sharded(x, y, 16, batch, by)
        checks["radius"] = torch.equal(pc.radius(x, y, 0.05, batch, by, max_num_neighbors=64),
                                       pc.radius_sharded(x, y, 0.05, batch, by, max_num_neighbors=64))
        checks["knn_one_segment"] = torch.equal(pc.knn_sharded(x, y, 8), pc.knn(x, y, 8))  # queries split, x whole
        # graph forms: batched clouds, then one cloud (its queries split over the ranks); a plan reused
        plan = pc.make_plan(x.size(0), x.size(0), batch, batch, len(sizes), world)
        one = x[:3000].contiguous()
        for flow in ("source_to_target", "target_to_source"):
            checks["knn_graph_" + flow] = torch.equal(pc.knn_graph_sharded(x, 12, batch, flow=flow, plan=plan),
                                                      pc.knn_graph(x, 12, batch, flow=flow))
            for cap in (9, 4000):
                checks[f"radius_graph_{flow}_{cap}"] = torch.equal(
                    pc.radius_graph_sharded(x, 0.05, batch, max_num_neighbors=cap, flow=flow, plan=plan),
                    pc.radius_graph(x, 0.05, batch, max_num_neighbors=cap, flow=flow))
                checks[f"radius_graph_one_{flow}_{cap}"] = torch.equal(
                    pc.radius_graph_sharded(one, 0.05, max_num_neighbors=cap, flow=flow),
                    pc.radius_graph(one, 0.05, max_num_neighbors=cap, flow=flow))
            checks["knn_graph_one_" + flow] = torch.equal(pc.knn_graph_sharded(one, 12, flow=flow),
                                                          pc.knn_graph(one, 12, flow=flow))
        checks["radius_graph_loop"] = torch.equal(pc.radius_graph_sharded(one, 0.05, loop=True),
                                                  pc.radius_graph(one, 0.05, loop=True))
        local = pc.radius_graph_sharded(x, 0.05, batch, max_num_neighbors=9, assemble=False)
        checks["local_slice_not_empty"] = local.shape[1] > 0
        failed = sorted(k for k, v in checks.items() if not v)
        torch.save({"ok": not failed, "failed": failed, "edges": int(got_knn.shape[1])},
                   os.path.join(out_dir, f"rank{rank}.pt"))
        torch.cuda.synchronize()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_equals_single_gpu(tmp_path):
    import torch.multiprocessing as mp

    world, port = 2, 29600 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for rank in range(world):
        res = torch.load(os.path.join(tmp_path, f"rank{rank}.pt"))
        assert res["ok"] and res["edges"] > 0, res["failed"]


def test_a_slice_of_the_queries_skips_the_pair_with_equal_global_rows():
    """What a rank of radius_graph_sharded does for one cloud, on one GPU: the queries are a slice of x,
    `query_index_base` tells the search which x row is the query itself — for every neighbour cap the
    slices put side by side are the result of the whole call, with and without the row swap."""
    import pytorch_cluster_b200  # noqa: F401

    part = torch.ops.torch_cluster.radius_part
    g = torch.Generator().manual_seed(11)
    for dim, dtype, r in ((3, torch.float, 0.08), (3, torch.double, 0.08), (12, torch.float, 0.9), (3, torch.half, 0.08)):
        x = torch.rand(5000, dim, generator=g).to("cuda:0", dtype)
        for cap in (3, 40, 600):
            for swap in (False, True):
                whole = part(x, x, None, None, r, cap, True, 0, swap)
                cuts = [0, 1700, 1701, 4000, 5000]
                pieces = []
                for lo, hi in zip(cuts, cuts[1:]):
                    e = part(x, x[lo:hi].contiguous(), None, None, r, cap, True, lo, swap)
                    e[1 if swap else 0] += lo
                    pieces.append(e)
                assert torch.equal(torch.cat(pieces, dim=1), whole), (dim, dtype, cap, swap)
                found = torch.ops.torch_cluster.radius(x, x, None, None, r, cap, 1, True)
                assert torch.equal(whole, found.flip(0) if swap else found)
                assert not bool((whole[0] == whole[1]).any())


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_one_process_two_devices():
    """One process using both GPUs in turn: launch configuration (the shared-memory opt-in of every
    kernel) is per device, and results do not depend on the device."""
    import pytorch_cluster_b200 as pc

    g = torch.Generator().manual_seed(5)
    x = torch.randn(6000, 3, generator=g)
    f = torch.randn(4096, 64, generator=g)
    batch = torch.arange(3).repeat_interleave(2000)
    res = []
    for d in ("cuda:0", "cuda:1", "cuda:0"):
        xd, bd, fd = x.to(d), batch.to(d), f.to(d)
        samples = pc.fps(xd, bd, ratio=0.1, random_start=False)
        res.append([t.cpu() for t in (
            pc.knn_graph(xd, 12, bd), pc.radius_graph(xd, 0.2, bd, max_num_neighbors=40),
            pc.knn(fd, fd, 9), pc.knn(fd, fd, 9, cosine=True), samples, pc.nearest(xd, xd[samples], bd, bd[samples]),
            pc.knn_graph_host(x, 12, batch, device=torch.device(d)))])
    for other in res[1:]:
        for a, b in zip(res[0], other):
            assert torch.equal(a, b)

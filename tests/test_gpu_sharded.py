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
        want_knn = pc.knn(x, y, 16, batch, by)
        got_knn = pc.knn_sharded(x, y, 16, batch, by)
        want_rad = pc.radius(x, y, 0.05, batch, by, max_num_neighbors=64)
        got_rad = pc.radius_sharded(x, y, 0.05, batch, by, max_num_neighbors=64)
        one = pc.knn_sharded(x, y, 8)  # single segment: queries split, x whole
        ok = (torch.equal(want_knn, got_knn) and torch.equal(want_rad, got_rad)
              and torch.equal(one, pc.knn(x, y, 8)))
        torch.save({"ok": bool(ok), "edges": int(got_knn.shape[1])}, os.path.join(out_dir, f"rank{rank}.pt"))
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
        assert res["ok"] and res["edges"] > 0


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

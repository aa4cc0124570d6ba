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

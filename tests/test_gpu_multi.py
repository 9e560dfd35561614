"""Two-GPU check of the sharded encode and the NCCL gather of packed codes (skipped on a single GPU)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from trellis_b200 import dist as tdist, qtip
        g = torch.Generator(device="cuda").manual_seed(123)          # same tiles on every rank
        tiles = torch.randn(301, 256, generator=g, device="cuda")
        every, local, (lo, hi) = tdist.encode_sharded(tiles, 3, "3inst")
        only0, _, _ = tdist.encode_sharded(tiles, 3, "3inst", dst=0)
        full = qtip.encode(tiles, 3, "3inst").packed
        ok = torch.equal(every, full) and torch.equal(local.packed, full[lo:hi]) and ((only0 is None) == (rank != 0))
        if rank == 0:
            ok = ok and torch.equal(only0, full)
        torch.cuda.synchronize()
        open(os.path.join(tmp, f"r{rank}"), "w").write("ok" if ok else "mismatch")
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_encode_and_nccl_gather(tmp_path):
    port = 30500 + os.getpid() % 2000
    mp.start_processes(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True, start_method="spawn")
    assert open(os.path.join(tmp_path, "r0")).read() == "ok"
    assert open(os.path.join(tmp_path, "r1")).read() == "ok"

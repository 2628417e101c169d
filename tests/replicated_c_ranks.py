"""Rank program of the two-GPU test (launched by tests/test_gemm_gpu.py under torch.distributed.run, NCCL): each rank
runs its M-row slab through ShardedGemm with a replicated C and compares the gathered C with the oracle's product."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from oracle import gemm_ref  # noqa: E402
from warpc_public_release_b200 import shard  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    for (m, n, k) in ((1024, 1024, 512), (4096, 2048, 1024)):
        a, bt = gemm_ref.inputs_integers(m, n, k)
        lo, hi = shard.slab_rows(m, world, rank)
        job = shard.ShardedGemm(m, n, k, rank, world, torch.from_numpy(a[lo:hi]).to(dev), torch.from_numpy(bt).to(dev), replicate_c=True, device=dev)
        for _ in range(3):
            c = job.launch()
        job.plan.status()
        job.wait()
        torch.cuda.synchronize()
        assert np.array_equal(c.cpu().numpy(), gemm_ref.gemm_ref(a, bt)), "rank %d: gathered C differs at %dx%dx%d" % (rank, m, n, k)
    dist.barrier()
    print("replicated C ok (rank %d)" % rank, flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

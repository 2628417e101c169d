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
    # shapes whose slab program stores through staging copies (the copy to the other GPUs can be fused into the kernel) and
    # one whose program stores from the registers (falls back to NCCL); both ways of replicating asked for explicitly
    import warpc_public_release_b200 as w
    clc = lambda r, n, k: w.swapped(r, n, k, 256, 256, 4, clc=True, serpentine=True, ask_ahead=True)   # the large shape's program
    stride = lambda r, n, k: w.swapped(r, n, k, 128, 128, 8, bufs=2)                                    # a fixed grid, two accumulators
    fold = lambda r, n, k: w.swapped(r, n, k, 128, 64, 13)                                              # one tile a CTA, staged store
    cases = [((1024, 1024, 512), "fused", fold, "fused"),
             ((1024, 1024, 512), "fused", None, "nccl"),           # the rule's program for the slab stores from the registers
             ((4096, 4096, 1024), "fused", clc, "fused"), ((8192, 2304, 256), "fused", stride, "fused"),
             ((8192, 4096, 1024), "fused", None, "nccl"),          # the rule's program stores from the registers: NCCL in row bands
             ((8192, 4096, 1024), "nccl", clc, "nccl"),
             ((4096, 4096, 4096), "fused", None, "nccl")]          # the rule's program shares K between CTAs (stream-K): one launch, one all-gather
    for (m, n, k), how, build, runs in cases:
        a, bt = gemm_ref.inputs_integers(m, n, k)
        lo, hi = shard.slab_rows(m, world, rank)
        job = shard.ShardedGemm(m, n, k, rank, world, torch.from_numpy(a[lo:hi]).to(dev), torch.from_numpy(bt).to(dev), replicate_c=True, device=dev,
                                how=how, variant=build(hi - lo, n, k) if build else None)
        assert job.how == runs, (m, n, k, how, job.how)
        for _ in range(3):
            c = job.launch()
            job.wait()
        job.status()
        torch.cuda.synchronize()
        assert np.array_equal(c.cpu().numpy(), gemm_ref.gemm_ref(a, bt)), "rank %d: gathered C differs at %dx%dx%d (%s)" % (rank, m, n, k, job.how)
        print("rank %d %dx%dx%d asked %s ran %s" % (rank, m, n, k, how, job.how), flush=True)
        dist.barrier()
        job.close()
        del job
        dist.barrier()
    dist.barrier()
    print("replicated C ok (rank %d)" % rank, flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

"""The multi-GPU plan's host logic on CPU ranks (gloo, world size 2): which rows a rank owns,
which program its slab gets, and that gathering the slabs in rank order rebuilds C.  The slabs'
values come from the oracle here (no GPU); the GPU path swaps in the kernel for that one step."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, m, n, k, out_dir):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from warpc_public_release_b200 import shard
    from oracle import gemm_ref
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    a, bt = gemm_ref.inputs_integers(m, n, k)          # every rank draws the same matrices, keeps its rows
    lo, hi = shard.slab_rows(m, world, rank)
    c_full = torch.full((m, n), float("nan"), dtype=torch.float32)
    c_local = c_full[lo:hi]
    c_local.copy_(torch.from_numpy(gemm_ref.gemm_ref(a[lo:hi], bt)))   # stand-in for the rank's kernel launch
    shard.gather_slabs(c_full, c_local)
    np.save(os.path.join(out_dir, "c_rank%d.npy" % rank), c_full.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_row_sharded_gemm_world_size_2(tmp_path):
    import torch.multiprocessing as mp
    from oracle import gemm_ref
    m, n, k, world = 512, 256, 128, 2
    mp.spawn(_rank_main, args=(world, _free_port(), m, n, k, str(tmp_path)), nprocs=world, join=True)
    a, bt = gemm_ref.inputs_integers(m, n, k)
    ref = gemm_ref.gemm_ref(a, bt)
    for r in range(world):
        assert np.array_equal(np.load(tmp_path / ("c_rank%d.npy" % r)), ref)


def test_slab_rows_and_programs():
    from warpc_public_release_b200 import shard
    assert [shard.slab_rows(16384, 8, r) for r in (0, 3, 7)] == [(0, 2048), (6144, 8192), (14336, 16384)]
    with pytest.raises(ValueError):
        shard.slab_rows(1000, 3, 0)
    covered = sorted(shard.slab_rows(16384, 4, r) for r in range(4))
    assert covered[0][0] == 0 and covered[-1][1] == 16384 and all(covered[i][1] == covered[i + 1][0] for i in range(3))
    # the slabs of the sharded shape keep the large-shape program while their 512 x 256 pair tiles fill the last wave of the
    # 74 resident pairs (13.8 and 6.9 waves on 2 and 4 GPUs); at 8 GPUs (3.46 waves) the rule's own program, re-tiled, runs
    for g in (1, 2, 4):
        v = shard.slab_variant(16384 // g, 16384, 16384)
        assert (v.tile_m, v.tile_n, v.depth, v.clc, v.serpentine) == (256, 256, 4, 1, 1)
    import warpc_public_release_b200 as w
    v = shard.slab_variant(2048, 16384, 16384)
    li = w.realise(v, 2048, 16384, 16384)
    assert (v.tile_m, v.tile_n) == (192, 128) and (li.tile_m, li.tile_n, li.sched, li.direct) == (256, 128, 1, 1)
    v = shard.slab_variant(2048, 16384, 16384, staged=True)          # the kernel is to fill other GPUs' copies of C too
    assert (v.tile_m, v.tile_n, v.clc) == (256, 256, 1)
    v = shard.slab_variant(2048, 16384, 16384, pin_large=False)
    assert (v.tile_m, v.tile_n) == (192, 128)
    v = shard.slab_variant(1024, 1024, 1024)
    assert (v.tile_m, v.tile_n) == (128, 64)


def test_row_bands_and_which_slabs_can_take_fused_copies():
    import warpc_public_release_b200 as w
    from warpc_public_release_b200 import shard
    # bands: whole 256-row tile rows, contiguous, covering the slab, as equal as whole tiles allow
    assert shard.band_rows(8192, 4, 256) == [(0, 2048), (2048, 4096), (4096, 6144), (6144, 8192)]
    assert shard.band_rows(512, 4, 256) == [(0, 256), (256, 512)]
    assert shard.band_rows(2304, 4, 256) == [(0, 512), (512, 1024), (1024, 1536), (1536, 2304)]
    for rows in (256, 1280, 2048, 4352):
        bands = shard.band_rows(rows, 4, 256)
        assert bands[0][0] == 0 and bands[-1][1] == rows and all(a[1] == b[0] for a, b in zip(bands, bands[1:]))
        assert all(b0 % 256 == 0 for b0, _ in bands)
    # a replicated C can be fused into programs that store through staging copies and do not share K between CTAs
    big = shard.slab_variant(8192, 16384, 16384)
    assert not shard.realise_sched_direct(big, 8192, 16384, 16384)                       # 256 x 256, launch control
    assert shard.realise_sched_direct(shard.slab_variant(4096, 4096, 1024), 4096, 4096, 1024)   # stores from the registers
    assert shard.realise_sched_direct(shard.slab_variant(2048, 4096, 4096), 2048, 4096, 4096)   # stream-K

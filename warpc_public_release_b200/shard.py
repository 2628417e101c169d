"""The largest shape across the GPUs of one box: M split in contiguous row blocks, one process
per GPU (torch.distributed / NCCL for the plumbing only).

Rank r of g holds A[r M/g : (r+1) M/g, :], all of Bt, and produces C[r M/g : (r+1) M/g, :]
(row-major, so each slab is contiguous).  The GEMM itself exchanges nothing.  Only when a
replicated C is asked for does a collective run: one in-place NCCL all-gather of the slabs over
NVLink.  The reference has no multi-GPU path (its harness opens device 0 only,
backend/node/cuda.py:105-114); the per-GPU program is what its rule picks for the slab's shape
(backend/programs.ml:46-80), or the 256 x 256 program pinned when the slab keeps whole tiles.
"""
from . import programs


def slab_rows(m, world, rank):
    """Rows [lo, hi) of A and C that `rank` of `world` owns: equal contiguous blocks."""
    if m % world != 0:
        raise ValueError("M = %d does not split into %d equal row blocks" % (m, world))
    rows = m // world
    return rank * rows, (rank + 1) * rows


def slab_variant(m_local, n, k, pin_large=True):
    """The program for one GPU's (M/g) x N x K share.  The rule falls back to 192 x 128 tiles
    once min(M/g, N, K) < 8192; a slab that still holds whole 256 x 256 pair tiles keeps the
    large-shape program (cluster launch control, serpentine walk, asking ahead).  (Dealing a poorly
    filled last wave's k-steps out stream-K does not pay at this tile: 2048 x 16384 x 16384, 3.46 waves,
    measured 965 us against 757 us -- the partial tiles' 256 KB stores are exposed and clusters stop
    sharing operand panels in step.)"""
    if pin_large and m_local % 256 == 0 and n % 512 == 0 and k % 64 == 0 and min(n, k) >= 8192 and \
            (m_local // 256) * (n // 256) >= 148:
        return programs.swapped(m_local, n, k, 256, 256, 4, clc=True, ask_ahead=True, serpentine=True)
    return programs.choose(m_local, n, k)


def gather_slabs(c_full, c_local):
    """Replicate C: every rank's slab into every rank's `c_full` (row blocks in rank order).
    `c_local` may be the rank's own rows of `c_full` (in place)."""
    import torch.distributed as dist
    if dist.get_backend() == "nccl":
        dist.all_gather_into_tensor(c_full, c_local)
    else:  # gloo on CPU ranks (tests): a list of row-block views
        world = dist.get_world_size()
        rows = c_full.shape[0] // world
        mine = c_local.clone()
        dist.all_gather([c_full[r * rows:(r + 1) * rows] for r in range(world)], mine)
    return c_full


class ShardedGemm:
    """One rank's share of C = A . Bt^T.  `a_local` (M/g x K fp16), `bt` (N x K fp16) are this
    rank's CUDA tensors; `c_full` (M x N fp32) is allocated on every rank only when
    `replicate_c` (the slab then lives inside it, so the all-gather is in place)."""

    def __init__(self, m, n, k, rank, world, a_local, bt, replicate_c=False, device=None, pin_large=True):
        import torch
        from .plan import Plan
        self.m, self.n, self.k, self.rank, self.world = m, n, k, rank, world
        self.lo, self.hi = slab_rows(m, world, rank)
        rows = self.hi - self.lo
        if tuple(a_local.shape) != (rows, k) or tuple(bt.shape) != (n, k):
            raise ValueError("A slab must be %d x %d and Bt %d x %d" % (rows, k, n, k))
        device = a_local.device if device is None else device
        self.replicate_c = replicate_c
        if replicate_c:
            self.c_full = torch.empty((m, n), dtype=torch.float32, device=device)
            self.c_local = self.c_full[self.lo:self.hi]
        else:
            self.c_full = None
            self.c_local = torch.empty((rows, n), dtype=torch.float32, device=device)
        self.variant = slab_variant(rows, n, k, pin_large)
        self.plan = Plan(self.variant, rows, n, k, a_local.data_ptr(), bt.data_ptr(), self.c_local.data_ptr(),
                         device=device.index or 0)
        self._keep = (a_local, bt)

    def launch(self):
        """This rank's GEMM (asynchronous, default stream); with `replicate_c`, followed by the all-gather."""
        self.plan.launch()
        if self.replicate_c and self.world > 1:
            gather_slabs(self.c_full, self.c_local)
        return self.c_full if self.replicate_c else self.c_local

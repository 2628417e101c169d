"""The largest shape across the GPUs of one box: M split in contiguous row blocks, one process
per GPU (torch.distributed / NCCL for the plumbing only).

Rank r of g holds A[r M/g : (r+1) M/g, :], all of Bt, and produces C[r M/g : (r+1) M/g, :]
(row-major, so each slab is contiguous).  The GEMM itself exchanges nothing.  Only when a
replicated C is asked for does a collective run: one in-place NCCL all-gather of the slabs over
NVLink.  The reference has no multi-GPU path (its harness opens device 0 only,
backend/node/cuda.py:105-114); the per-GPU program is what its rule picks for the slab's shape
(backend/programs.ml:46-80), or the 256 x 256 program pinned when the slab keeps whole tiles.
"""
import os

from . import programs


def slab_rows(m, world, rank):
    """Rows [lo, hi) of A and C that `rank` of `world` owns: equal contiguous blocks."""
    if m % world != 0:
        raise ValueError("M = %d does not split into %d equal row blocks" % (m, world))
    rows = m // world
    return rank * rows, (rank + 1) * rows


RESIDENT_PAIRS = 74   # CTA pairs the machine holds at one CTA an SM


def slab_variant(m_local, n, k, pin_large=True, staged=False):
    """The program for one GPU's (M/g) x N x K share.  The rule falls back to 192 x 128 tiles
    once min(M/g, N, K) < 8192; a slab that still holds whole 256 x 256 pair tiles keeps the
    large-shape program (cluster launch control, serpentine walk, asking ahead) -- as long as its
    512 x 256 pair tiles fill their last wave of the 74 resident pairs: 16384^3 over 2 and 4 GPUs is 13.8 and 6.9
    waves, over 8 GPUs 3.46, a seventh of the machine idle at the end.  There the rule's own program, re-tiled to
    256 x 128 on a fixed grid (6.9 waves again), is the faster one: 2048 x 16384 x 16384 on one GPU, twenty launches
    back to back, 721-870 us against 762-984 (cuBLASLt 727-854); on eight GPUs in one job, the slowest rank's time,
    820-842 against 802-1060 over sixty launches back to back (779 against 774 on GPUs that had idled).  (Dealing the poorly filled last wave's k-steps out
    stream-K does not pay at the large tile: 965 us against 757 -- the partial tiles' 256 KB stores are exposed and
    clusters stop sharing operand panels in step.)  `staged`: the caller needs a program that stores through staging
    copies (further copies of C filled by the kernel itself), which the re-tiled one does not: the large program then."""
    if pin_large and m_local % 256 == 0 and n % 512 == 0 and k % 64 == 0 and min(n, k) >= 8192 and \
            (m_local // 256) * (n // 256) >= 148:
        pairs = (m_local // 256) * (n // 256) // 2
        waves = -(-pairs // RESIDENT_PAIRS)
        if staged or 20 * pairs >= 19 * waves * RESIDENT_PAIRS:     # the last wave at least 95 % full
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
    `replicate_c` (the slab then lives inside it, so the gather is in place).

    With `replicate_c` the copy to the other GPUs is part of the GEMM itself (`how` = "fused", the default where it can
    be set up): every rank opens the other ranks' C through CUDA IPC, and the kernel stores each staged block of its
    slab to every GPU's copy, tile by tile, with TMA stores over NVLink -- no collective kernel runs and no SM is
    taken from the tensor cores' work; wait() is then a one-word all-reduce that tells every rank the others' launches
    are done.  Where that cannot be set up (`how` = "nccl": no peer access, a program that stores from the registers
    or shares K between CTAs) the slab is computed in `bands` row bands, one launch each on two alternating streams,
    and each band is sent to every other rank as soon as its launch is done: one group of NCCL sends and receives per
    band, straight into place (a band of every rank's slab is whole rows of C, so it is contiguous), on NCCL's own
    stream.  Programs whose CTAs wait for one another (split-K, stream-K) are not overlapped with NCCL's kernels,
    which take SMs: one launch, then one all-gather."""

    def __init__(self, m, n, k, rank, world, a_local, bt, replicate_c=False, device=None, pin_large=True, bands=4, how=None, variant=None):
        import torch
        from .plan import Plan
        from .programs import realise
        self.m, self.n, self.k, self.rank, self.world = m, n, k, rank, world
        self.lo, self.hi = slab_rows(m, world, rank)
        rows = self.hi - self.lo
        if tuple(a_local.shape) != (rows, k) or tuple(bt.shape) != (n, k):
            raise ValueError("A slab must be %d x %d and Bt %d x %d" % (rows, k, n, k))
        device = a_local.device if device is None else device
        self.device = device
        self.replicate_c = replicate_c
        if replicate_c:
            self.c_full = torch.empty((m, n), dtype=torch.float32, device=device)
            self.c_local = self.c_full[self.lo:self.hi]
        else:
            self.c_full = None
            self.c_local = torch.empty((rows, n), dtype=torch.float32, device=device)
        # `variant`: a program named by the caller for the slab's shape; else the slab's own (with a replicated C one the
        # kernel itself can send on: stored through staging copies)
        fusable = replicate_c and world > 1 and (how or os.environ.get("WARPC_REPLICATE", "fused")) == "fused"
        self.variant = variant if variant is not None else slab_variant(rows, n, k, pin_large, staged=fusable)
        dev_index = device.index or 0
        self.plan = Plan(self.variant, rows, n, k, a_local.data_ptr(), bt.data_ptr(), self.c_local.data_ptr(), device=dev_index)
        self._keep = (a_local, bt)
        self.band_plans, self._pending = [], []
        self.how = None
        if replicate_c and world > 1 and device.type == "cuda":
            want = how or os.environ.get("WARPC_REPLICATE", "fused")
            self.how = "fused" if want == "fused" and self._open_peers() else "nccl"
        if self.how == "nccl":
            self.band_rows = band_rows(rows, bands, 256)
            for (b0, b1) in self.band_rows:
                try:
                    v = slab_variant(b1 - b0, n, k, pin_large)
                    shares_k = realise(v, b1 - b0, n, k).sched in (3, 4)
                except Exception:
                    shares_k = True        # the rule has no program for a band of this height: the slab stays whole
                if shares_k:
                    self.band_plans = []   # CTAs that wait for one another: no NCCL kernel beside them, one launch then one gather
                    break
                self.band_plans.append(Plan(v, b1 - b0, n, k, a_local[b0:b1].data_ptr(), bt.data_ptr(), self.c_local[b0:b1].data_ptr(), device=dev_index))
            if self.band_plans:
                self._streams = [torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)]

    def _open_peers(self):
        """Every other rank's `c_full` mapped into this process for this rank's GPU (CUDA IPC, imported with this GPU
        current so the mapping carries peer access), and this rank's rows of each given to the plan as further copies
        of C.  False when any rank cannot (the ranks agree on the answer, so all take the same path)."""
        import torch
        import torch.distributed as dist
        from . import plan as wplan
        dev_index = self.device.index or 0
        ok, mine, peers = True, None, []
        try:
            if realise_sched_direct(self.variant, self.hi - self.lo, self.n, self.k):
                raise RuntimeError("the slab's program stores from the registers or shares K between CTAs")
            mine = wplan.ipc_export(self.c_full.data_ptr(), device=dev_index)
        except Exception:
            ok = False
        everyone = [None] * self.world
        dist.all_gather_object(everyone, (dev_index, mine))
        ok = ok and all(x[1] is not None for x in everyone)
        if ok:
            try:
                for q, (their_device, (handle, offset)) in enumerate(everyone):
                    if q == self.rank:
                        continue
                    if not torch.cuda.can_device_access_peer(dev_index, their_device):
                        raise RuntimeError("no peer access from GPU %d to GPU %d" % (dev_index, their_device))
                    peers.append(wplan.ipc_import(handle, offset, device=dev_index))
            except Exception:
                ok = False
        flag = torch.tensor([1 if ok else 0], device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            for ptr in peers:
                wplan.ipc_release(ptr, device=dev_index)
            return False
        self._peers = peers
        slab_offset = self.lo * self.n * 4               # this rank's rows inside every copy of C
        self.plan.set_replicas([ptr + slab_offset for ptr in peers])
        self._token = torch.zeros(1, device=self.device)
        return True

    def close(self):
        """Give the other ranks' buffers back.  Call it on every rank once all ranks are done launching (after a barrier)
        and before any rank frees its `c_full`: a kernel still running elsewhere may be writing this rank's copy."""
        from . import plan as wplan
        if getattr(self, "_peers", None):
            self.plan.set_replicas([])     # synchronises this device
            for ptr in self._peers:
                wplan.ipc_release(ptr, device=self.device.index or 0)
            self._peers = []

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def launch(self):
        """This rank's GEMM (asynchronous).  Without `replicate_c`: one launch on the default stream.  With it: the
        launch also fills the other ranks' copies (fused), or the bands' launches and their gathers are queued (nccl);
        call wait() before reading `c_full`."""
        import torch
        if not (self.replicate_c and self.world > 1):
            self.plan.launch()
            return self.c_local
        if self.how == "fused":
            self.plan.launch()
            return self.c_full
        if not self.band_plans:
            self.plan.launch()
            gather_slabs(self.c_full, self.c_local)
            return self.c_full
        import torch.distributed as dist
        rows = self.hi - self.lo
        start = torch.cuda.current_stream(self.device)
        for i, ((b0, b1), plan) in enumerate(zip(self.band_rows, self.band_plans)):
            s = self._streams[i % 2]
            if i < 2:
                s.wait_stream(start)   # what the caller queued before (the inputs) comes first
            with torch.cuda.stream(s):
                plan.launch(stream=s.cuda_stream)
                ops = []
                for q in range(self.world):
                    if q == self.rank:
                        continue
                    ops.append(dist.P2POp(dist.isend, self.c_local[b0:b1], q))
                    ops.append(dist.P2POp(dist.irecv, self.c_full[q * rows + b0:q * rows + b1], q))
                self._pending += dist.batch_isend_irecv(ops)   # NCCL's stream waits for this band's launch, not for the next
        return self.c_full

    def wait(self):
        """Make the current stream wait for everything launch() queued (band launches and gathers)."""
        import torch
        if self.how == "fused":
            import torch.distributed as dist
            dist.all_reduce(self._token)   # stream-ordered behind this rank's launch; done when every rank's launch is
            return
        if self.band_plans:
            cur = torch.cuda.current_stream(self.device)
            for work in self._pending:
                work.wait()
            self._pending = []
            for s in self._streams:
                cur.wait_stream(s)

    def status(self):
        self.plan.status()
        for p in self.band_plans:
            p.status()


class ShardedHostGemm:
    """The sharded product from HOST buffers, one rank's part: `run(hA, hBt_shard, hC)` takes this rank's rows of A
    (M/g x K), this rank's rows of Bt (N/g x K) and gives this rank's rows of C (M/g x N), all in pinned host memory.
    Every operand crosses PCIe once in the whole job: each rank uploads only its own rows of Bt, and the shards are
    gathered into every GPU's copy of Bt by one in-place NCCL all-gather over NVLink (plain NCCL on each GPU's own
    buffer).  A's rows go in and C's rows come out in row bands on streams of their own, a band's launch waiting only
    for that band of A (and for Bt), so the copies in, the tensor cores and the copies out overlap."""

    def __init__(self, m, n, k, rank, world, device, bands=None, pin_large=True):
        import torch
        from .plan import Plan
        self.m, self.n, self.k, self.rank, self.world, self.device = m, n, k, rank, world, device
        self.lo, self.hi = slab_rows(m, world, rank)
        self.blo, self.bhi = slab_rows(n, world, rank)
        rows = self.hi - self.lo
        self.a = torch.empty((rows, k), dtype=torch.float16, device=device)
        self.bt = torch.empty((n, k), dtype=torch.float16, device=device)
        self.c = torch.empty((rows, n), dtype=torch.float32, device=device)
        bands = bands or max(1, min(4, rows // 1024))
        self.bands = band_rows(rows, bands, 256)
        self.plans = [Plan(slab_variant(b1 - b0, n, k, pin_large), b1 - b0, n, k, self.a[b0:b1].data_ptr(), self.bt.data_ptr(),
                           self.c[b0:b1].data_ptr(), device=device.index or 0) for (b0, b1) in self.bands]
        self.s_in, self.s_mm, self.s_out = (torch.cuda.Stream(device=device) for _ in range(3))
        self.ev_bt = torch.cuda.Event()
        self.ev_a = [torch.cuda.Event() for _ in self.bands]
        self.ev_mm = [torch.cuda.Event() for _ in self.bands]
        self.h2d_bytes = rows * k * 2 + (self.bhi - self.blo) * k * 2
        self.d2h_bytes = rows * n * 4

    def run(self, hA, hBt_shard, hC):
        """hA (M/g x K fp16), hBt_shard (N/g x K fp16), hC (M/g x N fp32): pinned CPU tensors.  Returns when hC is complete."""
        import torch
        import torch.distributed as dist
        with torch.cuda.stream(self.s_in):
            self.bt[self.blo:self.bhi].copy_(hBt_shard, non_blocking=True)
            self.ev_bt.record()
            for (b0, b1), ev in zip(self.bands, self.ev_a):
                self.a[b0:b1].copy_(hA[b0:b1], non_blocking=True)
                ev.record()
        with torch.cuda.stream(self.s_mm):
            self.s_mm.wait_event(self.ev_bt)
            if self.world > 1:
                dist.all_gather_into_tensor(self.bt, self.bt[self.blo:self.bhi])   # in place: every rank's shard to every GPU
            for plan, ev_a, ev_mm in zip(self.plans, self.ev_a, self.ev_mm):
                self.s_mm.wait_event(ev_a)
                plan.launch(stream=self.s_mm.cuda_stream)
                ev_mm.record()
        with torch.cuda.stream(self.s_out):
            for (b0, b1), ev in zip(self.bands, self.ev_mm):
                self.s_out.wait_event(ev)
                hC[b0:b1].copy_(self.c[b0:b1], non_blocking=True)
        self.s_out.synchronize()

    def status(self):
        for p in self.plans:
            p.status()

    def close(self):
        for p in self.plans:
            p.close()


def realise_sched_direct(variant, m, n, k):
    """True when the program for this shape cannot take further copies of C (wg_plan_set_replicas refuses it)."""
    from .programs import realise
    li = realise(variant, m, n, k)
    return bool(li.direct) or li.sched in (3, 4)


def band_rows(rows, bands, tile_m):
    """`rows` cut into at most `bands` contiguous bands of whole tile rows, as equal as whole tiles allow."""
    tiles = max(1, rows // tile_m)
    bands = max(1, min(bands, tiles))
    cuts = [(i * tiles // bands) * tile_m for i in range(bands)] + [rows]
    return [(cuts[i], cuts[i + 1]) for i in range(bands) if cuts[i + 1] > cuts[i]]

"""Launch, check and time one GEMM kernel -- the reference's harness contract
(backend/node/run_tma.py:47-230) over this library's C ABI.

    python -m warpc_public_release_b200.gemm gemm 2048 2048 2048 > k.hdr
    python -m warpc_public_release_b200.run_tma k.hdr [repeat]          # the header names shape and program
    python -m warpc_public_release_b200.run_tma M N K [repeat]          # or: the rule's program for a shape

Like the reference: inputs from `np.random.default_rng(1)`, A drawn first, integers in [-3, 3]
(WARPC_INPUTS=hash: the index hash; WARPC_INPUTS=uniform: uniform[-1, 1], checked within
1e-3 sqrt(K)); the first launch is waited for and checked against numpy's fp32 matmul, "first
launch done, N wrong" goes to stderr, then `repeat` launches run back to back between two CUDA
events and the last line reads

    NAME MxNxK grid=(G, 1)  MATCH|MISMATCH bad=x/y  ms  TFLOP/s

WARPC_PDL=1 lets each timed launch begin while the one before it runs (the reference's AB_PDL,
backend/node/ab.py:95-118).  WARPC_NO_CHECK=1 skips the check (prints UNCHECKED), WARPC_VERIFY_LAST=1 also checks what the
last timed launch left, WARPC_STAMPS=1 prints the phase stamps of one more launch.  For a mismatch
(run_tma.py:144-168): WARPC_DUMP=file.npy saves C and the reference stacked, WARPC_TILES=1 prints which
output tiles are wrong and which of those were never written, WARPC_DIAG=1 where in a tile the wrong
entries sit.  WARPC_L2PROMO=0..3 is read by the library when it encodes the tensor maps (run_tma.py:42).  Returns
True when the check passed.  The numpy product is the harness's checker, exactly as in the
reference; the kernel never runs on the CPU.
"""
import os
import sys

import numpy as np

from . import launch_header, programs
from .plan import Plan

STAMP_NAMES = ["entry", "barriers initialised, cluster met", "producer: first stage issued", "producer: last stage issued",
               "MMA: first stage landed", "MMA: last stage issued", "epilogue: accumulator ready", "epilogue: tile's stores issued",
               "roles done", "exit", "MMA: accumulator free"]
FINE_STAMP_NAMES = ["set-up: barriers initialised", "set-up: tensor memory allocated", "set-up: first tile found",
                    "teardown: last stores read", "teardown: CTAs met", "teardown: tensor memory freed", "set-up: CTAs met"]


def make_inputs(m, n, k, seed=1):
    kind = os.environ.get("WARPC_INPUTS", "integers")
    rng = np.random.default_rng(seed)
    if kind == "hash":
        def val(count, salt):
            i = np.arange(count, dtype=np.uint64)
            return ((((i * np.uint64(2654435761)) + np.uint64(salt)) >> np.uint64(13)) % np.uint64(7)).astype(np.int64) - 3
        return val(m * k, 1).reshape(m, k).astype(np.float16), val(n * k, 7).reshape(n, k).astype(np.float16), 1e-3
    if kind == "uniform":
        a = rng.uniform(-1.0, 1.0, size=(m, k)).astype(np.float16)
        return a, rng.uniform(-1.0, 1.0, size=(n, k)).astype(np.float16), 1e-3 * k ** 0.5
    a = rng.integers(-3, 4, size=(m, k)).astype(np.float16)
    return a, rng.integers(-3, 4, size=(n, k)).astype(np.float16), 1e-3


def variant_from_header(text, m, n, k):
    """The exact program a header text names, rebuilt from its `# variant key=value ...` line (every
    rule field: tile, depth, cluster launch control, split-K, stream-K, serpentine, accumulators ...).
    Fails loudly when the line is missing or when the header derived from the rebuilt program is not
    the text given: a header is never run as some other program under the same kernel name."""
    f = launch_header.variant_fields(text)
    if f is None:
        raise RuntimeError("the header has no '# variant' line: it was not written by this library's gemm command")
    if f["prog"] == programs._lib.PROG_ONE:
        v = programs.one(m, n, k, f["depth"])
    elif f["prog"] == programs._lib.PROG_PAIR:
        v = programs.pair(m, n, k, f["depth"])
    elif f["retile"]:
        v = programs.choose(m, n, k)  # the rule's own program: only wg_choose marks a variant for re-tiling
    else:
        v = programs.swapped(m, n, k, f["tile_m"], f["tile_n"], f["depth"], clc=f["clc"], ask_ahead=f["ask_ahead"], direct=f["direct"],
                             serpentine=f["serpentine"], cluster_n=f["cluster_n"], bufs=f["bufs"], group=f["group"], streamk=f["streamk"],
                             split=f["split"], split_grid=f["split_grid"], split_add=f["split_add"], late_launch=f["late_launch"])
    again = programs.header(v, m, n, k)
    if again != text:
        raise RuntimeError("the header does not describe a program of this library for %dx%dx%d (re-derived header differs)" % (m, n, k))
    return v


def describe_mismatch(c, ref, bad, tol, li, out):
    """Where a wrong result is wrong, in this kernel's own geometry: CTA tiles of tile_m x tile_n; inside a tile an
    epilogue warp owns 32 columns (a lane a column) and handles them in blocks of 32 rows."""
    import collections
    m, n = c.shape
    tm, tn = li.tile_m, li.tile_n
    if os.environ.get("WARPC_TILES") and m % tm == 0 and n % tn == 0:
        wrong = ~(np.abs(c - ref) <= tol)
        per_tile = wrong.reshape(m // tm, tm, n // tn, tn).any(axis=(1, 3))
        untouched = (c == 0).reshape(m // tm, tm, n // tn, tn).all(axis=(1, 3))
        print("   wrong tiles %d of %d, of them all-zero (never written) %d" % (int(per_tile.sum()), per_tile.size, int((per_tile & untouched).sum())), file=out)
        for i in range(min(per_tile.shape[0], 16)):
            print("   " + "".join("x" if x else "." for x in per_tile[i, :128]), file=out)
    if os.environ.get("WARPC_DIAG"):
        rows, cols = bad[:, 0], bad[:, 1]
        count = lambda xs: sorted(collections.Counter(int(x) for x in xs).items())
        print("   zero where wrong: %d of %d" % (int(np.sum(c[rows, cols] == 0.0)), len(bad)), file=out)
        print("   tiles (row, column) most hit: %s" % collections.Counter(zip((rows // tm).tolist(), (cols // tn).tolist())).most_common(5), file=out)
        print("   32-row block in the tile: %s" % count((rows % tm) // 32), file=out)
        print("   epilogue warp (32-column group in the tile): %s" % count((cols % tn) // 32), file=out)
        print("   lane (column in the group), first ten: %s" % count(cols % 32)[:10], file=out)
        print("   row in the block, first ten: %s" % count(rows % 32)[:10], file=out)
        live = bad[c[rows, cols] != 0.0]
        if len(live):
            i, j = live[0]
            same = np.argwhere(np.abs(ref - c[i, j]) <= tol)[:4].tolist()
            print("   (%d,%d) holds %s; the reference has that value at %s" % (i, j, c[i, j], same), file=out)


def run(variant, m, n, k, repeat=20, seed=1, name=None, out=sys.stdout):
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("run_tma: no CUDA device (this library has no CPU path)")
    hdr = launch_header.parse_header(programs.header(variant, m, n, k))
    name = name or hdr["kernel"]
    if launch_header.shape_of(hdr) != (m, n, k):
        raise RuntimeError("%s: the kernel was built for %dx%dx%d, the run is %dx%dx%d" % ((name,) + launch_header.shape_of(hdr) + (m, n, k)))
    a, bt, tol = make_inputs(m, n, k, seed)
    ref = None if os.environ.get("WARPC_NO_CHECK") else a.astype(np.float32) @ bt.astype(np.float32).T
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(bt).cuda()
    dc = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    plan = Plan(variant, m, n, k, da.data_ptr(), db.data_ptr(), dc.data_ptr())
    grid = tuple(int(x) for x in hdr["grid"].split())
    plan.launch()
    plan.status()
    if os.environ.get("WARPC_PDL") == "1":
        plan.set_dependent_launch(True)
    if ref is None:
        ms = plan.time_launches(repeat, warmup=0)
        print("%-28s %dx%dx%d grid=%s  UNCHECKED  %.4f ms" % (name, m, n, k, grid, ms), file=out)
        return True
    c = dc.cpu().numpy()
    bad = np.argwhere(~(np.abs(c - ref) <= tol))
    if os.environ.get("WARPC_DUMP"):
        np.save(os.environ["WARPC_DUMP"], np.stack([c, ref]))
    print("first launch done, %d wrong" % len(bad), file=sys.stderr, flush=True)
    if len(bad) and (os.environ.get("WARPC_TILES") or os.environ.get("WARPC_DIAG")):
        describe_mismatch(c, ref, bad, tol, programs.realise(variant, m, n, k), out)
    ms = plan.time_launches(repeat, warmup=0)
    plan.status()
    if os.environ.get("WARPC_STAMPS"):
        plan.enable_stamps(True)
        plan.launch()
        st = plan.read_stamps().astype(np.int64)
        plan.enable_stamps(False)
        t0 = st[:, 0, 0][st[:, 0, 0] > 0].min()
        print("  %d CTAs ran; ns from the first CTA's entry: count:min/median/max per tile" % int((st[:, 0, 0] > 0).sum()), file=out)
        for ev, label in list(enumerate(STAMP_NAMES)) + list(zip(list(range(16, 22)) + [23], FINE_STAMP_NAMES)):
            cells = []
            for t in range(4):
                col = st[:, ev, t]
                col = col[col > 0] - t0
                cells.append("%5d:%7d/%7d/%7d" % (len(col), col.min(), np.median(col), col.max()) if len(col) else " " * 29)
            print("  %2d %-34s %s" % (ev, label, "  ".join(cells)), file=out)
        ran = st[:, 15, 0] > 0
        if ran.any():  # event 15: SM cycles from entry to exit, against the same interval on the GPU-wide timer
            mhz = 1e3 * st[ran, 15, 0] / np.maximum(st[ran, 9, 0] - st[ran, 0, 0], 1)
            print("  SM clock over the launch: %.0f MHz (median of CTAs)" % np.median(mhz), file=out)
        # events 11-14: SM cycles the first epilogue warp spent in each part of a tile's store
        for ev, label in zip((11, 12, 13, 14, 22), ("waiting for tcgen05.ld", "waiting for a staging copy", "st.shared + fence", "issuing the TMA store", "issuing tcgen05.ld / release")):
            cells = ["%5d:%7d/%7d/%7d" % (len(c), c.min(), np.median(c), c.max()) if len(c) else " " * 29
                     for c in (st[:, ev, t][st[:, ev, t] > 0] for t in range(4))]
            print("  %2d %-34s %s" % (ev, "epilogue cycles: " + label, "  ".join(cells)), file=out)
    if os.environ.get("WARPC_VERIFY_LAST"):
        c2 = dc.cpu().numpy()
        print("  last launch: %d wrong" % int(np.count_nonzero(~(np.abs(c2 - ref) <= tol))), file=out)
    flops = 2.0 * m * n * k
    print("%-28s %dx%dx%d grid=%s  %s bad=%d/%d  %.4f ms  %.1f TFLOP/s" % (
        name, m, n, k, grid, "MATCH" if len(bad) == 0 else "MISMATCH", len(bad), m * n, ms, flops / ms / 1e9), file=out)
    if len(bad):
        i, j = bad[0]
        print("   first bad (%d,%d): got %s ref %s" % (i, j, c[i, j], ref[i, j]), file=out)
    plan.close()
    return len(bad) == 0


def main(argv=None):
    args = list(sys.argv[1:] if argv is None else argv)
    if not args:
        print(__doc__, file=sys.stderr)
        return 2
    if os.path.exists(args[0]):
        text = open(args[0]).read()
        m, n, k = launch_header.shape_of(launch_header.parse_header(text))
        variant, rest = variant_from_header(text, m, n, k), args[1:]
    else:
        m, n, k = map(int, args[:3])
        variant, rest = programs.choose(m, n, k), args[3:]
    ok = run(variant, m, n, k, repeat=int(rest[0]) if rest else 30)
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())

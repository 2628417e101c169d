"""A/B GPU time per call: this library's kernel against cuBLASLt, in one process on one warm GPU.

The method is the reference's (README.md:504-525; backend/node/ab.py:63-93, ktrace.cpp): each
call runs alone (a synchronise after every launch), its GPU time is the kernel's start-to-end
from CUPTI activity records, a side's figure is the median over its last N calls, the sides run
interleaved ours, cuBLASLt, cuBLASLt, ours, twice, and the inputs are the index-hash integers in
[-3, 3] (or uniform[-1, 1] with --inputs uniform) so both sides multiply the same values.
cuBLASLt is timed on the fastest algorithm of its heuristic's list whose result is exact.
Before each side's turn the GPU is kept busy for a few tens of milliseconds so the clocks are
the loaded ones, not the idle ones.

    python -m warpc_public_release_b200.ab [--inputs hash|uniform] [--json out.json] [M N K ...]

--event-rounds R is the reference harness's other method (backend/node/ab.py:121-175): R rounds, the
order of the sides alternating, each side's turn --repeat launches back to back between two CUDA
events.  With it: --gap S idles S seconds before each turn (short runs after a gap stay under the
power cap, at the full clock: AB_GAP); --block queues each turn behind a long kernel on buffers of
its own, launched and not waited for, so the timed launches are all queued before the first of them
runs, whatever launching from Python costs (AB_BLOCK); --warm MS runs the side's own kernel for
about MS milliseconds right before its timed launches, not waited for (AB_WARM); --each prints
every turn as it is taken with the SM clock, the clock's limiting reasons and the energy the device
used per call, from NVML's counters, read-only (AB_EACH); --pdl lets each of this library's launches
begin while the one before it runs (AB_PDL).
"""
import argparse
import ctypes
import json
import os
import sys

from . import _lib, programs
from .clocks import ClockSampler
from .plan import Plan

HERE = os.path.dirname(os.path.abspath(__file__))
SHAPES = [(1024, 1024, 1024), (1536, 1536, 1536), (2048, 2048, 2048), (3072, 1280, 2048), (4096, 4096, 1024),
          (4096, 4096, 4096), (8192, 2048, 4096), (8192, 8192, 8192), (16384, 16384, 16384), (2048, 2048, 16384),
          (1024, 1024, 65536)]
# calls whose median is taken, by how long one call is (README.md:508-511)
LAST = {(4096, 4096, 1024): 300, (4096, 4096, 4096): 200, (8192, 2048, 4096): 200, (2048, 2048, 16384): 200,
        (1024, 1024, 65536): 200, (8192, 8192, 8192): 40, (16384, 16384, 16384): 12}
# what the reference publishes for its own kernels and for cuBLASLt 13.8 on its B200 (README.md:81-91), us
PUBLISHED = {(1024, 1024, 1024): (4.655, 5.41), (1536, 1536, 1536): (7.87, 7.84), (2048, 2048, 2048): (14.46, 13.79),
             (3072, 1280, 2048): (14.08, 13.57), (4096, 4096, 1024): (26.11, 26.85), (4096, 4096, 4096): (75.875, 75.55),
             (8192, 2048, 4096): (75.905, 75.87), (8192, 8192, 8192): (553.7, 557.6), (16384, 16384, 16384): (4186.1, 4159.7),
             (2048, 2048, 16384): (74.015, 78.43), (1024, 1024, 65536): (77.075, 84.96)}


class KernelTimer:
    def __init__(self):
        self.l = ctypes.CDLL(os.path.join(HERE, "libwarpc_b200_ktimer.so"))
        self.l.wk_median.argtypes = [ctypes.c_char_p, ctypes.c_int] + [ctypes.POINTER(ctypes.c_double)] * 3
        if self.l.wk_begin() != 0:
            raise RuntimeError("CUPTI activity recording is not available")

    def clear(self):
        self.l.wk_flush()
        self.l.wk_clear()

    def median(self, substr, last):
        self.l.wk_flush()
        med, lo, hi = ctypes.c_double(), ctypes.c_double(), ctypes.c_double()
        n = self.l.wk_median(substr.encode(), last, ctypes.byref(med), ctypes.byref(lo), ctypes.byref(hi))
        return (med.value, n) if n else (float("nan"), 0)

    def names(self):
        self.l.wk_flush()
        self.l.wk_get.argtypes = [ctypes.c_int, ctypes.c_char_p, ctypes.c_size_t, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double)]
        out = {}
        buf = ctypes.create_string_buffer(256)
        for i in range(self.l.wk_count()):
            self.l.wk_get(i, buf, 256, None, None)
            out[buf.value.decode()] = out.get(buf.value.decode(), 0) + 1
        return out

    def close(self):
        self.l.wk_end()


class CublasLt:
    def __init__(self, m, n, k, dA, dBt, dC, workspace=256 << 20):
        self.l = ctypes.CDLL(os.path.join(HERE, "libwarpc_b200_cublaslt.so"))
        self.l.wc_create.argtypes = [ctypes.c_int] * 3 + [ctypes.c_void_p] * 3 + [ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p),
                                                                                 ctypes.POINTER(ctypes.c_int)]
        self.l.wc_run.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
        self.l.wc_destroy.argtypes = [ctypes.c_void_p]
        self.h, n_algos = ctypes.c_void_p(), ctypes.c_int()
        r = self.l.wc_create(m, n, k, dA, dBt, dC, workspace, ctypes.byref(self.h), ctypes.byref(n_algos))
        if r != 0:
            raise RuntimeError("cuBLASLt set-up failed: %d" % r)
        self.n_algos = n_algos.value
        self.version = self.l.wc_version()

    def run(self, algo):
        r = self.l.wc_run(self.h, algo, None)
        if r != 0:
            raise RuntimeError("cublasLtMatmul: %d" % r)

    def close(self):
        self.l.wc_destroy(self.h)


def make_inputs(torch, kind, m, n, k):
    """The reference's index-hash inputs (run_tma.py:58-62) or uniform[-1,1], built on the device."""
    if kind == "hash":
        def val(count, salt):
            i = torch.arange(count, dtype=torch.int64, device="cuda")
            return ((((i * 2654435761 + salt) >> 13) % 7) - 3).to(torch.float16)
        return val(m * k, 1).reshape(m, k), val(n * k, 7).reshape(n, k)
    gen = torch.Generator(device="cuda").manual_seed(1)
    a = (torch.rand((m, k), generator=gen, device="cuda") * 2 - 1).to(torch.float16)
    bt = (torch.rand((n, k), generator=gen, device="cuda") * 2 - 1).to(torch.float16)
    return a, bt


def max_abs_diff(torch, x, y):
    """max |x - y| in row blocks (no temporary the size of the matrices)."""
    worst, step = 0.0, max(1, (64 << 20) // max(1, x.shape[1]))
    for r0 in range(0, x.shape[0], step):
        worst = max(worst, float((x[r0:r0 + step] - y[r0:r0 + step]).abs().max().item()))
    return worst


def fastest_correct_algo(torch, lt, c_lib, c_ours, tol, work):
    """The fastest cuBLASLt algorithm of the heuristic's list whose C agrees with `c_ours` within `tol`
    (backend/node/cublas_q7.cpp:61-63, 84-127), by a quick event timing of each candidate.  Returns (index, how many were correct)."""
    best, best_ms, correct = -1, None, 0
    for algo in range(lt.n_algos):
        c_lib.zero_()
        try:
            lt.run(algo)
        except RuntimeError:
            continue
        torch.cuda.synchronize()
        if max_abs_diff(torch, c_lib, c_ours) > tol:
            continue
        correct += 1
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 20 if work < 2 ** 36 else (5 if work < 2 ** 40 else 2)
        for _ in range(min(3, reps)):
            lt.run(algo)
        e0.record()
        for _ in range(reps):
            lt.run(algo)
        e1.record(); torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        if best_ms is None or ms < best_ms:
            best, best_ms = algo, ms
    if best < 0:
        raise RuntimeError("no correct cuBLASLt algorithm")
    return best, correct


def ab_shape(torch, timer, m, n, k, inputs="hash", rounds=2, variant=None, busy_ms=30.0, series=0, alternate=False):
    """One shape, both sides.  `alternate`: instead of the published order (a block of calls a side: ours, library,
    library, ours) the sides take turns call by call, each call still alone.  Long calls run the chip into its power cap
    and the clock drifts over a block of them (seconds), so a side's block is measured at another clock than the other's;
    taking turns gives both the same clock.  For short calls the published order is the fair one: a call that follows the
    other side's finds the other side's C in the L2 instead of its own operands."""
    a, bt = make_inputs(torch, inputs, m, n, k)
    c_ours = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    c_lib = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    v = variant or programs.choose(m, n, k)
    plan = Plan(v, m, n, k, a.data_ptr(), bt.data_ptr(), c_ours.data_ptr())
    lt = CublasLt(m, n, k, a.data_ptr(), bt.data_ptr(), c_lib.data_ptr())
    plan.launch()
    plan.status()
    exact = inputs == "hash"
    tol = 0.0 if exact else 1e-3 * (k ** 0.5)
    last = LAST.get((m, n, k), 400)
    calls = last + max(5, last // 10)

    def busy(run):
        # keep the GPU loaded with the side's own kernel for about busy_ms before its isolated calls
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); run(); e1.record(); torch.cuda.synchronize()
        one = max(e0.elapsed_time(e1), 1e-3)
        for _ in range(int(min(max(busy_ms / one, 3), 3000))):
            run()
        torch.cuda.synchronize()

    best, correct = fastest_correct_algo(torch, lt, c_lib, c_ours, tol, m * n * k)

    def by_events(run):
        # without CUPTI: each call alone between two events (includes the launch's latency on the stream), median of the last N
        ts = []
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(calls):
            e0.record(); run(); e1.record(); torch.cuda.synchronize()
            ts.append(1e3 * e0.elapsed_time(e1))
        ts = sorted(ts[-last:])
        return ts[len(ts) // 2]

    def isolated(run, tag):
        busy(run)
        if timer is None:
            return by_events(run), last
        timer.clear()
        for _ in range(calls):
            run()
            torch.cuda.synchronize()
        return timer.median(tag, last)

    ours, lib, lib_kernels = [], [], None
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    sampler.timed = True
    if alternate:
        for _ in range(rounds):
            busy(plan.launch)
            busy(lambda: lt.run(best))
            mine, theirs = [], []
            for _ in range(calls):
                for side in ("ours", "lib"):
                    if timer is not None:
                        timer.clear()
                    if timer is None:
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        e0.record()
                    (plan.launch() if side == "ours" else lt.run(best))
                    if timer is None:
                        e1.record()
                    torch.cuda.synchronize()
                    if timer is None:
                        t = 1e3 * e0.elapsed_time(e1)
                    else:
                        names = timer.names()
                        if side == "lib":
                            lib_kernels = list(names)
                        t = sum(timer.median(nm, 1)[0] for nm in names)
                    (mine if side == "ours" else theirs).append(t)
            med = lambda xs: sorted(xs[-last:])[len(xs[-last:]) // 2]
            ours.append(med(mine))
            lib.append(med(theirs))
    for _ in range(0 if alternate else rounds):
        for side in ("ours", "lib", "lib", "ours"):
            if side == "ours":
                ours.append(isolated(plan.launch, "gemm_kernel")[0])
            else:
                # a cuBLASLt call may be more than one kernel: its GPU time is the sum of its kernels' medians
                busy(lambda: lt.run(best))
                if timer is None:
                    lib.append(by_events(lambda: lt.run(best)))
                    continue
                timer.clear()
                for _ in range(calls):
                    lt.run(best)
                    torch.cuda.synchronize()
                names = [nm for nm in timer.names() if "gemm_kernel" not in nm]
                lib_kernels = names
                lib.append(sum(timer.median(nm, last)[0] for nm in names))
    plan.status()
    sampler.timed = False
    clocks = sampler.stop()
    err = max_abs_diff(torch, c_lib, c_ours)
    steady = None
    if series > 0:
        # the reference's other timing (backend/node/clusterlaunch.py:54-96, ab.py AB_SERIES / AB_PDL): mean of `series`
        # launches back to back between two events, warmed by launches of the same kind; ours also with dependent launch
        def back_to_back(run):
            for _ in range(max(3, series // 4)):
                run()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(series):
                run()
            e1.record()
            torch.cuda.synchronize()
            return 1e3 * e0.elapsed_time(e1) / series
        steady = {"launches": series, "ours_us": back_to_back(plan.launch), "cublaslt_us": back_to_back(lambda: lt.run(best))}
        plan.set_dependent_launch(True)
        steady["ours_dependent_launch_us"] = back_to_back(plan.launch)
        plan.set_dependent_launch(False)
        plan.status()
    flops = 2.0 * m * n * k
    mid = lambda xs: (min(xs) + max(xs)) / 2
    li = programs.realise(v, m, n, k)
    sched = ("one tile a CTA", "fixed grid", "launch control", "split-K", "stream-K")[li.sched]
    if li.sched == 4 and li.sk_dp:
        sched = "fixed grid for %d pair tiles, stream-K for the rest" % li.sk_dp
    row = {"shape": [m, n, k], "inputs": inputs, "program": "%dx%d d%d" % (v.tile_m, v.tile_n, v.depth),
           "runs_as": "%dx%d d%d %s" % (li.tile_m, li.tile_n, li.depth, sched), "calls_in_median": last,
           "ours_us": [min(ours), max(ours)], "cublaslt_us": [min(lib), max(lib)], "cublaslt_algo": best,
           "cublaslt_correct_algos": "%d of %d" % (correct, lt.n_algos), "cublaslt_version": lt.version,
           "cublaslt_kernels": lib_kernels, "ours_tflops": flops / mid(ours) / 1e6, "cublaslt_tflops": flops / mid(lib) / 1e6,
           "ours_vs_cublaslt_pct": 100.0 * (min(lib) / mid(ours) - 1.0),
           # the same comparison without the published formula's lean to the library (its fastest run against our midpoint): mean of runs against mean of runs
           "ours_vs_cublaslt_mean_pct": 100.0 * ((sum(lib) / len(lib)) / (sum(ours) / len(ours)) - 1.0), "max_abs_diff_vs_cublaslt": err,
           "timer": "CUPTI kernel start-to-end" if timer is not None else "CUDA events around each call",
           "order": "the sides take turns call by call" if alternate else "a block of calls a side: ours, library, library, ours",
           "published_warpc_us": PUBLISHED.get((m, n, k), (None, None))[0], "published_cublas138_us": PUBLISHED.get((m, n, k), (None, None))[1]}
    row["clocks"] = clocks  # over both sides' isolated calls: SM MHz (median), power (max), throttle reasons seen
    if steady is not None:
        row["back_to_back"] = steady
    plan.close()
    lt.close()
    return row


class Nvml:
    """SM clock, limiting reasons and the energy counter of one GPU (read-only); every method gives None without NVML."""

    def __init__(self, index):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv, self.h = pynvml, pynvml.nvmlDeviceGetHandleByIndex(index)
        except Exception:
            self.nv = self.h = None

    def energy_mj(self):
        try:
            return self.nv.nvmlDeviceGetTotalEnergyConsumption(self.h)
        except Exception:
            return None

    def clock(self):
        try:
            try:
                why = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
            except Exception:
                why = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
            return self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM), why
        except Exception:
            return None


def turn_time(torch, run, repeat, warm=0, blocker=None):
    """One side's turn of the event-rounds method: (optional) blocker and warming launches queued and not waited for,
    then `repeat` launches between two events; mean microseconds a launch."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if blocker is not None:
        blocker()
    for _ in range(warm):
        run()
    e0.record()
    for _ in range(repeat):
        run()
    e1.record()
    torch.cuda.synchronize()
    return 1e3 * e0.elapsed_time(e1) / repeat


def event_rounds(torch, m, n, k, rounds, repeat, inputs="hash", gap=0.0, block=False, warm_ms=0.0, each=False, pdl=False, out=sys.stdout):
    """The reference harness's event-timed rounds (backend/node/ab.py:121-175) for this library's kernel and cuBLASLt
    (its fastest correct algorithm) on one shape.  Returns a dict with each side's per-round microseconds."""
    import statistics
    import time
    a, bt = make_inputs(torch, inputs, m, n, k)
    c_ours = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    c_lib = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    v = programs.choose(m, n, k)
    plan = Plan(v, m, n, k, a.data_ptr(), bt.data_ptr(), c_ours.data_ptr())
    plan.launch()
    plan.status()
    lt = CublasLt(m, n, k, a.data_ptr(), bt.data_ptr(), c_lib.data_ptr())
    best = fastest_correct_algo(torch, lt, c_lib, c_ours, 0.0 if inputs == "hash" else 1e-3 * (k ** 0.5), m * n * k)[0]
    if pdl:
        plan.set_dependent_launch(True)
    sides = [("ours", plan.launch), ("cublaslt", lambda: lt.run(best))]
    blocker = None
    if block:
        # a long kernel of this library on buffers of its own: about a millisecond for the host to queue behind
        bm = 8192
        ba = torch.zeros((bm, bm), dtype=torch.float16, device="cuda")
        bc = torch.zeros((bm, bm), dtype=torch.float32, device="cuda")
        bplan = Plan(programs.choose(bm, bm, bm), bm, bm, bm, ba.data_ptr(), ba.data_ptr(), bc.data_ptr())
        blocker = bplan.launch
    nvml = Nvml(torch.cuda.current_device())
    once = {name: turn_time(torch, run, 3) for name, run in sides}
    res = {name: [] for name, _ in sides}
    for r in range(rounds):
        for name, run in (sides if r % 2 == 0 else sides[::-1]):
            if gap:
                time.sleep(gap)
            warm = max(1, int(1e3 * warm_ms / once[name])) if warm_ms else 0
            e0 = nvml.energy_mj() if each else None
            res[name].append(turn_time(torch, run, repeat, warm=warm, blocker=blocker))
            if each:
                e1, c = nvml.energy_mj(), nvml.clock()
                print("round %d %-9s %.2f us%s%s" % (r, name, res[name][-1], "" if c is None else "  clock %d MHz, reasons 0x%x" % c,
                      "" if e0 is None or e1 is None else "  energy %.1f mJ a call (the turn's blocker and warming launches included)" % ((e1 - e0) / (repeat + warm))),
                      file=out, flush=True)
    plan.status()
    for name, _ in sides:
        x = res[name]
        print("%-10s %dx%dx%d  median %.2f us  min %.2f  max %.2f  (%d x %d)" % (name, m, n, k, statistics.median(x), min(x), max(x), rounds, repeat), file=out)
    plan.close()
    lt.close()
    if block:
        bplan.close()
    return {"shape": [m, n, k], "rounds": rounds, "repeat": repeat, "gap_s": gap, "blocked": bool(block), "warm_ms": warm_ms, "pdl": bool(pdl),
            "ours_us": res["ours"], "cublaslt_us": res["cublaslt"]}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--inputs", default="hash", choices=["hash", "uniform"])
    ap.add_argument("--json", default=None)
    ap.add_argument("--rounds", type=int, default=2)
    ap.add_argument("--series", type=int, default=0, help="also time this many launches back to back between events (ours, ours with dependent launch, cuBLASLt)")
    ap.add_argument("--alternate", action="store_true", help="isolated calls, the sides taking turns call by call instead of in blocks (long calls under the power cap)")
    ap.add_argument("--event-rounds", type=int, default=0, help="the reference harness's event-timed rounds instead of isolated calls")
    ap.add_argument("--repeat", type=int, default=30, help="launches back to back per turn of an event round")
    ap.add_argument("--gap", type=float, default=0.0, help="seconds idle before each turn (event rounds)")
    ap.add_argument("--block", action="store_true", help="queue each turn behind a long kernel (event rounds)")
    ap.add_argument("--warm", type=float, default=0.0, help="milliseconds of the side's own kernel right before its timed launches (event rounds)")
    ap.add_argument("--each", action="store_true", help="print every turn with SM clock, limiting reasons and energy per call (event rounds)")
    ap.add_argument("--pdl", action="store_true", help="dependent launches for this library's side (event rounds)")
    ap.add_argument("dims", nargs="*", type=int)
    args = ap.parse_args(argv)
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("ab: needs a CUDA device")
    shapes = [tuple(args.dims[i:i + 3]) for i in range(0, len(args.dims), 3)] or list(SHAPES)
    if args.event_rounds:
        rows = [event_rounds(torch, m, n, k, args.event_rounds, args.repeat, inputs=args.inputs, gap=args.gap, block=args.block, warm_ms=args.warm,
                             each=args.each, pdl=args.pdl) for (m, n, k) in shapes]
        if args.json:
            json.dump({"method": "event-timed rounds, order alternating, %d launches back to back a turn" % args.repeat, "rows": rows}, open(args.json, "w"), indent=1)
        return 0
    timer = KernelTimer()
    rows = []
    print("%-18s %-12s %-28s %17s %17s %8s   %s" % ("M x N x K", "rule's program", "runs as", "ours us", "cuBLASLt us", "vs lib", "published warpc / cuBLAS 13.8 us"))
    for (m, n, k) in shapes:
        row = ab_shape(torch, timer, m, n, k, inputs=args.inputs, rounds=args.rounds, series=args.series, alternate=args.alternate)
        rows.append(row)
        print("%-18s %-12s %-28s %8.2f-%-8.2f %8.2f-%-8.2f %+7.1f%%   %s / %s" % (
            "%dx%dx%d" % (m, n, k), row["program"], row["runs_as"], *row["ours_us"], *row["cublaslt_us"], row["ours_vs_cublaslt_pct"],
            row["published_warpc_us"], row["published_cublas138_us"]), flush=True)
        if "back_to_back" in row:
            b = row["back_to_back"]
            print("%-18s back to back x%d: ours %.2f us, ours with dependent launch %.2f us, cuBLASLt %.2f us" % (
                "", b["launches"], b["ours_us"], b["ours_dependent_launch_us"], b["cublaslt_us"]), flush=True)
        if args.json:
            json.dump({"method": "CUPTI kernel start-to-end, each call alone, median of the last N, ours/lib/lib/ours x %d" % args.rounds,
                       "rows": rows}, open(args.json, "w"), indent=1)
    timer.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())

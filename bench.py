"""bench.py -- fp16-in / fp32-out GEMM (C = A . Bt^T) on B200: TFLOP/s and us/call.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--shapes]

Workload (config.workload): 16384 x 16384 x 16384, uniform[-1,1] fp16 inputs from a seeded
generator, fp32 C -- the one configuration that shards: at N GPUs rank r owns M/N contiguous
rows of A and C, Bt is replicated, and the GEMM exchanges nothing ("strong" scaling, total work
fixed).  A step is one call of the hot path (one kernel launch per rank).  `value` is whole-job
TFLOP/s with inputs resident in HBM, timed with CUDA events on the launching stream, max over
ranks; `e2e` is the same metric through the host-buffer C-ABI call (pinned host A, Bt in,
C out, every step; at N > 1 every rank uploads only its own rows of A and of Bt, and the Bt
shards are gathered over NVLink).  cuBLASLt (fastest correct algorithm of its heuristic's list)
runs on the same buffers in the same process, interleaved with ours: `cublaslt` in the line.  At
N = 1 the line also carries `shapes`: all eleven benchmark shapes, this library and cuBLASLt,
each call alone, GPU time from CUPTI, median of the last N calls (the reference's published
method, README.md:504-525), plus the mean of back-to-back launches.

--impl reference times the reference's own CPU path for the same config -- numpy's fp32 matmul
of the fp16 operands (backend/node/run_tma.py:67) -- on the host cores, on a bounded sample.
"""
import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = (16384, 16384, 16384)
SWEEP = [(1536, 1536, 1536), (2048, 2048, 2048), (3072, 1280, 2048), (4096, 4096, 1024), (4096, 4096, 4096)]
OTHERS = [(1024, 1024, 1024), (8192, 2048, 4096), (8192, 8192, 8192), (2048, 2048, 16384), (1024, 1024, 65536)]
NOMINAL_TFLOPS = 2250.0
METRIC = "TFLOP/s fp16->fp32 GEMM C=A.Bt^T (us/call in ms_per_step)"
WORKLOAD_NAME = "%dx%dx%d fp16 GEMM C=A.Bt^T, uniform[-1,1] fp16 inputs (seeded), fp32 C" % WORKLOAD


def measured_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))), "measured"
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


from warpc_public_release_b200.clocks import ClockSampler  # noqa: E402


_CPU_INPUTS = {}


def cpu_inputs(n, k, rows):
    """The CPU sample's operands, drawn once: `rows` rows of A and all of Bt, uniform[-1,1] fp16 from a seed."""
    import numpy as np
    if (n, k, rows) not in _CPU_INPUTS:
        rng = np.random.default_rng(1)
        _CPU_INPUTS[(n, k, rows)] = (rng.uniform(-1.0, 1.0, size=(rows, k)).astype(np.float16), rng.uniform(-1.0, 1.0, size=(n, k)).astype(np.float16))
    return _CPU_INPUTS[(n, k, rows)]


def cpu_numpy_sample(m, n, k, rows, repeats=1):
    """The reference's CPU path (numpy fp32 matmul of the fp16 operands, run_tma.py:67) on a
    row slab of the workload: `rows` rows of A against all of Bt.  Returns (seconds, threads)."""
    from oracle import gemm_ref
    a, bt = cpu_inputs(n, k, rows)
    # every host core the process may use, whatever OMP_NUM_THREADS says (torchrun sets it to 1 for its ranks)
    want = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    try:
        from threadpoolctl import threadpool_info, threadpool_limits
        limit = threadpool_limits(limits=want, user_api="blas")
    except Exception:
        threadpool_info, limit = None, None
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        c = gemm_ref.gemm_ref(a, bt)  # the conversion to fp32 is part of the reference's expression: timed
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    del c
    threads = want
    if threadpool_info is not None:
        blas = [p for p in threadpool_info() if p.get("user_api") == "blas"]
        if blas:
            threads = max(p.get("num_threads", 1) for p in blas)
    if limit is not None:
        limit.restore_original_limits()
    return best, threads


def reference_arm(args, rank):
    """bench.py --impl reference: rank 0 alone times numpy on the host cores."""
    if rank != 0:
        return 0
    m, n, k = WORKLOAD
    rows = 256  # a 256-row slab of A per step: 2*256*16384*16384 = 0.137 TFLOP, about a second of CPU work
    warmup, steps = max(0, min(args.warmup, 20)), max(1, min(args.steps, 100))   # exactly W and K (bounded: the run stays within minutes)
    for _ in range(warmup):
        cpu_numpy_sample(m, n, k, rows)
    times = []
    threads = 1
    for _ in range(steps):
        dt, threads = cpu_numpy_sample(m, n, k, rows)
        times.append(dt)
    sec = sum(times) / len(times)
    tflops = 2.0 * rows * n * k / sec / 1e12
    sample = "rows 0..%d of A (M' = %d of %d) against all of Bt, numpy fp32 matmul incl. fp16->fp32 conversion, mean of %d" % (
        rows, rows, m, len(times))
    line = {"impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": sec * 1e3, "ms_per_full_call_extrapolated": sec * 1e3 * (m / rows),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16->f32", "data": "synthetic",
            "config": {"workload": WORKLOAD_NAME},
            "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)
    return 0


def shapes_table(torch, shapes):
    """Every benchmark shape on uniform[-1,1] inputs: this library's kernel and cuBLASLt, each call alone, GPU time
    kernel start-to-end from CUPTI, median of the last N calls, ours / cuBLASLt / cuBLASLt / ours (README.md:504-525);
    and the mean of 50 launches back to back between two events (backend/node/run_tma.py:171-175)."""
    from warpc_public_release_b200 import ab
    try:
        timer = ab.KernelTimer()
    except Exception:
        timer = None   # no CUPTI on this box: CUDA events around each call instead, said so per row
    rows = []
    for (m, n, k) in shapes:
        long_calls = m * n * k >= 2 ** 35   # from 4096^3 up a block of calls runs into the power cap and the clock drifts across it:
        r = ab.ab_shape(torch, timer, m, n, k, inputs="uniform", rounds=2 if m * n * k < 2 ** 40 else 1, series=50 if m * n * k < 2 ** 40 else 10,
                        busy_ms=20.0 if not long_calls else 100.0, alternate=long_calls)   # there the sides take turns call by call
        mid = lambda xs: (min(xs) + max(xs)) / 2
        rows.append({"shape": [m, n, k], "program": r["program"], "runs_as": r["runs_as"], "us": mid(r["ours_us"]), "ours_us": r["ours_us"],
                     "cublaslt_us": r["cublaslt_us"], "vs_cublaslt_pct": r["ours_vs_cublaslt_pct"], "vs_cublaslt_mean_pct": r["ours_vs_cublaslt_mean_pct"], "tflops": r["ours_tflops"],
                     "cublaslt_tflops": r["cublaslt_tflops"], "calls_in_median": r["calls_in_median"], "timer": r["timer"], "order": r["order"],
                     "max_abs_diff_vs_cublaslt": r["max_abs_diff_vs_cublaslt"], "tol": 1e-3 * (k ** 0.5),
                     "ok": bool(r["max_abs_diff_vs_cublaslt"] <= 2e-3 * (k ** 0.5)),
                     "back_to_back_us": {"ours": r["back_to_back"]["ours_us"], "ours_dependent_launch": r["back_to_back"]["ours_dependent_launch_us"],
                                         "cublaslt": r["back_to_back"]["cublaslt_us"]},
                     "sm_mhz": r["clocks"].get("sm_mhz"), "published_warpc_us": r["published_warpc_us"], "published_cublas138_us": r["published_cublas138_us"]})
        torch.cuda.empty_cache()
    if timer is not None:
        timer.close()
    return rows


def time_cublaslt(torch, ab, rows, n, k, a, bt, c_ours, steps, tol):
    """cuBLASLt on the same operands: its fastest correct algorithm, `steps` launches back to back between events, twice."""
    c_lib = torch.empty_like(c_ours)
    lt = ab.CublasLt(rows, n, k, a.data_ptr(), bt.data_ptr(), c_lib.data_ptr())
    best, correct = ab.fastest_correct_algo(torch, lt, c_lib, c_ours, tol, rows * n * k)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for _ in range(2):
        for _ in range(3):
            lt.run(best)
        e0.record()
        for _ in range(steps):
            lt.run(best)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / steps)
    out = {"ms_per_step": min(times), "ms_per_step_runs": times, "algo": best, "correct_algos": "%d of %d" % (correct, lt.n_algos), "version": lt.version,
           "max_abs_diff_vs_ours": ab.max_abs_diff(torch, c_lib, c_ours)}
    lt.close()
    del c_lib
    return out


def ours(args, rank, world, local_rank):
    import torch
    import warpc_public_release_b200 as w
    from warpc_public_release_b200 import ab, shard
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this library has no CPU path (use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    m, n, k = WORKLOAD
    lo, hi = shard.slab_rows(m, world, rank)
    rows = hi - lo
    # synthetic inputs of the workload's shape and distribution, made on the device from a seed;
    # every rank draws the same Bt and its own rows of A
    gen = torch.Generator(device=dev).manual_seed(1)
    bt = (torch.rand((n, k), generator=gen, device=dev) * 2 - 1).to(torch.float16)
    gen_a = torch.Generator(device=dev).manual_seed(1000 + rank)
    a = (torch.rand((rows, k), generator=gen_a, device=dev) * 2 - 1).to(torch.float16)
    job = shard.ShardedGemm(m, n, k, rank, world, a, bt, device=dev)
    li = job.plan.info()
    tol = 1e-3 * (k ** 0.5)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def over_ranks(x):
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(max(3, args.warmup)):
        job.launch()
    job.plan.status()
    # parity on a row block of this rank's slab before anything is timed
    chk = min(rows, 256)
    ref = a[:chk].float() @ bt.float().T
    err = float((job.c_local[:chk] - ref).abs().max().item())
    barrier()
    sampler.timed = True
    ms = job.plan.time_launches(args.steps, warmup=0)  # CUDA events on the launching (default) stream
    sampler.timed = False
    barrier()
    job.plan.status()
    ms = over_ranks(ms)
    clocks = sampler.stop() if rank == 0 else None

    # cuBLASLt on the same operands, same process, right after: library `steps`, library `steps`, ours `steps` once more
    lib = None
    if not args.no_cublaslt:
        try:
            lib = time_cublaslt(torch, ab, rows, n, k, a, bt, job.c_local, args.steps, tol)
            lib["ms_per_step"] = over_ranks(lib["ms_per_step"])
            lib["ours_again_ms_per_step"] = over_ranks(job.plan.time_launches(args.steps, warmup=3))
        except Exception as e:  # the baseline library failing must not take the measurement with it
            lib = {"unavailable": str(e)[:200]}
        barrier()

    # a replicated C (N > 1): the slab in row bands, each band sent to every rank as it completes, NCCL beside the next band's tiles
    ms_rep = None
    if world > 1 and not args.no_allgather:
        rep = shard.ShardedGemm(m, n, k, rank, world, a, bt, replicate_c=True, device=dev)
        for _ in range(2):
            rep.launch()
            rep.wait()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            rep.launch()
            rep.wait()
        e1.record()
        torch.cuda.synchronize()
        ms_rep = over_ranks(e0.elapsed_time(e1) / args.steps)
        rep.status()
        rep_how = rep.how
        barrier()       # every rank is done writing the others' copies before any of them is unmapped or freed
        rep.close()
        del rep
        torch.cuda.empty_cache()
        barrier()

    # end to end: pinned host buffers in and out, every step.  One GPU: the C ABI's host-buffer call.  Several: every rank
    # uploads its rows of A and its rows of Bt only, the Bt shards are gathered over NVLink, C's rows go back to the host
    e2e_steps = max(1, min(args.steps, 5))
    hA = a.cpu().pin_memory()
    hC = torch.empty((rows, n), dtype=torch.float32).pin_memory()
    if world == 1:
        hB = bt.cpu().pin_memory()
        hplan = w.HostPlan(job.variant, rows, n, k, device=local_rank)
        run = lambda: hplan.run(hA.data_ptr(), hB.data_ptr(), hC.data_ptr())
        h2d, d2h = rows * k * 2 + n * k * 2, rows * n * 4
    else:
        hplan = shard.ShardedHostGemm(m, n, k, rank, world, dev)
        hB = bt[hplan.blo:hplan.bhi].cpu().pin_memory()
        run = lambda: hplan.run(hA, hB, hC)
        h2d, d2h = hplan.h2d_bytes, hplan.d2h_bytes
    run()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        run()
    torch.cuda.synchronize()
    e2e_s = over_ranks((time.perf_counter() - t0) / e2e_steps)
    hplan.status()
    e2e_err = float((hC[:chk].to(dev) - (a[:chk].float() @ bt.float().T)).abs().max().item())
    hplan.close()
    del hA, hB, hC

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return 0
    flops = 2.0 * m * n * k
    tflops = flops / (ms * 1e-3) / 1e12
    peaks, which = measured_peaks()
    per_gpu = tflops / world
    # which measured peak the timed region compares with: the clock record says whether it ran at the burst clock or under
    # the power cap's sustained one (the driver measured cuBLAS both ways)
    sm, sm_max = clocks.get("sm_mhz"), clocks.get("sm_max_mhz")
    burst = bool(sm and sm_max and sm >= 0.93 * sm_max)
    peak = peaks["bf16_tflops"] if burst else peaks["bf16_tflops_sustained"]
    line = {
        "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "us_per_call": ms * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16->f32", "data": "synthetic",
        "config": {"workload": WORKLOAD_NAME,
                   "parallelism": "M-row blocks over %d GPU(s), Bt replicated, no collective" % world,
                   "per_gpu_shape": [rows, n, k], "program": "%dx%d d%d %s" % (li.tile_m, li.tile_n, li.depth, w._lib.lib().wg_kernel_name(li.kernel_id).decode()),
                   "l2": "inputs (%.1f GB per GPU) exceed the 126 MB L2; no flush between steps" % ((rows * k * 2 + n * k * 2 + rows * n * 4) / 1e9)},
        "parity": {"max_err": err, "tol": tol, "ok": bool(err <= tol), "e2e_max_err": e2e_err, "rows_checked": chk},
        "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": "TFLOP/s", "frac": per_gpu / peak,
                     "peak_source": "%s cuBLAS bf16 %s, chosen by the clock record (median SM clock %s of %s MHz in the timed region)" % (
                         which, "burst" if burst else "sustained under the power cap", sm, sm_max),
                     "frac_of_burst": per_gpu / peaks["bf16_tflops"], "frac_of_sustained": per_gpu / peaks["bf16_tflops_sustained"],
                     "frac_of_nominal_2250": per_gpu / NOMINAL_TFLOPS,
                     "traffic": TRAFFIC_BYTES_PER_LAUNCH if world == 1 else None, "algorithmic_bytes": 2 * rows * k + 2 * n * k + 4 * rows * n},
        "e2e": {"value": flops / e2e_s / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_s * 1e3, "steps": e2e_steps,
                "h2d_bytes_per_step": world * h2d, "d2h_bytes_per_step": world * d2h,
                "path": "wg_host_run (C ABI, pipelined blocks)" if world == 1 else "per-rank rows of A and of Bt uploaded, Bt shards all-gathered over NVLink (NCCL), C rows downloaded"},
        "gpu_launches": args.steps * world,
        "clocks": clocks,
    }
    if lib is not None:
        if "ms_per_step" in lib:
            lib["tflops"] = flops / (lib["ms_per_step"] * 1e-3) / 1e12
            lib["vs_cublaslt_pct"] = 100.0 * (lib["ms_per_step"] / min(ms, lib["ours_again_ms_per_step"]) - 1.0)
            lib["method"] = "same operands and process: ours %d steps (the timed region), cuBLASLt %d steps twice (faster kept), ours %d steps again; back to back between CUDA events, max over ranks" % (
                args.steps, args.steps, args.steps)
        line["cublaslt"] = lib
    if ms_rep is not None:
        line["ms_per_step_with_allgather"] = ms_rep
        line["replicated_c"] = {"ms_per_step": ms_rep, "vs_sharded": ms_rep / ms,
                                "how": {"fused": "the kernel itself fills every GPU's copy of C: a forwarding warp reads each stored tile back from this GPU's L2 and stores it to the peers' memory over NVLink while the next tiles are computed; a one-word all-reduce ends the step",
                                        "nccl": "slab in 4 row bands on two streams, each band sent to every rank (grouped NCCL send/recv, in place) while the next band's tiles run"}[rep_how]}
    if world == 1 and not args.no_cpu:
        crow = 256
        sec, threads = cpu_numpy_sample(m, n, k, crow)
        line["cpu_baseline"] = {"value": 2.0 * crow * n * k / sec / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                "sample": "%d rows of A against all of Bt (%.3f TFLOP), numpy fp32 matmul incl. fp16->fp32 conversion, %.1f s" % (
                                    crow, 2.0 * crow * n * k / 1e12, sec)}
    if world == 1 and not args.no_sweep:
        del job, a, bt
        torch.cuda.empty_cache()
        try:
            table = shapes_table(torch, ab.SHAPES)
            sweep = [r for r in table if tuple(r["shape"]) in SWEEP]
            tot_f = sum(2.0 * r["shape"][0] * r["shape"][1] * r["shape"][2] for r in sweep)
            tot_t = sum(r["back_to_back_us"]["ours"] for r in sweep) * 1e-6
            line["shapes"] = {"method": "uniform[-1,1] inputs; us = GPU time of a call run alone, median of the last N calls; up to 4096x4096x1024 in the published order (a block of calls a side: ours / cuBLASLt / cuBLASLt / ours, twice), "
                                        "from 4096^3 up the sides take turns call by call (long calls run into the power cap and the clock drifts across a block; `order` per row); "
                                        "vs_cublaslt_pct = the library's fastest run against the midpoint of ours (README.md:93-95), vs_cublaslt_mean_pct = mean of runs against mean of runs; "
                                        "back_to_back_us = mean of launches back to back between CUDA events",
                              "within_2pct_of_cublaslt": sum(1 for r in table if r["vs_cublaslt_pct"] >= -2.0),
                              "within_2pct_of_cublaslt_mean_vs_mean": sum(1 for r in table if r["vs_cublaslt_mean_pct"] >= -2.0), "of": len(table),
                              "mid_size_sweep_tflops_back_to_back": tot_f / tot_t / 1e12, "rows": table}
        except Exception as e:
            line["shapes"] = {"unavailable": str(e)[:300]}
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()
    return 0


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel on the one-GPU
# workload (16384^3), from a one-pass ncu capture of those two counters: 8.82 GB read + 1.06 GB written.
# No capture exists for the per-GPU slabs of a sharded run, so those lines carry null.
TRAFFIC_BYTES_PER_LAUNCH = 9.88e9


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-allgather", action="store_true", help="N > 1: skip the extra leg that also replicates C on every rank")
    ap.add_argument("--no-cublaslt", action="store_true")
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        return reference_arm(args, rank)
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("bench.py --gpus %d: launch with torch.distributed.run --nproc-per-node %d" % (args.gpus, args.gpus))
    return ours(args, rank, world, local_rank)


if __name__ == "__main__":
    sys.exit(main())

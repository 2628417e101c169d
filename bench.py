"""bench.py -- fp16-in / fp32-out GEMM (C = A . Bt^T) on B200: TFLOP/s and us/call.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--shapes]

Workload (config.workload): 16384 x 16384 x 16384, uniform[-1,1] fp16 inputs from a seeded
generator, fp32 C -- the one configuration that shards: at N GPUs rank r owns M/N contiguous
rows of A and C, Bt is replicated, and the GEMM exchanges nothing ("strong" scaling, total work
fixed).  A step is one call of the hot path (one kernel launch per rank).  `value` is whole-job
TFLOP/s with inputs resident in HBM, timed with CUDA events on the launching stream, max over
ranks; `e2e` is the same metric through the host-buffer C-ABI call (pinned host A, Bt in,
C out, every step).  At N = 1 the line also carries `sweep`: the five mid-size shapes of the
single-GPU configuration (1536^3 ... 4096^3) and the other benchmark shapes, us/call each.

--impl reference times the reference's own CPU path for the same config -- numpy's fp32 matmul
of the fp16 operands (backend/node/run_tma.py:67) -- on the host cores, on a bounded sample.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
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


def cpu_numpy_sample(m, n, k, rows, repeats=1):
    """The reference's CPU path (numpy fp32 matmul of the fp16 operands, run_tma.py:67) on a
    row slab of the workload: `rows` rows of A against all of Bt.  Returns (seconds, threads)."""
    import numpy as np
    from oracle import gemm_ref
    rng = np.random.default_rng(1)
    a = rng.uniform(-1.0, 1.0, size=(rows, k)).astype(np.float16)
    bt = rng.uniform(-1.0, 1.0, size=(n, k)).astype(np.float16)
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
    rows = 256  # a 256-row slab of A per step: 2*256*16384*16384 = 0.137 TFLOP, seconds of CPU work
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_numpy_sample(m, n, k, rows)
    times = []
    threads = 1
    for _ in range(max(1, min(args.steps, 5))):
        dt, threads = cpu_numpy_sample(m, n, k, rows)
        times.append(dt)
    sec = sum(times) / len(times)
    tflops = 2.0 * rows * n * k / sec / 1e12
    sample = "rows 0..%d of A (M' = %d of %d) against all of Bt, numpy fp32 matmul incl. fp16->fp32 conversion, mean of %d" % (
        rows, rows, m, len(times))
    line = {"impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": len(times), "warmup": min(args.warmup, 1), "ms_per_step": sec * 1e3, "ms_per_full_call_extrapolated": sec * 1e3 * (m / rows),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16->f32", "data": "synthetic",
            "config": {"workload": WORKLOAD_NAME, "sample": sample},
            "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)
    return 0


def time_shape(w, torch, m, n, k, repeat, check=True):
    """One benchmark shape on the current device: parity on its first and last launch, then the
    mean of `repeat` back-to-back launches between CUDA events.  Returns a dict."""
    gen = torch.Generator(device="cuda").manual_seed(1)
    a = (torch.rand((m, k), generator=gen, device="cuda") * 2 - 1).to(torch.float16)
    bt = (torch.rand((n, k), generator=gen, device="cuda") * 2 - 1).to(torch.float16)
    c = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    v = w.choose(m, n, k)
    plan = w.Plan(v, m, n, k, a.data_ptr(), bt.data_ptr(), c.data_ptr(), device=torch.cuda.current_device())
    plan.launch()
    plan.status()
    ms = plan.time_launches(repeat, warmup=3)
    plan.status()
    out = {"shape": [m, n, k], "program": "%dx%d d%d" % (v.tile_m, v.tile_n, v.depth), "us": ms * 1e3,
           "tflops": 2.0 * m * n * k / ms / 1e9}
    if check:
        rows = min(m, 512)
        ref = a[:rows].float() @ bt.float().T
        err = float((c[:rows] - ref).abs().max().item())
        out["max_err_rows0_%d" % rows] = err
        out["tol"] = 1e-3 * (k ** 0.5)
        out["ok"] = bool(err <= out["tol"])
    plan.close()
    return out


def ours(args, rank, world, local_rank):
    import torch
    import warpc_public_release_b200 as w
    from warpc_public_release_b200 import shard
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
    job = shard.ShardedGemm(m, n, k, rank, world, a, bt, replicate_c=args.allgather, device=dev)
    li = job.plan.info()

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

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
    tol = 1e-3 * (k ** 0.5)
    del ref
    barrier()
    sampler.timed = True
    if args.allgather and world > 1:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            job.launch()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
    else:
        ms = job.plan.time_launches(args.steps, warmup=0)  # CUDA events on the launching (default) stream
    sampler.timed = False
    barrier()
    job.plan.status()
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())

    # end to end: pinned host A (this rank's rows) and Bt in, C slab out, every step
    e2e_steps = max(1, min(args.steps, 5))
    hA, hB = a.cpu().pin_memory(), bt.cpu().pin_memory()
    hC = torch.empty((rows, n), dtype=torch.float32).pin_memory()
    hplan = w.HostPlan(job.variant, rows, n, k, device=local_rank)
    hplan.run(hA.data_ptr(), hB.data_ptr(), hC.data_ptr())
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        hplan.run(hA.data_ptr(), hB.data_ptr(), hC.data_ptr())
    torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    hplan.status()
    e2e_err = float((hC[:chk].to(dev) - (a[:chk].float() @ bt.float().T)).abs().max().item())
    t = torch.tensor([e2e_s], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_s = float(t.item())
    hplan.close()
    del hA, hB, hC

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return 0
    clocks = sampler.stop()
    flops = 2.0 * m * n * k
    tflops = flops / (ms * 1e-3) / 1e12
    peaks, which = measured_peaks()
    per_gpu = tflops / world
    line = {
        "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "us_per_call": ms * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16->f32", "data": "synthetic",
        "config": {"workload": WORKLOAD_NAME,
                   "parallelism": "M-row blocks over %d GPU(s), Bt replicated, no collective%s" % (world, " + NCCL all-gather of C" if args.allgather and world > 1 else ""),
                   "per_gpu_shape": [rows, n, k], "program": "%dx%d d%d %s" % (li.tile_m, li.tile_n, li.depth, w._lib.lib().wg_kernel_name(li.kernel_id).decode()),
                   "l2": "inputs (%.1f GB per GPU) exceed the 126 MB L2; no flush between steps" % ((rows * k * 2 + n * k * 2 + rows * n * 4) / 1e9)},
        "parity": {"max_err": err, "tol": tol, "ok": bool(err <= tol), "e2e_max_err": e2e_err, "rows_checked": chk},
        "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                     "frac": per_gpu / peaks["bf16_tflops_sustained"], "peak_source": which + " (cuBLAS bf16 sustained)",
                     "frac_of_burst": per_gpu / peaks["bf16_tflops"], "frac_of_nominal_2250": per_gpu / NOMINAL_TFLOPS,
                     "traffic": TRAFFIC_BYTES_PER_LAUNCH if world == 1 else None, "algorithmic_bytes": 2 * rows * k + 2 * n * k + 4 * rows * n},
        "e2e": {"value": flops / e2e_s / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_s * 1e3, "steps": e2e_steps,
                "h2d_bytes_per_step": world * (rows * k * 2 + n * k * 2), "d2h_bytes_per_step": world * rows * n * 4},
        "gpu_launches": args.steps * world,
        "clocks": clocks,
    }
    if world == 1 and not args.no_cpu:
        crow = 256
        sec, threads = cpu_numpy_sample(m, n, k, crow)
        line["cpu_baseline"] = {"value": 2.0 * crow * n * k / sec / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                "sample": "%d rows of A against all of Bt (%.3f TFLOP), numpy fp32 matmul incl. fp16->fp32 conversion, %.1f s" % (
                                    crow, 2.0 * crow * n * k / 1e12, sec)}
    if world == 1 and not args.no_sweep:
        del job
        torch.cuda.empty_cache()
        sweep = [time_shape(w, torch, *s, repeat=50) for s in SWEEP]
        others = [time_shape(w, torch, *s, repeat=30) for s in OTHERS]
        tot_f = sum(2.0 * a_ * b_ * c_ for a_, b_, c_ in SWEEP)
        tot_t = sum(x["us"] for x in sweep) * 1e-6
        line["sweep"] = {"workload": "mid-size single-GPU sweep: " + ", ".join("%dx%dx%d" % s for s in SWEEP), "tflops": tot_f / tot_t / 1e12,
                         "timing": "mean of 50 back-to-back launches between CUDA events, per shape", "shapes": sweep, "other_shapes": others}
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()
    return 0


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel on the one-GPU
# workload (16384^3), from the one-pass ncu capture summarised in
# profiles/gemm_kernel_pair_256x256_16384x16384x16384_dram.md: 7.92 GB read + 1.06 GB written.
# No capture exists for the per-GPU slabs of a sharded run, so those lines carry null.
TRAFFIC_BYTES_PER_LAUNCH = 8.98e9


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--allgather", action="store_true", help="replicate C on every rank with an NCCL all-gather inside the step")
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

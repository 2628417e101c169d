"""Parity of the CUDA path against the oracle, through the C ABI, on a B200.

Bit-exact on the integer input families (sums of products of integers in [-3,3] are exact in
fp32, the reference's own reason for using them: backend/node/run_tma.py:55-67, 143); within
1e-3 * sqrt(K) * max|A| * max|B| on uniform[-1,1] inputs.  Full benchmark sizes are checked
through size-independent properties (exact sampled entries as backend/node/cublas_q7.cpp:91-97
does, exact row checksums) instead of a full CPU product.
"""
import hashlib
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
import warpc_public_release_b200 as w  # noqa: E402
from oracle import gemm_ref  # noqa: E402


def run_gemm(variant, m, n, k, a, bt, launches=1, prefill=float("nan"), dependent=False, mode=0):
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(bt).cuda()
    dc = torch.full((m, n), prefill, dtype=torch.float32, device="cuda")
    plan = w.Plan(variant, m, n, k, da.data_ptr(), db.data_ptr(), dc.data_ptr())
    plan.set_timeout_ms(1000)
    if dependent:
        plan.set_dependent_launch(True)
    if mode:
        plan.debug_set_mode(mode)
    for _ in range(launches):
        plan.launch()
    plan.status()
    out = dc.cpu().numpy()
    plan.close()
    return out


def check(variant, m, n, k, family, launches=1, **how):
    a, bt = gemm_ref.INPUTS[family](m, n, k)
    c = run_gemm(variant, m, n, k, a, bt, launches, **how)
    ref = gemm_ref.gemm_ref(a, bt)
    wrong = gemm_ref.count_wrong(c, ref, gemm_ref.tolerance(family, k, a, bt))
    assert wrong == 0, "%d of %d entries wrong" % (wrong, m * n)
    if family != "uniform":
        assert np.array_equal(c, ref)  # bit-exact


SW = w.swapped
CASES = [
    # (name, shape, variant builder)
    ("one_single_tile", (128, 128, 64), lambda s: w.one(*s, 4)),
    ("one_many_tiles", (256, 384, 512), lambda s: w.one(*s, 4)),
    ("pair_direct", (512, 768, 512), lambda s: SW(*s, 128, 128, 6, direct=True)),
    ("pair_direct_ring_wraps", (256, 256, 1024), lambda s: SW(*s, 128, 128, 3, direct=True)),
    ("pair_m128_fold_direct", (256, 256, 512), lambda s: SW(*s, 128, 64, 13, direct=True, ask_ahead=True)),
    ("pair_staged", (256, 512, 512), lambda s: SW(*s, 128, 128, 4)),
    ("pair_256x128", (512, 512, 256), lambda s: SW(*s, 256, 128, 5)),
    ("pair_192x128_ragged_rows", (448, 512, 256), lambda s: SW(*s, 192, 128, 7)),          # TMA clips the last tile row
    ("pair_192x128_clc", (384, 512, 256), lambda s: SW(*s, 192, 128, 7, clc=True)),
    ("pair_256x256", (512, 1024, 256), lambda s: SW(*s, 256, 256, 4)),
    ("pair_256x256_clc_serpentine", (1024, 2048, 512), lambda s: SW(*s, 256, 256, 4, clc=True, serpentine=True, ask_ahead=True)),
    ("persistent_stride_two_accumulators", (2048, 2304, 256), lambda s: SW(*s, 128, 128, 8, bufs=2, group=16)),
    ("clc_many_tiles", (2304, 2048, 128), lambda s: SW(*s, 192, 128, 7, clc=True)),
    ("split_k_grid_even", (512, 1024, 1024), lambda s: SW(*s, 256, 256, 4, split_grid=4, split_add=True)),
    ("split_k_grid_uneven", (512, 1024, 1088), lambda s: SW(*s, 256, 256, 4, split_grid=3, split_add=True, ask_ahead=True)),
    ("split_k_more_runs_than_blocks", (256, 512, 4096), lambda s: SW(*s, 256, 256, 4, split_grid=37, split_add=True)),
    ("split_k_workspace_variant", (512, 1024, 4096), lambda s: SW(*s, 256, 256, 4, split_grid=4, direct=True)),  # the reference's ws + FADD form
    ("split_k_workspace_uneven", (512, 1024, 1088), lambda s: SW(*s, 256, 256, 4, split_grid=3, direct=True)),
    ("split_k_workspace_more_runs_than_blocks", (256, 512, 4096), lambda s: SW(*s, 256, 256, 4, split_grid=37, direct=True)),
    ("split_in_cluster_workspace", (256, 512, 16384), lambda s: SW(*s, 128, 128, 9, split=2, cluster_n=2, direct=True)),
    ("stream_k_workspace", (2560, 2048, 512), lambda s: SW(*s, 256, 128, 6, streamk=True, direct=True, bufs=2)),
    ("stream_k_workspace_fold", (1280, 1024, 1024), lambda s: SW(*s, 128, 64, 8, streamk=True, direct=True)),
    ("stream_k", (1024, 512, 1024), lambda s: SW(*s, 256, 128, 6, streamk=True, split_add=True, bufs=2, ask_ahead=True)),
    ("stream_k_long", (1024, 1024, 4096), lambda s: SW(*s, 256, 128, 6, streamk=True, split_add=True, bufs=2)),
    ("fold_rounds_partial_last_round", (256, 256, 448), lambda s: SW(*s, 128, 64, 12, direct=True)),   # 7 k-steps in rounds of 4
    ("pair_128x128_rounds_odd_k", (256, 512, 320), lambda s: SW(*s, 128, 128, 8)),                      # 5 k-steps in rounds of 2
    ("stream_k_rounds", (512, 512, 1088), lambda s: SW(*s, 128, 128, 8, streamk=True, split_add=True, bufs=2)),
    ("split_in_cluster_as_grid", (256, 512, 16384), lambda s: w.choose(*s)),
    ("rule_pair_fallback", (512, 384, 256), lambda s: w.pair(*s, 8)),
    ("rule_small", (256, 384, 512), lambda s: w.choose(*s)),
]


@pytest.mark.parametrize("family", ["integers", "hash", "uniform"])
@pytest.mark.parametrize("name,shape,build", CASES, ids=[c[0] for c in CASES])
def test_variant_against_oracle(name, shape, build, family):
    check(build(shape), *shape, family)


@pytest.mark.parametrize("name,shape,build", [c for c in CASES if "workspace" in c[0]], ids=lambda x: x if isinstance(x, str) else None)
def test_workspace_forms_give_the_same_bits_every_launch(name, shape, build):
    """K shared through a workspace adds the partial sums in a fixed order (gemm_swapped.ml:45-48 names this as what the
    L2-add forms give up): on uniform inputs, where the order of fp32 additions shows, launch after launch and plan
    after plan leave identical bits, within the tolerance of the oracle's product."""
    m, n, k = shape
    a, bt = gemm_ref.inputs_uniform(m, n, k)
    v = build(shape)
    li = w.realise(v, m, n, k)
    assert li.direct == 1 and li.sched in (3, 4) and li.ws_words == li.grid * li.tile_m * li.tile_n
    first = run_gemm(v, m, n, k, a, bt, launches=1)
    again = run_gemm(v, m, n, k, a, bt, launches=5, dependent=True)
    assert np.array_equal(first, again)
    assert gemm_ref.count_wrong(first, gemm_ref.gemm_ref(a, bt), gemm_ref.tolerance("uniform", k, a, bt)) == 0


@pytest.mark.parametrize("name,shape,build", [c for c in CASES if c[0].startswith(("split", "stream", "clc", "persistent"))],
                         ids=lambda x: x if isinstance(x, str) else None)
def test_repeated_launches_leave_the_same_answer(name, shape, build):
    # hand-off flags count launches and are never reset (gemm_swapped.ml:608-626); the 1st and the 7th launch agree
    check(build(shape), *shape, "integers", launches=7)


@pytest.mark.parametrize("name,shape,build", [c for c in CASES if c[0] in (
    "pair_staged", "persistent_stride_two_accumulators", "clc_many_tiles", "split_k_grid_even", "stream_k", "rule_small", "pair_256x256")],
                         ids=lambda x: x if isinstance(x, str) else None)
def test_dependent_launches_back_to_back(name, shape, build):
    # each launch may begin while the one before it still runs (backend/node/clusterlaunch.py:54-74); the kernel's
    # griddepcontrol.wait keeps its reads and writes behind the launch before it, hand-off flags included
    check(build(shape), *shape, "integers", launches=7, dependent=True)


@pytest.mark.parametrize("ksub", [1, 2, 4])
def test_every_round_length_gives_the_same_product(ksub):
    for shape, build in (((512, 512, 1088), lambda s: SW(*s, 128, 128, 8)), ((256, 256, 576), lambda s: SW(*s, 128, 64, 12, direct=True))):
        check(build(shape), *shape, "hash", mode=ksub << 8)


def test_random_variants_bit_exact():
    """Tiles, ring depths, accumulator counts, schedules and launch counts drawn at random (seeded): whatever the
    geometry functions accept has to give the oracle's product exactly on integer inputs."""
    import random
    rng = random.Random(5)
    ran = 0
    for _ in range(160):
        tm, tn = rng.choice([(128, 64), (128, 128), (192, 128), (256, 128), (256, 256), (256, 64), (128, 256)])
        m = tm * rng.randint(1, 4) - rng.choice([0, 0, 0, 64])
        n = 2 * tn * rng.randint(1, 3)
        k = 64 * rng.randint(1, 20)
        kind = rng.choice(["plain", "plain", "direct", "clc", "split", "stream", "rule"])
        kw = dict(bufs=rng.choice([None, 1, 2]), group=rng.choice([1, 2, 8]), serpentine=rng.random() < 0.3)
        if kind == "clc":
            kw.update(clc=True)
        elif kind == "direct":
            kw.update(direct=True)
        elif kind == "split":
            kw.update(split_grid=rng.randint(2, 5), split_add=True)
        elif kind == "stream":
            kw.update(streamk=True, split_add=True, bufs=2)
        try:
            v = w.choose(m, n, k) if kind == "rule" else SW(m, n, k, tm, tn, rng.randint(2, 12), **kw)
            w.realise(v, m, n, k)
        except Exception:
            continue  # a combination the builder refuses
        a, bt = gemm_ref.inputs_integers(m, n, k, seed=ran + 1)
        c = run_gemm(v, m, n, k, a, bt, launches=rng.choice([1, 1, 3]), dependent=rng.random() < 0.3)
        assert np.array_equal(c, gemm_ref.gemm_ref(a, bt)), (m, n, k, tm, tn, kind, kw)
        ran += 1
    assert ran >= 40


def test_golden_products_bit_exact(golden_dir):
    recs = json.load(open(os.path.join(golden_dir, "inputs_and_products.json")))["records"]
    for r in recs:
        m, n, k = r["shape"]
        if m % 128 or n % 128:
            variant = None
        try:
            variant = w.choose(m, n, k)
        except Exception:
            continue  # a fixture shape the rule has no program for (the oracle alone covers it)
        a, bt = gemm_ref.INPUTS[r["family"]](m, n, k)
        c = run_gemm(variant, m, n, k, a, bt)
        assert hashlib.sha256(np.ascontiguousarray(c).tobytes()).hexdigest() == r["ref_sha256"], r["shape"]


BENCH_SHAPES = [(1024, 1024, 1024), (1536, 1536, 1536), (2048, 2048, 2048), (3072, 1280, 2048), (4096, 4096, 1024),
                (4096, 4096, 4096), (8192, 2048, 4096), (8192, 8192, 8192), (2048, 2048, 16384), (1024, 1024, 65536)]


@pytest.mark.parametrize("shape", BENCH_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_benchmark_shape_full_size_properties(shape):
    """The program the rule picks, at full size, on the index-hash inputs: 64 sampled entries
    exact, and every row checksum exact (sum_j C[i,j] == A[i,:] . sum_j Bt[j,:] in integers)."""
    m, n, k = shape
    a, bt = gemm_ref.inputs_hash(m, n, k)
    c = run_gemm(w.choose(m, n, k), m, n, k, a, bt, launches=2)
    assert gemm_ref.sampled_exact(c, m, n, k) == 0
    colsum = bt.astype(np.int64).sum(axis=0)
    want = a.astype(np.int64) @ colsum
    got = c.astype(np.float64).sum(axis=1)
    assert np.array_equal(got, want.astype(np.float64))
    # and columns: sum_i C[i,j] == Bt[j,:] . sum_i A[i,:]
    assert np.array_equal(c.astype(np.float64).sum(axis=0), (bt.astype(np.int64) @ a.astype(np.int64).sum(axis=0)).astype(np.float64))


# ---- the shape that shards (16384^3) and its per-GPU slabs: inputs and checks stay on the device, tied to the oracle by samples

BIG = 16384


@pytest.fixture(scope="module")
def big_hash_inputs():
    """A and B^T of 16384^3 on the index-hash inputs (run_tma.py:58-62), evaluated on the device in row chunks; three rows
    of each are compared with the oracle's own generator, so the device copy is the oracle's matrix."""
    def matrix(rows, cols, salt):
        out = torch.empty((rows, cols), dtype=torch.float16, device="cuda")
        step = 2048
        for r0 in range(0, rows, step):
            i = torch.arange(r0 * cols, (r0 + step) * cols, dtype=torch.int64, device="cuda")
            out[r0:r0 + step] = ((((i * 2654435761 + salt) >> 13) % 7) - 3).to(torch.float16).reshape(step, cols)
        for r in (0, rows // 3 + 1, rows - 1):
            assert np.array_equal(out[r].cpu().numpy().astype(np.int64), gemm_ref._hash_values_range(r * cols, cols, salt))
        return out
    a, bt = matrix(BIG, BIG, 1), matrix(BIG, BIG, 7)
    yield a, bt
    del a, bt
    torch.cuda.empty_cache()


def device_properties_exact(c, a, bt, row0=0):
    """Size-independent checks of C = A . Bt^T on the hash inputs without a full CPU product: 64 sampled entries against
    the oracle's integer dot products (cublas_q7.cpp:91-97), every row checksum and every column checksum exact
    (sum_j C[i,j] = A[i,:] . sum_j Bt[j,:]; all quantities are integers below 2^53, so float64 sums are exact in any order).
    `a`, `c` hold rows row0.. of the full A and C."""
    m, k = a.shape
    n = bt.shape[0]
    for s_ in range(64):
        i, j = (s_ * 7919 + 13) % m, (s_ * 104729 + 5) % n
        want = int(np.dot(gemm_ref._hash_values_range((row0 + i) * k, k, 1), gemm_ref._hash_values_range(j * k, k, 7)))
        assert float(c[i, j].item()) == float(want), (i, j)
    bsum = bt.sum(dim=0, dtype=torch.float64)
    asum = a.sum(dim=0, dtype=torch.float64)
    # the expected checksums themselves against the oracle's integers, at three rows / columns
    for i in (0, m // 2 + 3, m - 1):
        ra = gemm_ref._hash_values_range((row0 + i) * k, k, 1)
        assert float((a[i].double() * bsum).sum().item()) == float(int(np.dot(ra, bsum.cpu().numpy().astype(np.int64))))
    step = 2048
    for r0 in range(0, m, step):
        want_rows = a[r0:r0 + step].double() @ bsum
        assert torch.equal(c[r0:r0 + step].sum(dim=1, dtype=torch.float64), want_rows), "row checksums of rows %d.." % r0
    for c0 in range(0, n, step):
        want_cols = bt[c0:c0 + step].double() @ asum
        assert torch.equal(c[:, c0:c0 + step].sum(dim=0, dtype=torch.float64), want_cols), "column checksums of columns %d.." % c0


@pytest.mark.parametrize("gpus", [1, 2, 4, 8])
def test_sharded_shape_and_its_slabs_full_size(big_hash_inputs, gpus):
    """16384^3 (gpus = 1: the program the rule picks) and the slab one of 2 / 4 / 8 GPUs owns, launched the way the
    multi-GPU runner launches it (shard.ShardedGemm), two launches each, on rows
    [M/g, 2M/g) of A -- a slab that does not start at row 0."""
    from warpc_public_release_b200 import shard
    a, bt = big_hash_inputs
    rank = 1 if gpus > 1 else 0
    lo, hi = shard.slab_rows(BIG, gpus, rank)
    rows = hi - lo
    if gpus == 1:
        c = torch.full((rows, BIG), float("nan"), dtype=torch.float32, device="cuda")
        plan = w.Plan(w.choose(BIG, BIG, BIG), rows, BIG, BIG, a.data_ptr(), bt.data_ptr(), c.data_ptr())
        plan.set_timeout_ms(2000)
        plan.launch()
        plan.launch()
        plan.status()
        plan.close()
    else:
        job = shard.ShardedGemm(BIG, BIG, BIG, rank, gpus, a[lo:hi], bt, device=a.device)
        # the large-shape program while its pair tiles fill the last wave (2, 4 GPUs); the rule's re-tiled program at 8
        assert (job.variant.tile_m, job.variant.tile_n, job.variant.clc) == ((256, 256, 1) if gpus < 8 else (192, 128, 1))
        job.c_local.fill_(float("nan"))
        job.launch()
        job.launch()
        torch.cuda.synchronize()
        job.status()
        c = job.c_local
    device_properties_exact(c, a[lo:hi], bt, row0=lo)


def test_column_block_plans_side_by_side():
    """One product as two launches on two streams, each a column block of the same C (wg_plan_create_block: rows ldc
    apart), one through staging copies and TMA, one from the registers; bit-exact."""
    m, n, k, n1 = 512, 1536, 512, 1024
    a, bt = gemm_ref.inputs_integers(m, n, k)
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(bt).cuda()
    dc = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    p1 = w.Plan(SW(m, n1, k, 256, 256, 4, clc=True, serpentine=True, ask_ahead=True), m, n1, k, da.data_ptr(), db.data_ptr(), dc.data_ptr(), ldc=n)
    p2 = w.Plan(SW(m, n - n1, k, 256, 128, 7, clc=True, serpentine=True, direct=True, bufs=2), m, n - n1, k, da.data_ptr(), db[n1:].data_ptr(),
                dc[:, n1:].data_ptr(), ldc=n)
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    for _ in range(3):
        p1.launch(stream=s1.cuda_stream)
        p2.launch(stream=s2.cuda_stream)
    p1.status()
    p2.status()
    assert np.array_equal(dc.cpu().numpy(), gemm_ref.gemm_ref(a, bt))
    p1.close()
    p2.close()


@pytest.mark.parametrize("shape", BENCH_SHAPES + [(BIG, BIG, BIG)], ids=lambda s: "x".join(map(str, s)))
def test_benchmark_shape_uniform_inputs_within_tolerance(shape):
    """Every benchmark shape on uniform[-1,1] inputs: 64 rows spread over M against the oracle within
    1e-3 sqrt(K) max|A| max|B|; up to 4096^3 also linearity (the same kernel on 2A)."""
    m, n, k = shape
    a, bt = gemm_ref.inputs_uniform(m, n, k)
    c = run_gemm(w.choose(m, n, k), m, n, k, a, bt)
    rows = np.arange(0, m, max(1, m // 64))[:64]
    ref = gemm_ref.gemm_ref(a[rows], bt)
    tol = gemm_ref.tolerance("uniform", k, a, bt)
    assert float(np.abs(c[rows] - ref).max()) <= tol
    if m * n * k > 4096 ** 3:
        return
    # linearity: the same kernel on 2A gives exactly 2C (scaling by a power of two is exact in fp16 and fp32)
    c2 = run_gemm(w.choose(m, n, k), m, n, k, (a * np.float16(2)).astype(np.float16), bt)
    if not w.realise(w.choose(m, n, k), m, n, k).sched in (3, 4):
        assert np.array_equal(c2[rows], 2 * c[rows])
    else:  # L2 adds land in any order: equal within the tolerance only
        assert float(np.abs(c2[rows] - 2 * c[rows]).max()) <= 2 * tol


def test_phase_stamps_layout_and_order():
    """Timing builds' stamps (the reference's: backend/stamp.ml:9-24, decoded by run_tma.py:176-203): a launch of two tiles
    a CTA on a fixed grid, stamps on.  Per CTA 64 events x 4 tile slots; events are GPU-timer nanoseconds and must come
    in the documented order, slots of tiles a CTA never ran stay zero, MMA events exist in pair leaders only, and the
    product is still exact."""
    m, n, k = 256 * 74 * 2, 256, 512          # 296 CTA tiles of 256 x 128 on 148 CTAs: two tiles each
    a, bt = gemm_ref.inputs_integers(m, n, k)
    v = w.swapped(m, n, k, 256, 128, 5)
    li = w.realise(v, m, n, k)
    assert (li.sched, li.grid) == (1, 148)
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(bt).cuda()
    dc = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    plan = w.Plan(v, m, n, k, da.data_ptr(), db.data_ptr(), dc.data_ptr())
    plan.launch()
    plan.enable_stamps(True)
    plan.launch()
    st = plan.read_stamps().astype(np.int64)
    plan.enable_stamps(False)
    plan.status()
    assert st.shape == (148, 32, 4)
    assert np.array_equal(dc.cpu().numpy(), gemm_ref.gemm_ref(a, bt))
    ENTRY, SETUP, LOAD_FIRST, LOAD_LAST, MMA_FIRST, MMA_LAST, ACC_READY, STORED, TEARDOWN, EXIT, ACC_FREE = range(11)
    assert not st[:, :15, 2:].any() and not st[:, 22, 2:].any()          # tiles 3 and 4 never ran
    assert not st[:, [15, 16, 17, 18, 19, 20, 21, 23], 1:].any()            # set-up / teardown events are per launch: tile slot 0 only
    for cta in range(148):
        e = st[cta]
        leader = cta % 2 == 0
        # set-up: entry <= barriers initialised (16), first tile found (18) <= CTAs met (23) <= set-up done; a pair's tensor
        # memory is allocated (17) after the arrival at that barrier, before the first MMA (the timer ticks every 32 ns)
        for ev in (16, 18):
            assert e[ENTRY, 0] <= e[ev, 0] <= e[23, 0], (cta, ev)
        assert e[ENTRY, 0] <= e[17, 0] <= e[ACC_READY, 0]
        if leader:
            assert e[17, 0] <= e[ACC_FREE, 0] + 64
        assert e[23, 0] <= e[SETUP, 0] <= e[LOAD_FIRST, 0]
        for t in range(2):
            assert 0 < e[LOAD_FIRST, t] <= e[LOAD_LAST, t]
            assert e[LOAD_FIRST, t] < e[ACC_READY, t] <= e[STORED, t]
            if leader:
                assert e[ACC_FREE, t] <= e[MMA_FIRST, t] <= e[MMA_LAST, t] <= e[ACC_READY, t] + 1000, (cta, t)
                assert e[LOAD_FIRST, t] < e[MMA_FIRST, t]
            else:
                assert not e[[MMA_FIRST, MMA_LAST, ACC_FREE], t].any()
        assert e[LOAD_FIRST, 0] < e[LOAD_FIRST, 1] and e[STORED, 0] < e[STORED, 1]
        # teardown, per stamping thread: the first epilogue warp's stores issued <= read (19); thread 0's roles done <= CTAs met
        # (20) <= exit; tensor memory is freed (21) by the MMA warp after the CTAs met (the timer ticks every 32 ns)
        assert e[STORED, 1] <= e[19, 0] and e[TEARDOWN, 0] <= e[20, 0] <= e[EXIT, 0] and e[20, 0] <= e[21, 0] + 64
        assert e[15, 0] > 0                                                 # SM cycles entry to exit
        assert 0 < e[EXIT, 0] - e[ENTRY, 0] < 1_000_000                     # under a millisecond
    plan.close()


@pytest.mark.parametrize("shape", [(1024, 1024, 512), (1536, 1536, 320), (2048, 2048, 256), (4096, 4096, 128), (4608, 4096, 192)],
                         ids=lambda s: "x".join(map(str, s)))
def test_simple_instance_and_its_full_twin_give_the_same_bits(shape):
    """The rule's whole-tile launches from the registers run in a simple instance of their tile; with phase stamps on, the
    same plan launches the full instance.  Same geometry, same parameters: the products must be the same bits, and exact."""
    m, n, k = shape
    v = w.choose(m, n, k)
    li = w.realise(v, m, n, k)
    assert w.kernel_is_simple(li.kernel_id) and li.sched in (0, 1)
    a, bt = gemm_ref.inputs_integers(m, n, k)
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(bt).cuda()
    dc = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    plan = w.Plan(v, m, n, k, da.data_ptr(), db.data_ptr(), dc.data_ptr())
    plan.launch()
    plan.status()
    simple = dc.cpu().numpy().copy()
    dc.fill_(float("nan"))
    plan.enable_stamps(True)
    plan.launch()
    st = plan.read_stamps()
    plan.enable_stamps(False)
    plan.status()
    full = dc.cpu().numpy().copy()
    assert st.any(), "the launch with stamps on wrote no stamps: it did not run in the full instance"
    dc.fill_(float("nan"))
    plan.launch()                                  # and back in the simple instance
    plan.status()
    assert np.array_equal(simple, gemm_ref.gemm_ref(a, bt))
    assert np.array_equal(simple, full) and np.array_equal(simple, dc.cpu().numpy())
    plan.close()


def test_one_thread_two_devices_and_replicated_c():
    """Two GPUs (skipped with fewer).  (1) One host thread drives a plan on each device in turn, the current device
    left where the caller had it.  (2) Two ranks under NCCL: ShardedGemm with a replicated C; every rank's gathered C
    equals the oracle's product."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    m, n, k = 512, 1024, 512
    a, bt = gemm_ref.inputs_integers(m, n, k)
    ref = gemm_ref.gemm_ref(a, bt)
    torch.cuda.set_device(0)
    outs, plans = [], []
    for dev in (0, 1):
        da, db = torch.from_numpy(a).to("cuda:%d" % dev), torch.from_numpy(bt).to("cuda:%d" % dev)
        dc = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda:%d" % dev)
        plans.append((w.Plan(w.choose(m, n, k), m, n, k, da.data_ptr(), db.data_ptr(), dc.data_ptr(), device=dev), da, db))
        outs.append(dc)
        assert torch.cuda.current_device() == 0
    for _ in range(3):
        for p, _, _ in plans:
            p.launch()
            assert torch.cuda.current_device() == 0
    for (p, _, _), dc in zip(plans, outs):
        p.status()
        assert np.array_equal(dc.cpu().numpy(), ref)
        p.close()
    import subprocess
    import sys as _sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([_sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", "29541", os.path.join(root, "tests", "replicated_c_ranks.py")], cwd=root, env=env,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("replicated C ok") == 2


def test_host_buffer_entry_matches_device_entry():
    m, n, k = 1024, 1024, 512
    a, bt = gemm_ref.inputs_integers(m, n, k)
    v = w.choose(m, n, k)
    hp = w.HostPlan(v, m, n, k)
    hc = np.full((m, n), np.nan, np.float32)
    hp.run(a.ctypes.data, bt.ctypes.data, hc.ctypes.data)
    hp.status()
    assert np.array_equal(hc, gemm_ref.gemm_ref(a, bt))
    hp.close()


def test_host_buffer_entry_pipelined_blocks():
    # a problem large enough (>= 256 MB moved, 2048-row and -column blocks) runs as a pipeline of block products:
    # the same C as one launch on device buffers, twice over (the second run re-uses every event and flag)
    m, n, k = 4096, 6144, 8192
    a, bt = gemm_ref.inputs_hash(m, n, k)
    v = w.choose(m, n, k)
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(bt).cuda()
    dc = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    plan = w.Plan(v, m, n, k, da.data_ptr(), db.data_ptr(), dc.data_ptr())
    plan.launch()
    plan.status()
    want = dc.cpu().numpy()
    plan.close()
    assert gemm_ref.sampled_exact(want, m, n, k) == 0
    ha, hb = torch.from_numpy(a).pin_memory(), torch.from_numpy(bt).pin_memory()
    hc = torch.full((m, n), float("nan"), dtype=torch.float32).pin_memory()
    hp = w.HostPlan(v, m, n, k)
    for _ in range(2):
        hc.fill_(float("nan"))
        hp.run(ha.data_ptr(), hb.data_ptr(), hc.data_ptr())
        hp.status()
        assert np.array_equal(hc.numpy(), want)
    hp.close()


def test_plans_sharing_a_kernel_with_rings_of_different_depth():
    # the dynamic shared memory limit is an attribute of the kernel function, not of a launch: a plan with a shallow ring
    # made after a plan with a deep one must not lower it under the first plan's launches
    m, n, k = 512, 512, 512
    a, bt = gemm_ref.inputs_integers(m, n, k)
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(bt).cuda()
    outs, plans = [], []
    for depth in (6, 2, 4):
        dc = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
        plans.append(w.Plan(SW(m, n, k, 256, 128, depth), m, n, k, da.data_ptr(), db.data_ptr(), dc.data_ptr()))
        outs.append(dc)
    for p in plans + plans[::-1]:
        p.launch()
    ref = gemm_ref.gemm_ref(a, bt)
    for p, dc in zip(plans, outs):
        p.status()
        assert np.array_equal(dc.cpu().numpy(), ref)
        p.close()


def test_edges_and_errors():
    with pytest.raises(Exception):
        w.Plan(w.choose(256, 256, 64), 256, 256, 64, 0, 0, 0)             # null pointers
    a = torch.zeros(256 * 64 + 8, dtype=torch.float16, device="cuda")
    c = torch.zeros(256 * 256, dtype=torch.float32, device="cuda")
    with pytest.raises(Exception):
        w.Plan(w.choose(256, 256, 64), 256, 256, 64, a.data_ptr() + 2, a.data_ptr(), c.data_ptr())  # misaligned A
    # all-zero operands give an all-zero C over a NaN-prefilled buffer (every entry is written)
    z = np.zeros((256, 64), np.float16)
    assert not run_gemm(w.choose(256, 256, 64), 256, 256, 64, z, z).any()


def test_a_wait_that_runs_out_is_reported_not_hung():
    """Split-K partners wait for each other's flags; a flag nothing will ever set to the awaited
    value must end in a status word within the wait's limit, with the context still usable."""
    m, n, k = 512, 1024, 1024
    a, bt = gemm_ref.inputs_integers(m, n, k)
    v = w.swapped(m, n, k, 256, 256, 4, split_grid=4, split_add=True)
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(bt).cuda()
    dc = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    plan = w.Plan(v, m, n, k, da.data_ptr(), db.data_ptr(), dc.data_ptr())
    plan.set_timeout_ms(50)
    plan.debug_set_flag(0, 1000)          # CTA 0 now counts launches from 1000: its partners never see their value
    plan.launch()
    with pytest.raises(w.DeviceWaitError) as e:
        plan.status()
    assert e.value.status[0] == 8         # a partner's flag never came up
    plan.reset()
    plan.set_timeout_ms(1000)
    plan.launch()
    plan.status()
    assert np.array_equal(dc.cpu().numpy(), gemm_ref.gemm_ref(a, bt))   # the context and the plan still work
    plan.close()

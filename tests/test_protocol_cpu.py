"""The hand-off protocol of the kernel's roles, checked on the host (no GPU): barrier counts and
parities, ring slots, accumulator states, coverage of every tile's k-steps, under seeded random
interleavings -- and the same model with one rule of the protocol broken, which it has to catch.
The reference does this by interpreting its generated kernel (backend/interp.ml:311-332, 402-417,
454-487); here the role programs are restated over the launch geometry the library reports."""
import pytest

import warpc_public_release_b200 as w
from warpc_public_release_b200 import protocol

SW = w.swapped
VARIANTS = [
    ("one", (256, 384, 512), lambda s: w.one(*s, 4)),
    ("pair_fallback", (512, 384, 256), lambda s: w.pair(*s, 8)),
    ("fold_rounds_of_four_partial", (256, 256, 448), lambda s: SW(*s, 128, 64, 12, direct=True)),
    ("rounds_of_two_odd_k", (256, 512, 320), lambda s: SW(*s, 128, 128, 8)),
    ("ring_wraps", (256, 256, 1024), lambda s: SW(*s, 128, 128, 3, direct=True)),
    ("one_tile_256x128", (512, 512, 256), lambda s: SW(*s, 256, 128, 5)),
    ("stride_two_accumulators", (2048, 2304, 256), lambda s: SW(*s, 128, 128, 8, bufs=2, group=16)),
    ("clc_more_clusters_than_fit", (2304, 2048, 128), lambda s: SW(*s, 192, 128, 7, clc=True)),
    ("clc_256x256", (1024, 2048, 512), lambda s: SW(*s, 256, 256, 4, clc=True, serpentine=True)),
    ("split_k_even", (512, 1024, 1024), lambda s: SW(*s, 256, 256, 4, split_grid=4, split_add=True)),
    ("split_k_uneven", (512, 1024, 1088), lambda s: SW(*s, 256, 256, 4, split_grid=3, split_add=True)),
    ("split_k_more_runs_than_blocks", (256, 512, 4096), lambda s: SW(*s, 256, 256, 4, split_grid=37, split_add=True)),
    ("stream_k", (1024, 512, 1024), lambda s: SW(*s, 256, 128, 6, streamk=True, split_add=True, bufs=2)),
    ("stream_k_rounds", (512, 512, 1088), lambda s: SW(*s, 128, 128, 8, streamk=True, split_add=True, bufs=2)),
    ("split_k_workspace", (512, 1024, 4096), lambda s: SW(*s, 256, 256, 4, split_grid=4, direct=True)),
    ("split_k_workspace_uneven", (512, 1024, 1088), lambda s: SW(*s, 256, 256, 4, split_grid=3, direct=True)),
    ("split_in_cluster_workspace", (256, 512, 16384), lambda s: SW(*s, 128, 128, 9, split=2, cluster_n=2, direct=True)),
    ("stream_k_workspace", (2560, 2048, 512), lambda s: SW(*s, 256, 128, 6, streamk=True, direct=True, bufs=2)),
    ("rule_2048", (2048, 2048, 2048), lambda s: w.choose(*s)),
    ("rule_4096_stream_k", (4096, 4096, 1024 * 2), lambda s: w.choose(*s)),      # three waves by stride, the last wave's tiles shared
    ("rule_stream_k_remainder_too_fine", (4096, 4864, 2048), lambda s: w.choose(*s)),  # 304 pair tiles: 4 waves + 8: one wave less by stride
    ("rule_split_k_long", (1024, 1024, 8192), lambda s: w.choose(*s)),
]


@pytest.mark.parametrize("name,shape,build", VARIANTS, ids=[v[0] for v in VARIANTS])
def test_protocol_holds_under_random_interleavings(name, shape, build):
    v = build(shape)
    for seed in ((0, 1, 2) if shape[0] * shape[1] * shape[2] < 2 ** 31 else (0,)):
        assert protocol.check(v, *shape, seed=seed) > 0


@pytest.mark.parametrize("mutation,needle", [
    ({"acc_empty_count": 7}, ""),                          # the accumulator is handed back before its last reader is done
    ({"acc_empty_count": 9}, "nothing can move"),          # a release that never comes: the MMA warp waits for ever
    ({"full_count": 2}, "nothing can move"),               # a second arrival the producer never makes
    ({"producer_rounds": 3}, ""),                          # producer and MMA issuer disagree about the ring's length
    ({"tx_short": 4096}, ""),                              # the leader states fewer bytes than land: the stage opens early
    ({"no_acc_empty_wait": True}, ""),                     # the MMA warp starts a tile on an accumulator still being read
])
def test_a_broken_protocol_is_caught(mutation, needle):
    shape = (2048, 2304, 256)  # 288 tiles on a fixed grid of 148: two tiles a CTA; one accumulator where its reuse is the point
    v = SW(*shape, 128, 128, 8, bufs=1 if "no_acc_empty_wait" in mutation else 2, group=16)
    assert protocol.check(v, *shape) > 0
    with pytest.raises(protocol.Violation) as e:
        for seed in range(4):
            protocol.check(v, *shape, seed=seed, mutate=mutation)
    assert needle in str(e.value)


@pytest.mark.parametrize("name,shape,build", [
    ("split_k_workspace", (512, 1024, 4096), lambda s: SW(*s, 256, 256, 4, split_grid=4, direct=True)),
    ("stream_k_workspace", (2560, 2048, 512), lambda s: SW(*s, 256, 128, 6, streamk=True, direct=True, bufs=2))], ids=["split", "stream"])
def test_partial_sums_read_before_their_flag_is_caught(name, shape, build):
    # through the workspace a CTA adds other CTAs' partial sums: without the wait for their flags it reads slots not written yet
    v = build(shape)
    assert protocol.check(v, *shape) > 0
    with pytest.raises(protocol.Violation) as e:
        for seed in range(6):
            protocol.check(v, *shape, seed=seed, mutate={"ws_no_flag_wait": True})
    assert "partial sums" in str(e.value)


REPLICATED = [
    ("launch_control_256x256", (1024, 2048, 512), lambda s: SW(*s, 256, 256, 4, clc=True, serpentine=True)),
    ("launch_control_more_clusters_than_fit", (2304, 2048, 128), lambda s: SW(*s, 192 + 64, 128, 6, clc=True)),
    ("stride_two_accumulators_last_tile_from_the_ring", (2048, 2304, 256), lambda s: SW(*s, 128, 128, 8, bufs=2, group=16)),
    ("one_tile_a_cta", (512, 512, 256), lambda s: SW(*s, 256, 128, 5)),
]


@pytest.mark.parametrize("name,shape,build", REPLICATED, ids=[v[0] for v in REPLICATED])
def test_a_replicated_c_reaches_every_copy_once(name, shape, build):
    # every tile goes to the other copies exactly once: handed to the forwarding warp through the two slots, or (a CTA's
    # last tile, staged whole in the ring) stored to them by the epilogue itself
    v = build(shape)
    for seed in (0, 1, 2):
        assert protocol.check(v, *shape, seed=seed, replicas=3) > 0


def test_a_forwarding_slot_overwritten_before_it_is_taken_is_caught():
    # a forwarding warp that runs far behind (its copies cross NVLink) and an epilogue that does not wait for the slot's last
    # use to have been taken: the slot is overwritten, or its barrier gets a fifth arrival
    shape = (4096, 2304, 64)
    v = SW(*shape, 128, 128, 8, bufs=2, group=16)   # eight tiles a CTA: the two slots are used several times
    assert protocol.check(v, *shape, replicas=1, mutate={"fwd_copy_ticks": 600}) > 0
    with pytest.raises(protocol.Violation) as e:
        for seed in range(8):
            protocol.check(v, *shape, seed=seed, replicas=1, mutate={"fwd_no_empty_wait": True, "fwd_copy_ticks": 600})
    assert "forwarding slot" in str(e.value) or "beyond its" in str(e.value) or "parity would alias" in str(e.value)


SIMPLE_SHAPES = [(1024, 1024, 512), (1536, 1536, 256), (2048, 2048, 256), (4096, 4096, 128), (1024, 1024, 192)]


@pytest.mark.parametrize("shape", SIMPLE_SHAPES)
def test_ctas_of_a_simple_instance_may_leave_on_their_own(shape):
    # one tile a CTA or a fixed grid by stride, stored from the registers: no cluster barrier before the exit.  Nothing may
    # reach a CTA after its own roles are done -- and the same holds, trivially, with the cluster barrier kept
    v = w.choose(*shape)
    li = w.realise(v, *shape)
    assert w.kernel_is_simple(li.kernel_id) and li.sched in (0, 1) and li.direct
    for seed in range(4):
        assert protocol.check(v, *shape, seed=seed) > 0                       # the kernel's own way: each CTA on its own
    assert protocol.check(v, *shape, seed=9, teardown="cluster") > 0


def test_a_leader_that_leaves_before_its_accumulator_is_released_is_caught():
    # what lets the pair's leader go alone is its MMA issuer's last wait, for every accumulator's release: eight arrivals,
    # four of them from the other CTA.  Without that wait an epilogue warp of the other CTA arrives on a barrier of a CTA
    # that has left.  Held at a cluster barrier the leader would still be there.
    shape = (1024, 1024, 256)
    v = w.choose(*shape)
    with pytest.raises(protocol.Violation) as e:
        for seed in range(40):
            protocol.check(v, *shape, seed=seed, mutate={"mma_no_final_drain": True})
    assert "has left" in str(e.value)
    for seed in range(4):
        assert protocol.check(v, *shape, seed=seed, mutate={"mma_no_final_drain": True}, teardown="cluster") > 0


@pytest.mark.parametrize("mutation,needle,shape", [
    ("mma_no_tmem_wait", "which is not allocated yet", (1024, 1024, 128)),
    ("mma_no_tmem_wait", "which is not allocated yet", (2048, 2048, 128)),
    ("epilogue_no_tmem_wait", "rehearses its epilogue on tensor memory that is not allocated", (1536, 1536, 128)),
])
def test_tensor_memory_allocated_after_the_set_up_barrier_has_its_own_hand_offs(mutation, needle, shape):
    # a pair's CTAs allocate after arriving at the set-up barrier: the leader's MMA lane waits for the other CTA's warp 1
    # on a barrier of its own, each CTA's epilogue warps for their own warp 1 at a named barrier; without either wait
    # tensor memory is touched before it exists
    v = w.choose(*shape)
    assert protocol.check(v, *shape, seed=2) > 0
    with pytest.raises(protocol.Violation) as e:
        for seed in range(12):
            protocol.check(v, *shape, seed=seed, mutate={mutation: True})
    assert needle in str(e.value)


def test_full_instances_keep_the_cluster_barrier():
    # launch control's last answer is released on the first CTA's barrier by takers of both CTAs, and nobody waits for
    # that: letting those CTAs go alone is a finding
    shape = (2048, 4096, 256)
    v = w.swapped(*shape, 256, 256, 4, clc=True)
    li = w.realise(v, *shape)
    assert li.sched == 2 and not w.kernel_is_simple(li.kernel_id)
    assert protocol.check(v, *shape, seed=1) > 0
    with pytest.raises(protocol.Violation) as e:
        for seed in range(20):
            protocol.check(v, *shape, seed=seed, teardown="cta")
    assert "has left" in str(e.value)


@pytest.mark.parametrize("shape", [(1024, 1024, 1024), (1536, 1536, 1536), (3072, 1280, 2048), (4096, 4096, 1024), (1024, 1024, 65536)],
                         ids=lambda s: "x".join(map(str, s)))
def test_the_rules_program_for_a_benchmark_shape(shape):
    assert protocol.check(w.choose(*shape), *shape, seed=0) > 0


def test_random_variants_small_shapes():
    """Tiles, ring depths, accumulator counts and schedules drawn at random (seeded) on small shapes: whatever
    the geometry functions accept has to run through the model clean."""
    import random
    rng = random.Random(7)
    ran = 0
    for _ in range(200):
        tm, tn = rng.choice([(128, 64), (128, 128), (192, 128), (256, 128), (256, 256), (256, 64), (128, 256)])
        m = tm * rng.randint(1, 5) - rng.choice([0, 0, 0, 64])
        n = 2 * tn * rng.randint(1, 4)
        k = 64 * rng.randint(1, 24)
        kind = rng.choice(["plain", "plain", "clc", "split", "stream", "split_ws", "stream_ws"])
        kw = dict(bufs=rng.choice([None, 1, 2]), group=rng.choice([1, 2, 8]), serpentine=rng.random() < 0.3)
        if kind == "clc":
            kw.update(clc=True)
        elif kind == "split":
            kw.update(split_grid=rng.randint(2, 5), split_add=True)
        elif kind == "stream":
            kw.update(streamk=True, split_add=True, bufs=2)
        elif kind == "split_ws":
            kw.update(split_grid=rng.randint(2, 5), direct=True)
        elif kind == "stream_ws":
            m, n = tm * rng.randint(8, 12), 2 * tn * rng.randint(3, 5)   # a tile's worth of k-steps per cluster at least
            kw.update(streamk=True, direct=True, bufs=2)
        try:
            v = SW(m, n, k, tm, tn, rng.randint(2, 12), **kw)
            w.realise(v, m, n, k)
        except Exception:
            continue  # a combination the builder refuses
        assert protocol.check(v, m, n, k, seed=rng.randint(0, 99)) > 0, (m, n, k, tm, tn, kind, kw)
        ran += 1
    assert ran >= 40


def test_cli(capsys):
    assert protocol.main(["1024", "1024", "1024"]) == 0
    assert "protocol ok" in capsys.readouterr().out

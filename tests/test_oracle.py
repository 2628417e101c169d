"""The oracle pinned: against fixtures made by executing the reference's own statements
(tests/golden/make_golden.py), against the reference's published known answers, and the numpy
restatement against the independent plain-C one."""
import hashlib
import json
import os

import numpy as np
import pytest

from oracle import gemm_ref, rule


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def test_inputs_and_products_match_reference_digests(golden_dir):
    recs = json.load(open(os.path.join(golden_dir, "inputs_and_products.json")))["records"]
    assert len(recs) >= 8
    for r in recs:
        m, n, k = r["shape"]
        a, bt = gemm_ref.INPUTS[r["family"]](m, n, k, seed=r["seed"])
        assert a.dtype == np.float16 and bt.dtype == np.float16
        assert sha(a) == r["a_sha256"] and sha(bt) == r["bt_sha256"], r["shape"]
        ref = gemm_ref.gemm_ref(a, bt)
        assert ref.dtype == np.float32
        # integer inputs: sums are exact in fp32, so the product is bit-identical whatever the BLAS order
        assert sha(ref) == r["ref_sha256"], r["shape"]
        assert float(ref.astype(np.float64).sum()) == r["ref_sum"]
        assert [float(x) for x in ref[0, :6]] == r["ref_row0"]


@pytest.mark.parametrize("family", ["integers", "hash", "uniform"])
@pytest.mark.parametrize("shape", [(64, 64, 64), (128, 192, 256), (96, 40, 512)])
def test_numpy_oracle_against_plain_c(oracle_c, family, shape):
    m, n, k = shape
    a, bt = gemm_ref.INPUTS[family](m, n, k)
    ref = gemm_ref.gemm_ref(a, bt)
    c32 = np.empty((m, n), np.float32)
    c64 = np.empty((m, n), np.float64)
    oracle_c.oracle_gemm_f16_f32(a.ctypes.data, bt.ctypes.data, c32.ctypes.data, m, n, k)
    oracle_c.oracle_gemm_f16_f64(a.ctypes.data, bt.ctypes.data, c64.ctypes.data, m, n, k)
    if family == "uniform":
        tol = gemm_ref.tolerance("uniform", k, a, bt)
        assert np.abs(ref - c64).max() <= tol and np.abs(c32 - c64).max() <= tol
    else:
        assert np.array_equal(ref, c32) and np.array_equal(ref.astype(np.float64), c64)
        assert gemm_ref.count_wrong(c32, ref, gemm_ref.tolerance(family, k)) == 0


def test_hash_inputs_and_sampled_check(oracle_c):
    m, n, k = 128, 256, 320
    a, bt = gemm_ref.inputs_hash(m, n, k)
    raw = np.empty(m * k, np.int16)
    oracle_c.oracle_hash_fill(raw.ctypes.data, m * k, 1)
    assert np.array_equal(raw.reshape(m, k).astype(np.float16), a)
    assert a.min() == -3 and a.max() == 3
    ref = gemm_ref.gemm_ref(a, bt)
    assert gemm_ref.sampled_exact(ref, m, n, k) == 0
    assert oracle_c.oracle_hash_sampled_wrong(ref.ctypes.data, m, n, k) == 0
    assert float(ref[5, 9]) == float(oracle_c.oracle_hash_entry(5, 9, k))
    broken = ref.copy()
    i, j = 13 % m, 5 % n  # the first sampled entry (s = 0)
    broken[i, j] += 1
    assert gemm_ref.sampled_exact(broken, m, n, k) == 1
    assert oracle_c.oracle_hash_sampled_wrong(broken.ctypes.data, m, n, k) == 1


def test_integer_sums_are_exact_up_to_the_longest_k():
    # |sum| <= 9 K < 2^24 for K <= 65536: the reference's reason for integer inputs (run_tma.py:55-67)
    assert 9 * 65536 < 2 ** 24
    a, bt = gemm_ref.inputs_integers(8, 8, 65536)
    ref = gemm_ref.gemm_ref(a, bt)
    exact = a.astype(np.int64) @ bt.astype(np.int64).T
    assert np.array_equal(ref.astype(np.int64), exact)


def test_tolerances():
    assert gemm_ref.tolerance("integers", 4096) == 1e-3 and gemm_ref.tolerance("hash", 64) == 1e-3
    a = np.full((2, 2), 0.5, np.float16)
    assert gemm_ref.tolerance("uniform", 4096, a, a) == pytest.approx(1e-3 * 64 * 0.25)
    c = np.array([[1.0, np.nan]], np.float32)
    assert gemm_ref.count_wrong(c, np.array([[1.0, 0.0]], np.float32), 1e-3) == 1


# ---------------------------------------------------------------- the rule, pinned on the README table

def _programs(golden_dir):
    return json.load(open(os.path.join(golden_dir, "readme_programs.json")))


def test_rule_reproduces_readme_program_table(golden_dir):
    for row in _programs(golden_dir)["programs"]:
        m, n, k = row["shape"]
        r = rule.choose(m, n, k)
        assert r["prog"] == "swapped"
        assert [r["tile_m"], r["tile_n"]] == row["tile"] and r["depth"] == row["depth"], row
        for key in ("ask_ahead", "direct", "late_launch", "clc", "streamk", "split_add"):
            assert bool(r[key]) == bool(row.get(key, False)) or (key == "late_launch" and "late_launch" not in row), (row, key)
        for key in ("nbuf", "grid", "group", "cluster_n", "split_grid"):
            if key in row:
                assert r[key] == row[key], (row, key)


def test_rule_reproduces_readme_header_2048(golden_dir):
    h = _programs(golden_dir)["header_2048"]
    r = rule.choose(2048, 2048, 2048)
    assert r["name"] == h["kernel"] and r["dynsmem"] == h["dynsmem"] and r["grid"] == h["grid"][0]
    assert r["mbarriers"] == h["mbarriers"] and r["ctas"] == h["cluster"]
    lines = [".tmap " + " ".join(map(str, t)) for t in h["tmap"]]
    assert r["param_lines"] == lines


def test_rule_geometry_known_answers():
    # per-shape geometry: stage bytes, expected-transaction bytes, tensor-memory columns (gemm_swapped.ml:50-108)
    r = rule.choose(8192, 8192, 8192)
    assert (r["stage_bytes"], r["tx_bytes"], r["dynsmem"], r["alloc_cols"], r["grid"], r["mbarriers"]) == (49152, 98304, 204800, 512, 1024, 12)
    r = rule.choose(1024, 1024, 1024)
    assert (r["stage_bytes"], r["tx_bytes"], r["dynsmem"], r["alloc_cols"], r["grid"]) == (16384, 32768, 212992, 64, 128)
    r = rule.choose(4096, 4096, 4096)
    assert (r["tiles_m"], r["tiles_n"], r["grid"], r["dynsmem"], r["alloc_cols"]) == (22, 32, 704, 208896, 512)
    r = rule.choose(1024, 1024, 65536)
    assert (r["grid"], r["nflags"], r["split_grid"]) == (144, 144, 9)
    r = rule.choose(2048, 2048, 16384)
    assert (r["grid"], r["nflags"], r["nbuf"]) == (148, 148 + 128, 2)
    r = rule.choose(2048, 16384, 16384)  # one GPU's share of 16384^3 on 8 GPUs
    assert (r["tile_m"], r["tile_n"], r["grid"], r["clc"]) == (192, 128, 1408, True)


def test_rule_fallbacks_and_refusals():
    assert rule.choose(2048, 1152, 512)["prog"] == "pair"      # more than half a wave of tiles, n % 256 != 0, m % 256 == 0
    assert rule.choose(1152, 1152, 64)["prog"] == "one"        # ... and m % 256 != 0
    assert rule.choose(256, 384, 512)["tile_n"] == 64          # few tiles: the M = 128 pair
    with pytest.raises(rule.Refused):
        rule.choose(100, 100, 100)
    with pytest.raises(rule.Refused):
        rule.swapped(1024, 1024, 1024, 128, 128, 4, streamk=True, clc=True)
    with pytest.raises(rule.Refused):
        rule.swapped(1024, 1024, 1024, 128, 128, 4, direct=True, split_grid=2, split_add=True)  # adding in the L2 goes through the staging copies
    with pytest.raises(rule.Refused):
        rule.swapped(1000, 1024, 1024, 128, 128, 4, direct=True)  # the store from the registers needs whole tiles
    assert rule.choose(2048, 2048, 16384, "sm_103a")["streamk"] is False
    assert rule.choose(1024, 1024, 1024, "sm_103a")["late_launch"] is True


def test_tile_walk_known_answers():
    # 8192^3: 32 x 32 tiles of 256 x 256, groups of 8 rows, serpentine (tiles.ml:32-80)
    at = lambda t: rule.tile_origin(t, 32, 32, 256, 256, group=8, serpentine=True)
    assert [at(t) for t in (0, 1, 2, 14, 16, 256)] == [(0, 0), (0, 256), (256, 0), (1792, 0), (0, 512), (2048, 7680)]
    # every walk is a bijection onto the tiles
    for (tm, tn, g, serp, tiles_m, tiles_n) in [(256, 256, 8, True, 32, 32), (128, 128, 16, False, 16, 16), (192, 128, 8, False, 22, 32),
                                                (128, 128, 8, False, 12, 12), (128, 64, 8, False, 8, 16)]:
        seen = {rule.tile_origin(t, tiles_m, tiles_n, tm, tn, group=g, serpentine=serp) for t in range(tiles_m * tiles_n)}
        assert len(seen) == tiles_m * tiles_n
        assert seen == {(r * tm, c * tn) for r in range(tiles_m) for c in range(tiles_n)}


def test_split_and_streamk_partitions():
    # 1024x1024x65536: kt = 1024 k-steps in 9 runs of 113 or 114 (gemm_swapped.ml:111-116)
    runs = [rule.split_run(1024, s, 9) for s in range(9)]
    assert runs[0][0] == 0 and runs[-1][1] == 1024 and all(runs[i][1] == runs[i + 1][0] for i in range(8))
    assert {e - b for b, e in runs} == {113, 114}
    # 2048x2048x16384: 64 cluster tiles x 256 k-steps over 74 clusters, 221 or 222 units each (gemm_swapped.ml:270-285)
    units, covered = 64 * 256, []
    for c in range(74):
        segs = rule.streamk_range(c, units, 74, 256)
        assert sum(ke - kb for _, kb, ke in segs) in (221, 222)
        covered += [(t, kk) for t, kb, ke in segs for kk in range(kb, ke)]
    assert len(covered) == units and len(set(covered)) == units

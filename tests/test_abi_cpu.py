"""Host side of the C ABI, no GPU needed: the library loads and exports what include/*.h
declares; the C++ rule, geometry, tile walk and header agree with the oracle and with the
fixtures the reference's own reader produced."""
import ctypes
import json
import os
import re
import subprocess
import sys

import numpy as np
import pytest

import warpc_public_release_b200 as w
from warpc_public_release_b200 import _lib, launch_header
from oracle import rule

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BENCH_SHAPES = [(1024, 1024, 1024), (1536, 1536, 1536), (2048, 2048, 2048), (3072, 1280, 2048), (4096, 4096, 1024),
                (4096, 4096, 4096), (8192, 2048, 4096), (8192, 8192, 8192), (16384, 16384, 16384), (2048, 2048, 16384),
                (1024, 1024, 65536)]


def test_library_exports_every_declared_symbol():
    text = open(os.path.join(ROOT, "include", "warpc_b200.h")).read()
    declared = sorted(set(re.findall(r"\b(wg_[a-z_0-9]+)\s*\(", text)))
    assert len(declared) >= 20
    lib = ctypes.CDLL(_lib.LIB_PATH)
    missing = [name for name in declared if not hasattr(lib, name)]
    assert missing == []
    assert _lib.lib().wg_kernel_count() >= 12
    assert _lib.lib().wg_strerror(-1).decode() == "no program for this shape"


RULE_FIELDS = ("tile_m", "tile_n", "depth", "cluster_n", "clc", "ask_ahead", "direct", "serpentine", "group", "streamk", "split",
               "split_grid", "split_add", "late_launch", "reps", "atom_m", "tmem_cols", "nbuf", "alloc_cols", "tiles_m", "tiles_n",
               "total_tiles", "ctas", "grid", "kt", "a_box_rows", "bt_box_rows", "stage_bytes", "tx_bytes", "nflags")


def _same(v, r):
    assert ("swapped", "pair", "one")[v.prog] == r["prog"]
    if r["prog"] != "swapped":
        assert (v.grid, v.total_tiles, v.depth, v.ref_dynsmem) == (r["grid"], r["total_tiles"], r["depth"], r["dynsmem"])
        return
    for f in RULE_FIELDS:
        assert int(getattr(v, f)) == int(r[f]), (f, getattr(v, f), r[f])
    assert v.ref_dynsmem == r["dynsmem"] and v.ref_mbarriers == r["mbarriers"]


@pytest.mark.parametrize("sm", ["sm_100a", "sm_103a"])
def test_rule_matches_oracle_on_benchmark_shapes(sm):
    for s in BENCH_SHAPES + [(2048, 16384, 16384), (4096, 16384, 16384), (8192, 16384, 16384)]:
        _same(w.choose(*s, sm=sm), rule.choose(*s, target=sm))


def test_rule_matches_oracle_on_a_grid_of_shapes():
    ms = [64, 128, 192, 256, 384, 512, 640, 1024, 1152, 1536, 2048, 2304, 3072, 4096, 8192]
    ks = [64, 128, 1024, 4096, 8192, 16384, 65536]
    checked = refused = 0
    for m in ms:
        for n in ms:
            for k in ks:
                try:
                    r = rule.choose(m, n, k)
                except rule.Refused:
                    with pytest.raises(_lib.WarpcError) as e:
                        w.choose(m, n, k)
                    assert e.value.code == _lib.WG_E_SHAPE
                    refused += 1
                    continue
                _same(w.choose(m, n, k), r)
                checked += 1
    assert checked > 1000 and refused > 0


def test_explicit_variants_and_refusals():
    _same(w.swapped(1024, 1024, 65536, 256, 256, 4, split_grid=9, split_add=True, ask_ahead=True), rule.choose(1024, 1024, 65536))
    _same(w.swapped(4096, 4096, 4096, 128, 128, 8, cluster_n=2, clc=True), rule.swapped(4096, 4096, 4096, 128, 128, 8, cluster_n=2, clc=True))
    _same(w.pair(2048, 1152, 512, 8), rule.pair(2048, 1152, 512, 8))
    _same(w.one(1152, 1152, 64, 4), rule.one(1152, 1152, 64, 4))
    for kw in (dict(streamk=True, clc=True), dict(direct=True, split_grid=2, split_add=True), dict(split_add=True),
               dict(split=2, cluster_n=1, direct=True)):
        with pytest.raises(rule.Refused):
            rule.swapped(1024, 1024, 1024, 128, 128, 4, **kw)
        with pytest.raises(_lib.WarpcError) as e:
            w.swapped(1024, 1024, 1024, 128, 128, 4, **kw)
        assert e.value.code == _lib.WG_E_VARIANT
    with pytest.raises(_lib.WarpcError):
        w.swapped(1000, 1024, 1024, 128, 128, 4, direct=True)   # the store from the registers needs whole tiles
    with pytest.raises(_lib.WarpcError):
        w.swapped(1024, 1024, 1024, 256, 256, 8)                # shared memory
    with pytest.raises(ValueError):
        w.choose(1024, 1024, 1024, sm="sm_90a")


def test_tile_walk_matches_oracle():
    r, c = ctypes.c_int(), ctypes.c_int()
    for s in BENCH_SHAPES[:8] + [(2048, 2048, 16384), (1024, 1024, 65536), (512, 768, 512)]:
        v = w.choose(*s)
        li = w.realise(v, *s)
        tiles_m, tiles_n = -(-s[0] // li.tile_m), -(-s[1] // li.tile_n)
        seen = set()
        for t in range(tiles_m * tiles_n):
            assert _lib.lib().wg_tile_origin(ctypes.byref(li), t, ctypes.byref(r), ctypes.byref(c)) == 0
            want = rule.tile_origin(t, tiles_m, tiles_n, li.tile_m, li.tile_n, pair=li.cg, pairs=1, pair_on_cols=True,
                                    group=li.group, serpentine=bool(li.serpentine))
            assert (r.value, c.value) == want, (s, t)
            seen.add(want)
        assert len(seen) == tiles_m * tiles_n


def test_headers_match_what_the_reference_reader_parsed(golden_dir):
    gold = json.load(open(os.path.join(golden_dir, "headers.json")))["headers"]
    assert len(gold) == 11
    for g in gold:
        m, n, k = g["shape"]
        text = w.header(w.choose(m, n, k), m, n, k)
        assert text == g["text"], "header text changed: rerun tests/golden/make_golden.py"
        assert launch_header.parse_header(text) == g["parsed_by_reference"]
        hdr = launch_header.parse_header(text)
        assert launch_header.shape_of(hdr) == (m, n, k)
        li = w.realise(w.choose(m, n, k), m, n, k)
        assert int(hdr["dynsmem"]) == li.dynsmem and hdr["grid"] == "%d 1" % li.grid and int(hdr["cluster"]) == li.cluster
        assert hdr["kernel"] == rule.choose(m, n, k)["name"]
        a, bt = launch_header.parameter(hdr, "a"), launch_header.parameter(hdr, "bt")
        assert (a["box_rows"], a["box_cols"], a["swizzle"]) == (li.a_box_rows, 64, 128)
        assert (bt["box_rows"], bt["box_cols"], bt["swizzle"]) == (li.bt_box_rows, 64, 128)
        assert li.dynsmem <= 232448 and li.tmem_cols <= 512


def test_realisation_invariants():
    for s in BENCH_SHAPES + [(2048, 1152, 512), (1152, 1152, 64), (256, 384, 512)]:
        v = w.choose(*s)
        li = w.realise(v, *s)
        assert li.grid % li.cluster == 0 and li.threads == 256
        if li.sched in (3, 4):        # K shared between CTAs: every CTA resident at once, flags sized for the grid
            assert li.grid <= 148 and li.nflags >= li.grid
        if li.sched == 1:
            assert li.grid == 148
        if li.sched == 4:              # stream-K: whole waves of pair tiles by stride, at least one wave's worth of tiles shared
            pairs = (s[0] // li.tile_m) * (s[1] // li.tile_n) // 2
            assert li.sk_dp % 74 == 0 and 0 <= li.sk_dp <= pairs - 74 or li.sk_dp == 0
        assert li.group & (li.group - 1) == 0
        # the ring: rounds of ksub slots, all of it inside the 227 KB a CTA may have
        assert li.ksub in (1, 2, 4) and li.rounds >= 2 and li.rounds * li.ksub <= li.depth
        assert li.mbarriers == 2 * li.rounds + 7
        assert li.dynsmem == 1024 + li.depth * li.stage_bytes + li.staging_bytes + 512 and li.dynsmem <= 232448
        if li.staging_bytes == 0 and not li.direct:            # no cycling copies: only where every tile is staged in the ring
            assert li.sched == 0 and li.wide_rows > 0 and li.depth * li.stage_bytes >= li.tile_m * li.tile_n * 4
        if li.direct:                                              # the store from the registers: whole tiles, K not shared
            assert li.sched in (0, 1) and li.tile_n in (64, 128) and s[0] % li.tile_m == 0 and s[1] % li.tile_n == 0 and li.staging_bytes == 0
    # an explicitly named tile is the tile run; the rule's choice may be re-tiled for this machine
    assert w.realise(w.swapped(2048, 2048, 2048, 128, 128, 8), 2048, 2048, 2048).tile_m == 128
    assert w.realise(w.choose(2048, 2048, 2048), 2048, 2048, 2048).tile_m == 256
    assert w.choose(2048, 2048, 2048).tile_m == 128 and w.choose(2048, 2048, 2048).retile == 1


def test_whole_tile_launches_from_the_registers_run_in_the_simple_instances():
    name = lambda li: _lib.lib().wg_kernel_name(li.kernel_id).decode()
    for s, kernel in (((1024, 1024, 1024), "pair_128x64_simple"), ((1536, 1536, 1536), "pair_128x128_simple"),
                      ((2048, 2048, 2048), "pair_256x128_simple"), ((3072, 1280, 2048), "pair_256x128_simple"),
                      ((4096, 4096, 1024), "pair_256x128_simple")):
        li = w.realise(w.choose(*s), *s)
        assert name(li) == kernel and li.direct == 1 and li.sched in (0, 1) and w.kernel_is_simple(li.kernel_id)
        assert "# b200 kernel %s:" % kernel in w.header(w.choose(*s), *s) and ".ptr c %d %d 4" % s[:2] in w.header(w.choose(*s), *s)
    # launch control, K shared between CTAs, the staged store and ragged tiles stay in the full instances
    for s in ((8192, 8192, 8192), (4096, 4096, 4096), (1024, 1024, 65536), (2048, 2048, 16384)):
        assert not w.kernel_is_simple(w.realise(w.choose(*s), *s).kernel_id)
    assert not w.kernel_is_simple(w.realise(w.swapped(2048, 2048, 2048, 256, 128, 6), 2048, 2048, 2048).kernel_id)        # staged
    assert not w.kernel_is_simple(w.realise(w.swapped(1920, 2048, 512, 256, 128, 6), 1920, 2048, 512).kernel_id)            # 7.5 tiles down
    # the rule's long programs run in the instance compiled for their one scheduling mode
    for s, kernel in (((4096, 4096, 4096), "pair_256x128_staged_stream_k"), ((2048, 2048, 16384), "pair_256x128_staged_stream_k"),
                      ((8192, 8192, 8192), "pair_256x256_staged_launch_control"), ((1024, 1024, 65536), "pair_256x256_staged_split_k")):
        assert name(w.realise(w.choose(*s), *s)) == kernel
    assert name(w.realise(w.swapped(4096, 4096, 1024, 256, 128, 6, clc=True), 4096, 4096, 1024)) == "pair_256x128_staged"   # no such instance
    # an instance fixes its round: a launch that needs another one runs in the full instance
    li = w.realise(w.swapped(1024, 1024, 1024, 128, 128, 3, direct=True), 1024, 1024, 1024)
    assert (li.ksub, w.kernel_is_simple(li.kernel_id)) in ((2, True), (1, False))


def test_stream_k_shares_only_the_last_wave_where_the_library_chose_it():
    # 4096^3: 256 pair tiles on 74 resident pairs: two waves walked whole by stride, the third and the remainder dealt out
    li = w.realise(w.choose(4096, 4096, 4096), 4096, 4096, 4096)
    assert (li.sched, li.grid, li.sk_dp, li.nbuf) == (4, 148, 148, 2)
    assert w.realise(w.choose(8192, 2048, 4096), 8192, 2048, 4096).sk_dp == 148
    # the rule's own stream-K program (under a wave of tiles) and explicitly named stream-K deal every tile out, as the reference does
    assert w.realise(w.choose(2048, 2048, 16384), 2048, 2048, 16384).sk_dp == 0
    v = w.swapped(4096, 4096, 4096, 256, 128, 6, streamk=True, split_add=True, bufs=2)
    assert w.realise(v, 4096, 4096, 4096).sk_dp == 0


def test_workspace_forms_are_realised_as_named():
    # explicitly named: the store from the registers with K shared means partial sums through a workspace, a slot a CTA
    s = (512, 1024, 4096)
    li = w.realise(w.swapped(*s, 256, 256, 4, split_grid=4, direct=True), *s)
    assert (li.direct, li.sched, li.split, li.grid, li.ws_words) == (1, 3, 4, 32, 32 * 256 * 256)
    assert ".ptr ws 32 65536 4" in w.header(w.swapped(*s, 256, 256, 4, split_grid=4, direct=True), *s)
    li = w.realise(w.swapped(*s, 256, 256, 4, split_grid=4, split_add=True), *s)
    assert (li.direct, li.sched, li.ws_words) == (0, 3, 0)
    s = (2560, 2048, 512)
    li = w.realise(w.swapped(*s, 256, 128, 6, streamk=True, direct=True, bufs=2), *s)
    assert (li.direct, li.sched, li.grid, li.ws_words) == (1, 4, 148, 148 * 256 * 128)
    # the rule's own split-in-cluster choice keeps adding in the L2
    s = (1024, 1024, 16384)
    v = w.choose(*s)
    assert (v.split, v.cluster_n, v.direct) == (2, 2, 1)
    li = w.realise(v, *s)
    assert (li.direct, li.sched, li.split, li.ws_words) == (0, 3, 2, 0)
    # named explicitly, the same program goes through the workspace
    li = w.realise(w.swapped(*s, 128, 128, 9, split=2, cluster_n=2, direct=True), *s)
    assert (li.direct, li.sched, li.split) == (1, 3, 2) and li.ws_words > 0
    # a stream-K share shorter than a tile's k-steps could give a tile three parts: refused for the workspace form
    with pytest.raises(_lib.WarpcError):
        w.swapped(1024, 1024, 4096, 256, 128, 6, streamk=True, direct=True, bufs=2)


def test_gemm_command_line():
    run = lambda *a: subprocess.run([sys.executable, "-m", "warpc_public_release_b200.gemm", *a], cwd=ROOT, capture_output=True, text=True)
    ok = run("gemm", "2048", "2048", "2048")
    assert ok.returncode == 0 and ".kernel swapped_2048_2048_2048_128x128_s8" in ok.stdout and ".cluster 2" in ok.stdout
    assert run("--sm", "sm_103a", "gemm", "1024", "1024", "1024").returncode == 0
    assert run("gemm", "100", "100", "100").returncode == 1
    assert run("--sm", "sm_90a", "gemm", "1024", "1024", "1024").returncode == 1
    assert run("frobnicate").returncode == 2
    sw = run("swapped", "1024", "1024", "65536", "256", "256", "4", "--split-grid", "9", "--split-add", "--ask-ahead")
    assert sw.returncode == 0 and ".ptr flags 1 144 4" in sw.stdout


def test_a_header_text_rebuilds_the_exact_program():
    """gemm -> header text -> run_tma's variant_from_header gives back the same program (same launch geometry), for
    the rule's choices and for explicitly named split-K, stream-K, launch-control and serpentine programs; a header
    whose directives were edited, or that carries no variant line, is refused rather than run as something else."""
    from warpc_public_release_b200 import run_tma
    cases = [(s, w.choose(*s)) for s in BENCH_SHAPES]
    cases += [((512, 1024, 1088), w.swapped(512, 1024, 1088, 256, 256, 4, split_grid=3, split_add=True, ask_ahead=True)),
              ((1024, 512, 1024), w.swapped(1024, 512, 1024, 256, 128, 6, streamk=True, split_add=True, bufs=2, ask_ahead=True)),
              ((384, 512, 256), w.swapped(384, 512, 256, 192, 128, 7, clc=True)),              # launch control with <= 148 tiles
              ((1024, 2048, 512), w.swapped(1024, 2048, 512, 256, 256, 4, clc=True, serpentine=True, ask_ahead=True)),
              ((2048, 2304, 256), w.swapped(2048, 2304, 256, 128, 128, 8, bufs=2, group=16)),
              ((512, 1024, 4096), w.swapped(512, 1024, 4096, 256, 256, 4, split_grid=4, direct=True)),
              ((256, 512, 16384), w.swapped(256, 512, 16384, 128, 128, 9, split=2, cluster_n=2, direct=True)),
              ((512, 384, 256), w.pair(512, 384, 256, 8)), ((256, 384, 512), w.one(256, 384, 512, 4))]
    for s, v in cases:
        text = w.header(v, *s)
        back = run_tma.variant_from_header(text, *s)
        assert w.realise(back, *s).as_dict() == w.realise(v, *s).as_dict(), s
        assert w.header(back, *s) == text
    text = w.header(cases[-4][1], *cases[-4][0])
    with pytest.raises(RuntimeError):
        run_tma.variant_from_header(text.replace(".grid ", ".grid 1"), *cases[-4][0])
    with pytest.raises(RuntimeError):
        run_tma.variant_from_header("\n".join(l for l in text.splitlines() if not l.startswith("# variant")), *cases[-4][0])


def test_mismatch_diagnostics(monkeypatch):
    """run_tma's description of a wrong result (the reference's WARPC_TILES / WARPC_DIAG, run_tma.py:144-168) on a doctored C:
    one tile never written and one entry holding a value from elsewhere."""
    import io
    from warpc_public_release_b200 import run_tma
    monkeypatch.setenv("WARPC_TILES", "1")
    monkeypatch.setenv("WARPC_DIAG", "1")
    m, n, k = 512, 512, 256
    li = w.realise(w.swapped(m, n, k, 256, 128, 5), m, n, k)
    ref = np.arange(m * n, dtype=np.float32).reshape(m, n)
    c = ref.copy()
    c[256:512, 128:256] = 0
    c[3, 5] = ref[7, 9]
    out = io.StringIO()
    run_tma.describe_mismatch(c, ref, np.argwhere(~(np.abs(c - ref) <= 1e-3)), 1e-3, li, out)
    text = out.getvalue()
    assert "wrong tiles 2 of 8, of them all-zero (never written) 1" in text and "x...\n" in text and ".x..\n" in text
    assert "zero where wrong: 32768 of 32769" in text and "the reference has that value at [[7, 9]]" in text


def test_no_cpu_fallback_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    v = w.choose(256, 256, 64)
    with pytest.raises(_lib.WarpcError) as e:
        w.Plan(v, 256, 256, 64, 0x1000, 0x2000, 0x3000)
    assert e.value.code != 0
    with pytest.raises(_lib.WarpcError):
        w.HostPlan(v, 256, 256, 64)

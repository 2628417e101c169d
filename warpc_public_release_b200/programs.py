"""The programs `warpc gemm|swapped|pair|one` name (reference: backend/warpc.ml:19-28,
backend/programs.ml:46-80) as Python calls over the C ABI."""
import ctypes

from . import _lib
from ._lib import Variant, LaunchInfo, check


def choose(m, n, k, sm="sm_100a"):
    """`warpc [--sm S] gemm M N K`: the variant the rule picks. Raises where the reference's
    command fails (no program for the shape)."""
    if sm not in ("sm_100a", "sm_103a"):
        raise ValueError("warpc: no target %s (sm_100a, sm_103a)" % sm)  # backend/warpc.ml:35
    v = Variant()
    check(_lib.lib().wg_choose(m, n, k, _lib.SM_100A if sm == "sm_100a" else _lib.SM_103A, ctypes.byref(v)),
          "gemm %d %d %d" % (m, n, k))
    return v


def swapped(m, n, k, tile_m, tile_n, depth, clc=False, ask_ahead=False, direct=False, serpentine=False, cluster_n=1,
            bufs=None, group=8, streamk=False, split=1, split_grid=1, split_add=False, late_launch=False):
    """`warpc swapped M N K TM TN DEPTH [flags]` (backend/warpc.ml:23-28)."""
    v = Variant()
    v.prog, v.tile_m, v.tile_n, v.tile_k, v.depth = _lib.PROG_SWAPPED, tile_m, tile_n, 64, depth
    v.clc, v.ask_ahead, v.direct, v.serpentine = int(clc), int(ask_ahead), int(direct), int(serpentine)
    v.cluster_n, v.bufs, v.group = cluster_n, bufs or 0, group
    v.streamk, v.split, v.split_grid, v.split_add, v.late_launch = int(streamk), split, split_grid, int(split_add), int(late_launch)
    check(_lib.lib().wg_derive(m, n, k, ctypes.byref(v)), "swapped %d %d %d %d %d %d" % (m, n, k, tile_m, tile_n, depth))
    return v


def pair(m, n, k, depth):
    """`warpc pair M N K DEPTH` (backend/warpc.ml:22)."""
    v = Variant()
    v.prog, v.depth = _lib.PROG_PAIR, depth
    check(_lib.lib().wg_derive(m, n, k, ctypes.byref(v)), "pair %d %d %d %d" % (m, n, k, depth))
    return v


def one(m, n, k, depth):
    """`warpc one M N K DEPTH` (backend/warpc.ml:21)."""
    v = Variant()
    v.prog, v.depth = _lib.PROG_ONE, depth
    check(_lib.lib().wg_derive(m, n, k, ctypes.byref(v)), "one %d %d %d %d" % (m, n, k, depth))
    return v


def realise(v, m, n, k):
    """The kernel of this library that runs `v` and its launch geometry."""
    li = LaunchInfo()
    check(_lib.lib().wg_realise(ctypes.byref(v), m, n, k, ctypes.byref(li)), "realise")
    return li


def kernel_is_simple(kernel_id):
    """Is the compiled kernel with this id one of the "simple" instances (whole tiles, one a CTA or a fixed grid by stride,
    stored from the registers, nothing else compiled in)?  Their CTAs leave without meeting their pair's other CTA."""
    name = _lib.lib().wg_kernel_name(kernel_id)
    return bool(name) and name.decode().endswith("_simple")


def header(v, m, n, k):
    """The launch header text (`.kernel/.tmap/.grid/...`, backend/compile.ml:171-186)."""
    buf = ctypes.create_string_buffer(4096)
    r = _lib.lib().wg_header(ctypes.byref(v), m, n, k, buf, len(buf))
    if r < 0:
        check(r, "header")
    return buf.value.decode()

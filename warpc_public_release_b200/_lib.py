"""ctypes binding of libwarpc_b200.so (declarations: include/warpc_b200.h)."""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libwarpc_b200.so")

WG_OK = 0
WG_E_SHAPE, WG_E_VARIANT, WG_E_ARG, WG_E_NOKERNEL, WG_E_DEVICE_WAIT, WG_E_NODRIVER, WG_E_LIMIT = -1, -2, -3, -4, -5, -6, -7
PROG_SWAPPED, PROG_PAIR, PROG_ONE = 0, 1, 2
SM_100A, SM_103A = 100, 103


class Variant(ctypes.Structure):
    """wg_variant: the rule's decision and the geometry it implies."""
    _fields_ = [(n, ctypes.c_int) for n in (
        "prog", "tile_m", "tile_n", "tile_k", "depth", "cluster_n", "clc", "ask_ahead", "direct", "serpentine", "group",
        "streamk", "split", "split_grid", "split_add", "late_launch", "bufs",
        "reps", "atom_m", "tmem_cols", "nbuf", "alloc_cols", "tiles_m", "tiles_n", "total_tiles", "ctas", "grid",
        "persistent", "kt", "a_box_rows", "bt_box_rows", "stage_bytes", "tx_bytes", "ref_dynsmem", "ref_mbarriers", "nflags", "retile")]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_}

    def __repr__(self):
        return "Variant(%s)" % ", ".join("%s=%d" % kv for kv in self.as_dict().items())


class LaunchInfo(ctypes.Structure):
    """wg_launch_info: how this library launches a variant."""
    _fields_ = [(n, ctypes.c_int) for n in (
        "kernel_id", "cg", "tile_m", "tile_n", "direct", "epi_rows", "grid", "cluster", "threads", "dynsmem", "mbarriers",
        "tmem_cols", "sched", "depth", "nbuf", "group", "cl_n", "serpentine", "ask_ahead", "split", "nflags",
        "a_box_rows", "bt_box_rows", "c_box_rows", "ksub", "rounds", "wide_rows", "stage_bytes", "staging_bytes", "ws_words", "sk_dp")]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_}


_lib = None


def lib():
    """The shared library, loaded once. Raises if it has not been built: there is no fallback."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError("libwarpc_b200.so is not built (run `python -c 'import __graft_entry__ as g; g.build()'` "
                           "or `make -C warpc_public_release_b200/csrc`); there is no CPU fallback")
    l = ctypes.CDLL(LIB_PATH)
    vp, i, u = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint
    PV, PL = ctypes.POINTER(Variant), ctypes.POINTER(LaunchInfo)
    sig = {
        "wg_choose": ([i, i, i, i, PV], i),
        "wg_derive": ([i, i, i, PV], i),
        "wg_realise": ([PV, i, i, i, PL], i),
        "wg_header": ([PV, i, i, i, ctypes.c_char_p, ctypes.c_size_t], i),
        "wg_plan_create": ([i, PV, i, i, i, vp, vp, vp, ctypes.POINTER(vp)], i),
        "wg_plan_create_block": ([i, PV, i, i, i, vp, vp, vp, i, ctypes.POINTER(vp)], i),
        "wg_plan_set_timeout_ms": ([vp, u], i),
        "wg_plan_info": ([vp, PL], i),
        "wg_launch": ([vp, vp], i),
        "wg_last_device_status": ([vp, ctypes.POINTER(u * 4)], i),
        "wg_plan_reset": ([vp], i),
        "wg_plan_destroy": ([vp], i),
        "wg_host_plan_create": ([i, PV, i, i, i, ctypes.POINTER(vp)], i),
        "wg_host_run": ([vp, vp, vp, vp], i),
        "wg_host_plan_buffer": ([vp, i], vp),
        "wg_time_launches": ([vp, i, i, ctypes.POINTER(ctypes.c_float)], i),
        "wg_plan_enable_stamps": ([vp, i], i),
        "wg_plan_set_dependent_launch": ([vp, i], i),
        "wg_plan_set_replicas": ([vp, i, ctypes.POINTER(vp)], i),
        "wg_ipc_export": ([i, vp, ctypes.c_char_p, ctypes.POINTER(ctypes.c_ulonglong)], i),
        "wg_ipc_import": ([i, ctypes.c_char_p, ctypes.c_ulonglong, ctypes.POINTER(vp)], i),
        "wg_ipc_release": ([i, vp], i),
        "wg_plan_read_stamps": ([vp, ctypes.POINTER(ctypes.c_ulonglong), ctypes.c_size_t], i),
        "wg_plan_debug_set_flag": ([vp, i, u], i),
        "wg_plan_debug_set_mode": ([vp, u], i),
        "wg_tile_origin": ([PL, i, ctypes.POINTER(i), ctypes.POINTER(i)], i),
        "wg_launch_noalloc": ([i, PV, i, i, i, vp, vp, vp, vp], i),
        "wg_noalloc_status": ([i, ctypes.POINTER(u * 4)], i),
        "wg_noalloc_max_flags": ([], i),
        "wg_kernel_count": ([], i),
        "wg_kernel_name": ([i], ctypes.c_char_p),
        "wg_strerror": ([i], ctypes.c_char_p),
    }
    for name, (args, res) in sig.items():
        f = getattr(l, name)
        f.argtypes, f.restype = args, res
    _lib = l
    return l


class WarpcError(RuntimeError):
    def __init__(self, what, code):
        self.code = code
        msg = lib().wg_strerror(code).decode()
        super().__init__("%s: %s (%d)" % (what, msg, code))


def check(code, what):
    if code != WG_OK:
        raise WarpcError(what, code)

"""Plans and launches over the C ABI (include/warpc_b200.h). Device memory comes from the
caller (any allocator: raw pointers are passed); a HostPlan owns device copies and moves
host buffers in and out, the way backend/node/run_tma.py:68-70, 142 does around a launch."""
import ctypes

from . import _lib
from ._lib import LaunchInfo, check

STATUS_NAMES = {0: "ok", 1: "producer: ring stage never released", 2: "MMA: ring stage never filled",
                3: "MMA: accumulator never released", 4: "epilogue: accumulator never completed",
                5: "no answer from the scheduler", 6: "scheduler: answer never taken", 7: "scheduler: no answer to the request",
                8: "a partner's flag never came up", 9: "tensor memory"}


class DeviceWaitError(RuntimeError):
    """A bounded device-side wait gave up; `.status` is (code, detail, cta, parity)."""

    def __init__(self, status):
        self.status = tuple(status)
        super().__init__("device wait gave up: %s (detail %#x, CTA %d, parity/target %d)" %
                         (STATUS_NAMES.get(status[0], "code %d" % status[0]), status[1], status[2], status[3]))


class _Base:
    _h = None

    def info(self):
        li = LaunchInfo()
        check(_lib.lib().wg_plan_info(self._h, ctypes.byref(li)), "wg_plan_info")
        return li

    def set_timeout_ms(self, ms):
        check(_lib.lib().wg_plan_set_timeout_ms(self._h, int(ms)), "wg_plan_set_timeout_ms")

    def launch(self, stream=None):
        """One asynchronous launch on `stream` (an integer cudaStream_t; None = default stream)."""
        check(_lib.lib().wg_launch(self._h, ctypes.c_void_p(stream or 0)), "wg_launch")

    def time_launches(self, repeat, warmup=3):
        """Mean milliseconds of `repeat` back-to-back launches between CUDA events (run_tma.py:171-175)."""
        ms = ctypes.c_float()
        check(_lib.lib().wg_time_launches(self._h, int(warmup), int(repeat), ctypes.byref(ms)), "wg_time_launches")
        return ms.value

    def set_dependent_launch(self, on=True):
        """Launches that follow may begin while the one before them in the stream still runs (the
        reference's `pdl`, backend/node/clusterlaunch.py:54-74); the kernel waits before it reads
        or writes global memory."""
        check(_lib.lib().wg_plan_set_dependent_launch(self._h, int(bool(on))), "wg_plan_set_dependent_launch")

    def set_replicas(self, pointers):
        """Further copies of C (integer device addresses this process can write, e.g. other GPUs' memory opened through
        CUDA IPC): every launch that follows stores each block of C to all of them too, tile by tile."""
        arr = (ctypes.c_void_p * max(1, len(pointers)))(*[ctypes.c_void_p(x) for x in pointers])
        check(_lib.lib().wg_plan_set_replicas(self._h, len(pointers), arr), "wg_plan_set_replicas")

    def enable_stamps(self, on=True):
        check(_lib.lib().wg_plan_enable_stamps(self._h, int(bool(on))), "wg_plan_enable_stamps")

    def read_stamps(self):
        """Phase stamps of the last launches: array [grid, 32 events, 4 tiles]; events 11-14 and 16-20 are cycle sums of GPU-timer nanoseconds (0 = not reached)."""
        import numpy as np
        grid = self.info().grid
        buf = (ctypes.c_ulonglong * (grid * 256))()
        r = _lib.lib().wg_plan_read_stamps(self._h, buf, grid * 256)
        if r < 0:
            check(r, "wg_plan_read_stamps")
        return np.frombuffer(buf, dtype=np.uint64).reshape(grid, 64, 4)[:, :32, :].copy()

    def status(self):
        """Synchronise and raise DeviceWaitError if any launch gave up."""
        st = (ctypes.c_uint * 4)()
        r = _lib.lib().wg_last_device_status(self._h, ctypes.byref(st))
        if r == _lib.WG_E_DEVICE_WAIT:
            raise DeviceWaitError(list(st))
        check(r, "wg_last_device_status")
        return tuple(st)

    def debug_set_flag(self, index, value):
        check(_lib.lib().wg_plan_debug_set_flag(self._h, int(index), int(value)), "wg_plan_debug_set_flag")

    def debug_set_mode(self, flags):
        check(_lib.lib().wg_plan_debug_set_mode(self._h, int(flags)), "wg_plan_debug_set_mode")

    def reset(self):
        check(_lib.lib().wg_plan_reset(self._h), "wg_plan_reset")

    def close(self):
        if self._h is not None:
            _lib.lib().wg_plan_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Plan(_Base):
    """Tensor maps + kernel-owned words for device pointers dA (M x K fp16), dBt (N x K fp16),
    dC (M x N fp32), row-major, 16-byte aligned."""

    def __init__(self, variant, m, n, k, dA, dBt, dC, device=0, ldc=None):
        """`ldc`: C is a column block of a wider matrix whose rows are ldc fp32 words apart (wg_plan_create_block)."""
        h = ctypes.c_void_p()
        if ldc is None:
            check(_lib.lib().wg_plan_create(device, ctypes.byref(variant), m, n, k, ctypes.c_void_p(dA), ctypes.c_void_p(dBt),
                                            ctypes.c_void_p(dC), ctypes.byref(h)), "wg_plan_create")
        else:
            check(_lib.lib().wg_plan_create_block(device, ctypes.byref(variant), m, n, k, ctypes.c_void_p(dA), ctypes.c_void_p(dBt),
                                                  ctypes.c_void_p(dC), int(ldc), ctypes.byref(h)), "wg_plan_create_block")
        self._h, self.shape, self.variant = h, (m, n, k), variant


class HostPlan(_Base):
    """A plan that owns device buffers; run(hA, hBt, hC) copies in, launches, copies out, synchronises."""

    def __init__(self, variant, m, n, k, device=0):
        h = ctypes.c_void_p()
        check(_lib.lib().wg_host_plan_create(device, ctypes.byref(variant), m, n, k, ctypes.byref(h)), "wg_host_plan_create")
        self._h, self.shape, self.variant = h, (m, n, k), variant

    def run(self, hA, hBt, hC):
        """hA, hBt, hC: integer host addresses (e.g. numpy `.ctypes.data`, pinned torch `.data_ptr()`)."""
        check(_lib.lib().wg_host_run(self._h, ctypes.c_void_p(hA), ctypes.c_void_p(hBt), ctypes.c_void_p(hC)), "wg_host_run")

    def buffer(self, which):
        return _lib.lib().wg_host_plan_buffer(self._h, which)


def ipc_export(dptr, device=0):
    """(handle bytes, offset) naming a device buffer of this process for another process of the same box (wg_ipc_export)."""
    handle, offset = ctypes.create_string_buffer(64), ctypes.c_ulonglong()
    check(_lib.lib().wg_ipc_export(device, ctypes.c_void_p(dptr), handle, ctypes.byref(offset)), "wg_ipc_export")
    return handle.raw, offset.value


def ipc_import(handle, offset, device=0):
    """Another process's buffer mapped for `device` of this process (peer access over NVLink); returns its address here."""
    out = ctypes.c_void_p()
    check(_lib.lib().wg_ipc_import(device, handle, offset, ctypes.byref(out)), "wg_ipc_import")
    return out.value


def ipc_release(dptr, device=0):
    check(_lib.lib().wg_ipc_release(device, ctypes.c_void_p(dptr)), "wg_ipc_release")


def launch_noalloc(variant, m, n, k, dA, dBt, dC, device=0, stream=None):
    """One launch that allocates no device memory (wg_launch_noalloc): for callers that may
    not call cudaMalloc where they call the GEMM -- code inside another framework's memory
    pool or a fixed memory budget, latency-critical loops.  The kernel's flags and status words
    sit in an array built into the library (up to `noalloc_max_flags()` hand-off words); calls
    on one device share it, so calls that overlap on the GPU race.  `variant` None = the rule's
    choice.  Make the first call on a device before any stream capture."""
    vref = ctypes.byref(variant) if variant is not None else None
    check(_lib.lib().wg_launch_noalloc(device, vref, m, n, k, ctypes.c_void_p(dA), ctypes.c_void_p(dBt), ctypes.c_void_p(dC),
                                       ctypes.c_void_p(stream or 0)), "wg_launch_noalloc")


def noalloc_status(device=0):
    """Synchronise and raise DeviceWaitError if a no-allocation launch gave up."""
    st = (ctypes.c_uint * 4)()
    r = _lib.lib().wg_noalloc_status(device, ctypes.byref(st))
    if r == _lib.WG_E_DEVICE_WAIT:
        raise DeviceWaitError(list(st))
    check(r, "wg_noalloc_status")
    return tuple(st)


def noalloc_max_flags():
    return _lib.lib().wg_noalloc_max_flags()

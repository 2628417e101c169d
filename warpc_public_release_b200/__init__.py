"""B200-native fp16-in / fp32-out GEMM (C = A . Bt^T) behind the reference's operator surface.

Host code here is thin: the rule, the launch header and the launch / check / time contract
call the C ABI in ``include/warpc_b200.h`` (``libwarpc_b200.so``, hand-written sm_100a CUDA)
through ctypes.  There is no CPU fallback: without the shared library every entry raises.
"""
from .programs import Variant, LaunchInfo, choose, swapped, pair, one, realise, header, kernel_is_simple  # noqa: F401
from .plan import Plan, HostPlan, DeviceWaitError  # noqa: F401

__all__ = ["Variant", "LaunchInfo", "choose", "swapped", "pair", "one", "realise", "header", "Plan", "HostPlan",
           "DeviceWaitError"]

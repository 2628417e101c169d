import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")


@pytest.fixture(scope="session")
def oracle_c():
    """The plain-C oracle (oracle/gemm_ref.c), built on demand with gcc."""
    import ctypes
    import subprocess
    so = os.path.join(ROOT, "oracle", "liboracle_gemm.so")
    if not os.path.exists(so):
        subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle"), "liboracle_gemm.so"])
    lib = ctypes.CDLL(so)
    vp, i = ctypes.c_void_p, ctypes.c_int
    lib.oracle_gemm_f16_f32.argtypes = [vp, vp, vp, i, i, i]
    lib.oracle_gemm_f16_f64.argtypes = [vp, vp, vp, i, i, i]
    lib.oracle_hash_fill.argtypes = [vp, ctypes.c_size_t, ctypes.c_uint64]
    lib.oracle_hash_entry.argtypes = [i, i, i]
    lib.oracle_hash_entry.restype = ctypes.c_long
    lib.oracle_hash_sampled_wrong.argtypes = [vp, i, i, i]
    lib.oracle_hash_sampled_wrong.restype = i
    return lib

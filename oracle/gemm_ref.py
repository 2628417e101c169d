"""Oracle for the GEMM's values -- TEST INFRASTRUCTURE, never on the product path.

The reference checks its kernels against numpy: `ref = A.astype(np.float32) @
Bt.astype(np.float32).T` (backend/node/run_tma.py:67), with inputs from a seeded generator
(run_tma.py:55-65) and `|C - ref| > 1e-3` counted as wrong (run_tma.py:143).  This file
restates exactly that, plus the uniform[-1,1] family and tolerance the build's configs name.

Pinned by tests/test_oracle.py against: tests/golden/inputs_and_products.json (digests made
by tests/golden/make_golden.py from the reference's own expressions, run in a container that
holds the reference), the exact-integer identity (sums of products of integers in [-3,3] are
exact in fp32 for K <= 65536, run_tma.py:55-67), and oracle/gemm_ref.c (an independent
plain-C triple loop).
"""
import numpy as np


def inputs_integers(m, n, k, seed=1):
    """run_tma.py:55,64-65: one generator, A drawn first, integers in [-3, 3] as fp16."""
    rng = np.random.default_rng(seed)
    a = rng.integers(-3, 4, size=(m, k)).astype(np.float16)
    bt = rng.integers(-3, 4, size=(n, k)).astype(np.float16)
    return a, bt


def _hash_values(count, salt):
    """run_tma.py:58-61 / cublas_q7.cpp:26: ((i * 2654435761 + salt) >> 13) % 7 - 3 in 64-bit arithmetic."""
    i = np.arange(count, dtype=np.uint64)
    return ((((i * np.uint64(2654435761)) + np.uint64(salt)) >> np.uint64(13)) % np.uint64(7)).astype(np.int64) - 3


def inputs_hash(m, n, k):
    """run_tma.py:56-62 (WARPC_INPUTS=hash): salt 1 for A, 7 for B^T."""
    a = _hash_values(m * k, 1).reshape(m, k).astype(np.float16)
    bt = _hash_values(n * k, 7).reshape(n, k).astype(np.float16)
    return a, bt


def inputs_uniform(m, n, k, seed=1):
    """The build's benchmark family: i.i.d. uniform[-1, 1] rounded to fp16, the same
    generator and draw order as run_tma.py:55,64-65 (A first)."""
    rng = np.random.default_rng(seed)
    a = rng.uniform(-1.0, 1.0, size=(m, k)).astype(np.float16)
    bt = rng.uniform(-1.0, 1.0, size=(n, k)).astype(np.float16)
    return a, bt


INPUTS = {"integers": inputs_integers, "hash": lambda m, n, k, seed=1: inputs_hash(m, n, k), "uniform": inputs_uniform}


def gemm_ref(a, bt):
    """run_tma.py:67, verbatim in meaning: fp32 matmul of the fp16 operands."""
    return a.astype(np.float32) @ bt.astype(np.float32).T


def tolerance(kind, k, a=None, bt=None):
    """Absolute bound on |C - ref| per entry.  Integer families: the reference's 1e-3
    (run_tma.py:143; the sums are exact, so any difference is a bug).  Uniform family:
    1e-3 * sqrt(K) * max|A| * max|B|."""
    if kind in ("integers", "hash"):
        return 1e-3
    amax = float(np.abs(a).max()) if a is not None else 1.0
    bmax = float(np.abs(bt).max()) if bt is not None else 1.0
    return 1e-3 * (k ** 0.5) * amax * bmax


def count_wrong(c, ref, tol):
    """run_tma.py:143: entries with |C - ref| > tol (NaNs count as wrong)."""
    return int(np.count_nonzero(~(np.abs(c - ref) <= tol)))


def sampled_exact(c, m, n, k, samples=64):
    """cublas_q7.cpp:91-97: exact integer check of 64 sampled entries on the hash inputs,
    without forming the reference product (usable at any size)."""
    bad = 0
    for s in range(samples):
        i, j = (s * 7919 + 13) % m, (s * 104729 + 5) % n
        ra = _hash_values_range(i * k, k, 1)
        rb = _hash_values_range(j * k, k, 7)
        if float(c[i, j]) != float(int(np.dot(ra, rb))):
            bad += 1
    return bad


def _hash_values_range(start, count, salt):
    i = np.arange(start, start + count, dtype=np.uint64)
    return ((((i * np.uint64(2654435761)) + np.uint64(salt)) >> np.uint64(13)) % np.uint64(7)).astype(np.int64) - 3

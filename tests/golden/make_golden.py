"""Generates the golden fixtures in this folder.  Run where the reference is present:

    python tests/golden/make_golden.py REFERENCE_ROOT        (or WARPC_REFERENCE=REFERENCE_ROOT)

It executes the reference's OWN code, not a restatement of it:
  * inputs_and_products.json -- the input-generation and numpy-check statements of
    backend/node/run_tma.py (the lines between `rng = np.random.default_rng(seed)` and
    `ref = ...`, lines 55-67) are cut from that file's text and executed here for both input
    families; the digests of A, Bt and ref are recorded.
  * headers.json -- this library's launch headers for the reference's benchmark shapes, parsed
    by the reference's own reader backend/node/header.py:read_header.
The fixtures are small digests / dictionaries; nothing of the reference's source is stored.
"""
import hashlib
import importlib.util
import json
import os
import re
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

SMALL_SHAPES = [(128, 128, 64), (256, 384, 512), (192, 256, 1024), (1024, 1024, 1024)]
BENCH_SHAPES = [(1024, 1024, 1024), (1536, 1536, 1536), (2048, 2048, 2048), (3072, 1280, 2048), (4096, 4096, 1024),
                (4096, 4096, 4096), (8192, 2048, 4096), (8192, 8192, 8192), (16384, 16384, 16384), (2048, 2048, 16384),
                (1024, 1024, 65536)]


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def reference_inputs_snippet(ref_root):
    """The statements of run_tma.run() that make A, Bt and ref, as text, dedented."""
    src = open(os.path.join(ref_root, "backend/node/run_tma.py")).read()
    m = re.search(r"^( +)rng = np\.random\.default_rng\(seed\)\n.*?^\1ref = [^\n]*\n", src, re.S | re.M)
    if not m:
        raise SystemExit("run_tma.py: input statements not found")
    indent = m.group(1)
    return "".join(l[len(indent):] if l.startswith(indent) else l for l in m.group(0).splitlines(True))


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("WARPC_REFERENCE")
    if not ref_root or not os.path.isdir(os.path.join(ref_root, "backend", "node")):
        raise SystemExit("usage: make_golden.py REFERENCE_ROOT  (the checkout of the reference; or set WARPC_REFERENCE)")
    snippet = reference_inputs_snippet(ref_root)
    records = []
    for family, env_inputs in (("integers", None), ("hash", "hash")):
        for (M, N, K) in SMALL_SHAPES:
            os.environ.pop("WARPC_INPUTS", None)
            os.environ.pop("WARPC_NO_CHECK", None)
            if env_inputs:
                os.environ["WARPC_INPUTS"] = env_inputs
            scope = {"np": np, "os": os, "M": M, "N": N, "K": K, "seed": 1}
            exec(snippet, scope)  # the reference's own statements
            A, Bt, ref = scope["A"], scope["Bt"], scope["ref"]
            records.append({"family": family, "shape": [M, N, K], "seed": 1, "a_sha256": sha(A), "bt_sha256": sha(Bt),
                            "ref_sha256": sha(ref.astype(np.float32)), "ref_sum": float(ref.astype(np.float64).sum()),
                            "ref_abs_max": float(np.abs(ref).max()), "ref_row0": [float(x) for x in ref[0, :6]],
                            "a_row0": [float(x) for x in A[0, :8]], "bt_row0": [float(x) for x in Bt[0, :8]]})
    os.environ.pop("WARPC_INPUTS", None)
    json.dump({"made_by": "tests/golden/make_golden.py", "source": "backend/node/run_tma.py:55-67 executed", "records": records},
              open(os.path.join(HERE, "inputs_and_products.json"), "w"), indent=1)

    spec = importlib.util.spec_from_file_location("ref_header", os.path.join(ref_root, "backend/node/header.py"))
    ref_header = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref_header)
    import warpc_public_release_b200 as w
    parsed = []
    for (M, N, K) in BENCH_SHAPES:
        text = w.header(w.choose(M, N, K), M, N, K)
        with tempfile.NamedTemporaryFile("w", suffix=".sass", delete=False) as f:
            f.write(text)
        parsed.append({"shape": [M, N, K], "text": text, "parsed_by_reference": ref_header.read_header(f.name)})
        os.unlink(f.name)
    json.dump({"made_by": "tests/golden/make_golden.py", "source": "backend/node/header.py:read_header executed", "headers": parsed},
              open(os.path.join(HERE, "headers.json"), "w"), indent=1)
    print("wrote inputs_and_products.json (%d records), headers.json (%d headers)" % (len(records), len(parsed)))


if __name__ == "__main__":
    main()

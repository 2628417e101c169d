"""Reading the launch header back.

`gemm M N K` (this package's gemm.py, over wg_header in the C ABI) prints a block of dotted
directives above a kernel; the runner rebuilds the launch from it.  The directive grammar is
the reference's (written by backend/compile.ml:171-186, read by backend/node/header.py:12-32):
a line is `.key rest`, `#` and `//` start comments, and

    integer directives   regs barriers threads smem mbarriers
    list of integers     params
    flag                 tcgen05
    parameter lines      tmap name rows cols elem box_rows box_cols swizzle
                         ptr  name rows cols elem          (kept in parameter order)
    anything else        stored as the text after the key (kernel, sm, grid, cluster, tile, dynsmem ...)

The dictionary returned uses the same keys, defaults and value types as the reference reader,
so code written against either reads the other's output; tests/golden/headers.json holds the
reference reader's own parse of this library's headers.
"""

_INT_KEYS = frozenset(("regs", "barriers", "threads", "smem", "mbarriers"))


def _defaults():
    return {"kernel": "k", "sm": "sm_100a", "regs": 16, "barriers": 0, "params": [], "threads": None, "smem": 0,
            "tcgen05": False, "mbarriers": 1}


def _strip_comment(line):
    for mark in ("#", "//"):
        cut = line.find(mark)
        if cut >= 0:
            line = line[:cut]
    return line.strip()


def parse_header(text):
    out = _defaults()
    params = []
    for line in map(_strip_comment, text.splitlines()):
        if not line.startswith("."):
            continue
        words = line[1:].split(" ", 1)
        key, rest = words[0], (words[1] if len(words) > 1 else "")
        if key in _INT_KEYS:
            out[key] = int(rest, 0)
        elif key == "params":
            out[key] = [int(tok, 0) for tok in rest.split()]
        elif key == "tcgen05":
            out[key] = True
        elif key in ("tmap", "ptr"):
            params.append(rest.split() if key == "tmap" else ["ptr"] + rest.split())
        else:
            out[key] = rest.strip()
    if params:
        out["tmap"] = params
    return out


def variant_fields(text):
    """The rule fields wg_header records in its `# variant key=value ...` comment line (a comment, so
    the reference's reader skips it), as a dict of ints; None when the text has no such line."""
    for line in text.splitlines():
        words = line.split()
        if words[:2] == ["#", "variant"]:
            return {key: int(value) for key, value in (w.split("=", 1) for w in words[2:])}
    return None


def read_header(path):
    with open(path) as handle:
        return parse_header(handle.read())


def parameter(hdr, name):
    """The header's parameter line for `name` as a dict (kind 'tmap' or 'ptr')."""
    for toks in hdr.get("tmap", []):
        plain = toks[0] == "ptr"
        fields = toks[1:] if plain else toks
        if fields[0] != name:
            continue
        d = {"kind": "ptr" if plain else "tmap", "rows": int(fields[1]), "cols": int(fields[2]), "elem": int(fields[3])}
        if not plain:
            d.update(box_rows=int(fields[4]), box_cols=int(fields[5]), swizzle=int(fields[6]))
        return d
    raise KeyError(name)


def shape_of(hdr):
    """(M, N, K): `a` is M x K and `bt` is N x K (the reference derives the shape the same
    way, backend/node/run_tma.py:218-226)."""
    a, bt = parameter(hdr, "a"), parameter(hdr, "bt")
    return a["rows"], bt["rows"], a["cols"]

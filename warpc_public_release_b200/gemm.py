"""`python -m warpc_public_release_b200.gemm [--sm S] gemm M N K` -- the reference's command line
(backend/warpc.ml:1-52) for the commands that name a kernel: prints the launch header of the
program chosen (or named) for the shape.  Exit 2 on usage, 1 where the reference's builder fails."""
import sys

from . import programs
from ._lib import WarpcError

USAGE = """usage: gemm [--sm sm_100a | sm_103a] <command>
       gemm M N K                         the program chosen for the shape
       one M N K DEPTH                    one CTA a 128 x 128 tile
       pair M N K DEPTH                   CUTLASS's orientation, a 2x1 cluster
       swapped M N K TM TN DEPTH [--clc] [--ask-ahead] [--direct] [--serpentine] [--cluster-n N] [--bufs B]
               [--group G] [--streamk] [--split S] [--split-grid S] [--split-add] [--late-launch]"""


def build(args, sm="sm_100a"):
    """The (variant, M, N, K) a command names (backend/warpc.ml:19-28)."""
    if len(args) == 4 and args[0] == "gemm":
        m, n, k = map(int, args[1:])
        return programs.choose(m, n, k, sm), m, n, k
    if len(args) == 5 and args[0] in ("one", "pair"):
        m, n, k, d = map(int, args[1:])
        return (programs.one if args[0] == "one" else programs.pair)(m, n, k, d), m, n, k
    if len(args) >= 7 and args[0] == "swapped":
        m, n, k, tm, tn, d = map(int, args[1:7])
        rest = args[7:]

        def value(flag):
            return int(rest[rest.index(flag) + 1]) if flag in rest and rest.index(flag) + 1 < len(rest) else None
        kw = dict(clc="--clc" in rest, ask_ahead="--ask-ahead" in rest, direct="--direct" in rest, serpentine="--serpentine" in rest,
                  streamk="--streamk" in rest, split_add="--split-add" in rest, late_launch="--late-launch" in rest)
        for flag, name in (("--cluster-n", "cluster_n"), ("--bufs", "bufs"), ("--split", "split"), ("--split-grid", "split_grid"),
                           ("--group", "group")):
            if value(flag) is not None:
                kw[name] = value(flag)
        return programs.swapped(m, n, k, tm, tn, d, **kw), m, n, k
    raise SystemExit(2)


def main(argv=None):
    args = list(sys.argv[1:] if argv is None else argv)
    sm = "sm_100a"
    if args[:1] == ["--sm"]:
        if len(args) < 2 or args[1] not in ("sm_100a", "sm_103a"):
            print("warpc: no target %s (sm_100a, sm_103a)" % (args[1] if len(args) > 1 else ""), file=sys.stderr)
            return 1
        sm, args = args[1], args[2:]
    try:
        v, m, n, k = build(args, sm)
    except SystemExit:
        print(USAGE, file=sys.stderr)
        return 2
    except (WarpcError, ValueError) as e:
        print("warpc: %s" % e, file=sys.stderr)
        return 1
    sys.stdout.write(programs.header(v, m, n, k))
    return 0


if __name__ == "__main__":
    sys.exit(main())

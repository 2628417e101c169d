"""Oracle for the host-side decisions -- TEST INFRASTRUCTURE, never on the product path.

A pure-Python restatement of
  * the per-shape rule `Programs.choose`            (backend/programs.ml:46-80),
  * the geometry `Gemm_swapped.build` derives       (backend/gemm_swapped.ml:27, 50-108),
  * the CTA-index -> output-tile map `Tiles.origin` (backend/tiles.ml:32-80),
  * the header's parameter lines                    (backend/compile.ml:86-88; gemm_swapped.ml:841-862).
The product computes the same things in C++ (warpc_public_release_b200/csrc/rule.cpp and the
kernel's tile map); tests compare the two.

Pinned against the reference's own published answers: the per-shape program table
(README.md:450-462), the 2048^3 header (README.md:289-300) and the known answers of
backend/test_derive.ml:20-28, 117-128 -- see tests/test_oracle.py.
"""
SMS = 148
TILE_K = 64
MAX_INT = 1 << 62


def resident_clusters(ctas):  # gemm_swapped.ml:27
    return {1: SMS, 2: 74, 4: 33, 8: 15}[ctas]


def tmem_columns(n):  # atom.ml:216-218
    c = 32
    while c < n:
        c *= 2
    return c


class Refused(Exception):
    """The reference's builder raises `failwith` for this combination."""


def swapped(m, n, k, tile_m, tile_n, depth, clc=False, ask_ahead=False, direct=False, serpentine=False, cluster_n=1,
            epi_rows=8, bufs=None, group=8, streamk=False, split=1, split_grid=1, split_add=False, late_launch=False):
    """gemm_swapped.ml:30-139: the checks and the derived numbers."""
    if streamk and (clc or cluster_n > 1 or direct == split_add):
        raise Refused("stream-K")
    if split > 1 and (split > 4 or cluster_n != split or clc or streamk or not direct):
        raise Refused("split-K in the cluster")
    if split_grid > 1 and (split > 1 or clc or streamk or direct == split_add):
        raise Refused("split-K over the grid")
    if split_add and split_grid == 1 and not streamk:
        raise Refused("adding in the L2")
    pair, elem, out_elem, epi_warps = 2, 2, 4, 4
    ctas = pair * cluster_n
    rows_needed = tile_n * pair
    atom_m = min(rows_needed, 256)
    if rows_needed % atom_m:
        raise Refused("atoms")
    reps = rows_needed // atom_m
    if atom_m not in (128, 256) or tile_m % 16 or not 16 <= tile_m <= 256:  # atom.ml:146-154
        raise Refused("UMMA shape")
    a_rows = atom_m // pair
    sb_rows, sa_rows = reps * a_rows, tile_m // pair
    acc_rows = atom_m // pair
    span = tile_m if acc_rows == 128 else tile_m // 2  # atom.ml:235-251
    tiles_m, tiles_n = -(-m // tile_m), -(-n // tile_n)
    sharing = 1 if split > 1 else cluster_n
    if tiles_m % sharing or tiles_n % pair or k % (TILE_K * split) or k // TILE_K < split_grid:
        raise Refused("clusters")
    if direct and (m % tile_m or n % tile_n):
        raise Refused("whole tiles")
    ncols = tmem_columns(reps * span)
    total = tiles_m * tiles_n
    nbuf = bufs if bufs else (2 if 2 * ncols <= 512 and total > SMS else 1)
    if ncols * nbuf > 512:
        raise Refused("tensor memory")
    if streamk:
        grid = SMS // ctas * ctas
    elif split > 1:
        grid = total * split
    elif split_grid > 1:
        grid = total * split_grid
    elif clc or total <= SMS:
        grid = total
    else:
        grid = resident_clusters(ctas) * ctas
    if split_grid > 1 and grid // ctas > resident_clusters(ctas):
        raise Refused("resident")
    stage = sa_rows * TILE_K * elem + sb_rows * TILE_K * elem
    staging = 0 if direct else epi_warps * 2 * epi_rows * 32 * out_elem
    dynsmem = depth * stage + staging
    if dynsmem + 0x800 > 232448:  # mem.ml:228
        raise Refused("shared memory")
    if split_add:
        nflags = grid + total if streamk else grid
    elif streamk or split_grid > 1:
        nflags = grid
    else:
        nflags = 0
    c_line = ".ptr c %d %d 4" % (m, n) if direct else ".tmap c %d %d 4 %d 32 128" % (m, n, epi_rows)
    return dict(prog="swapped", name="swapped_%d_%d_%d_%dx%d_s%d" % (m, n, k, tile_m, tile_n, depth), tile_m=tile_m, tile_n=tile_n,
                depth=depth, cluster_n=cluster_n, clc=clc, ask_ahead=ask_ahead, direct=direct, serpentine=serpentine, group=group,
                streamk=streamk, split=split, split_grid=split_grid, split_add=split_add, late_launch=late_launch,
                reps=reps, atom_m=atom_m, tmem_cols=ncols, nbuf=nbuf, alloc_cols=tmem_columns(ncols * nbuf), tiles_m=tiles_m,
                tiles_n=tiles_n, total_tiles=total, ctas=ctas, grid=grid, kt=k // TILE_K // split, a_box_rows=sa_rows,
                bt_box_rows=sb_rows // sharing, stage_bytes=stage, tx_bytes=pair * stage, dynsmem=dynsmem,
                mbarriers=2 * depth + 2 * nbuf + (2 if clc else 0) + (1 if split > 1 else 0), nflags=nflags,
                param_lines=[c_line, ".tmap a %d %d 2 %d 64 128" % (m, k, sa_rows), ".tmap bt %d %d 2 %d 64 128" % (n, k, sb_rows // sharing)])


def pair(m, n, k, depth=8):  # gemm_pair.ml:16-43
    if m % 256 or n % 128 or k % TILE_K:
        raise Refused("gemm_pair: whole cluster tiles")
    total = (m // 128) * (n // 128)
    return dict(prog="pair", name="pair_%d_%d_%d_s%d" % (m, n, k, depth), tile_m=128, tile_n=128, depth=depth, ctas=2,
                grid=total if total <= SMS else SMS // 2 * 2, total_tiles=total, nbuf=1, tmem_cols=128,
                dynsmem=depth * (128 * 128 + 64 * 128) + 4 * 2 * 32 * 32 * 4)


def one(m, n, k, depth=4):  # gemm_one.ml:17-30
    if m % 128 or n % 128 or k % TILE_K:
        raise Refused("gemm_one: whole tiles")
    total = (m // 128) * (n // 128)
    return dict(prog="one", name="one_%d_%d_%d_s%d" % (m, n, k, depth), tile_m=128, tile_n=128, depth=depth, ctas=1, grid=total,
                total_tiles=total, nbuf=1, tmem_cols=128, dynsmem=depth * 2 * 128 * 128)


def choose(m, n, k, target="sm_100a"):
    """programs.ml:46-80, branch for branch."""
    tiles = m // 128 * (n // 128)
    pair_fits = m % 256 == 0 and n % 128 == 0 and k % 64 == 0
    swapped_fits = n % 256 == 0 and m % 64 == 0 and k % 64 == 0 and (m + 255) // 256 * (n // 128) >= SMS

    def waves(cn):
        rc = resident_clusters(2 * cn)
        return (tiles // (2 * cn) + rc - 1) // rc if m % (128 * cn) == 0 else MAX_INT

    pair_tiles = m // 256 * (n // 512) if m % 256 == 0 and n % 512 == 0 else 0
    runs = resident_clusters(2) // pair_tiles if pair_tiles > 0 else 0
    if swapped_fits and n % 512 == 0 and m % 256 == 0 and min(m, n, k) >= 8192:
        return swapped(m, n, k, 256, 256, 4, clc=True, ask_ahead=True, serpentine=True)
    if swapped_fits and k <= 1024 and m % 256 == 0:
        return swapped(m, n, k, 256, 128, 5, late_launch=True)
    if swapped_fits:
        return swapped(m, n, k, 192, 128, 7, clc=k >= 4096)
    if 2 * tiles <= SMS and n % 128 == 0 and m % 128 == 0 and k % 64 == 0:
        if k >= 65536 and runs >= 2 and k // 64 >= runs:
            return swapped(m, n, k, 256, 256, 4, split_grid=runs, split_add=True, ask_ahead=True)
        if k >= 16384 and n // 128 % 2 == 0 and k % 128 == 0 and tiles // 2 <= resident_clusters(4):
            return swapped(m, n, k, 128, 128, 9, split=2, cluster_n=2, direct=True)
        return swapped(m, n, k, 128, 64, 13, direct=True, ask_ahead=True, late_launch=(target == "sm_103a"))
    if tiles <= SMS and n % 256 == 0 and m % 128 == 0 and k % 64 == 0:
        return swapped(m, n, k, 128, 128, 6, direct=True, late_launch=True)
    if tiles > SMS and k >= 16384 and m % 512 == 0 and n % 256 == 0 and m // 512 * (n // 256) <= resident_clusters(4):
        if target == "sm_100a":
            return swapped(m, n, k, 256, 128, 6, streamk=True, split_add=True, bufs=2, ask_ahead=True)
        return swapped(m, n, k, 256, 128, 6, cluster_n=2, late_launch=True)
    if tiles > SMS and n % 256 == 0 and k % 64 == 0 and waves(2) != MAX_INT:
        cluster_n = 4 if waves(4) <= waves(2) else (1 if waves(1) <= waves(2) else 2)
        return swapped(m, n, k, 128, 128, 9 if k >= 8192 else 8, clc=cluster_n > 1, cluster_n=cluster_n,
                       late_launch=cluster_n == 4, group=16)
    if pair_fits:
        return pair(m, n, k, 8)
    return one(m, n, k, 4)


def _pow2(x):
    return x > 0 and x & (x - 1) == 0


def tile_origin(t, tiles_m, tiles_n, tile_m, tile_n, pair=2, pairs=1, pair_on_cols=True, group=1, serpentine=False):
    """tiles.ml:32-80 (the `along_n = false` walk): the (row, col) of CTA index t's tile.
    Digits of t, fastest first: the pair partner, the pair within the cluster, the row
    within a group of cluster rows, the cluster column, the band of groups."""
    cm, cn = (pairs, pair) if pair_on_cols else (pair, pairs)
    cl_m, cl_n = tiles_m // cm, tiles_n // cn
    if cl_m * cm != tiles_m or cl_n * cn != tiles_n:
        raise Refused("Tiles: the clusters do not tile the output")
    walked, other = cl_m, cl_n
    g = 1
    while g * 2 <= walked and g < group:
        g *= 2
    g = g if _pow2(other) and walked % g == 0 else 1
    width = tiles_n
    row_stride, col_stride = cm * width, cn
    x = t
    if pair_on_cols:
        within_sizes, within_strides = [pair, pairs], [1, width]
    else:
        within_sizes, within_strides = [pair, pairs], [width, 1]
    off = 0
    for size, stride in zip(within_sizes, within_strides):
        off += (x % size) * stride
        x //= size
    for size, stride in ((g, row_stride), (cl_n, col_stride), (cl_m // g, g * row_stride)):
        off += (x % size) * stride
        x //= size
    trow, tcol = off // width, off % width
    serp = serpentine and _pow2(cl_n) and cl_n > 1
    if serp:
        band = trow // (g * cm) % 2
        tcol ^= (cl_n - 1) * cn * band
    return trow * tile_m, tcol * tile_n


def split_run(kt, s, runs):
    """gemm_swapped.ml:111-116: run s of `runs` covers k-steps [s q + s r / S, (s+1) q + (s+1) r / S)."""
    q, r = kt // runs, kt % runs
    return s * q + s * r // runs, (s + 1) * q + (s + 1) * r // runs


def streamk_range(c, units, clusters, kt):
    """gemm_swapped.ml:270-285: cluster c's units and its (tile, kb, ke) segments, last tile first."""
    q, r = units // clusters, units % clusters
    b, l = c * q + c * r // clusters, (c + 1) * q + (c + 1) * r // clusters - 1
    t_first, kb_first, t_last, ke_last = b // kt, b % kt, l // kt, l % kt + 1
    return [(t, kb_first if t == t_first else 0, ke_last if t == t_last else kt) for t in range(t_last, t_first - 1, -1)]

"""Host-side check of the kernel's hand-off protocol, no GPU needed.

The reference checks its generated kernels on the host by interpreting them against a model of
mbarriers, tensor-memory column states and happens-before (backend/interp.ml:454-487 barriers,
402-417 tensor memory, 311-332 ordering).  This library's kernel is CUDA C++, which cannot be
interpreted here, so the check is one level up: the role programs of gemm_kernel (producer, MMA
issuer, epilogue warps, cluster-launch-control scheduler; csrc/gemm_kernel.cuh) are restated below
as event generators over the launch geometry `wg_realise` reports, and run against the same kind
of model under a seeded random interleaving, with loads and commits completing late and out of
step.  It reports

  * an arrival beyond a barrier's count, a wait that could be fooled by a phase two ahead,
  * a load into a ring slot that still holds unread operands, an MMA on a slot whose bytes
    have not all landed (or landed for another k-step),
  * an MMA that overwrites an accumulator nobody has read, or adds to one that was read out,
    an epilogue read of an accumulator whose MMAs are not complete,
  * a k-step of a tile multiplied twice or never, a tile stored twice or added to before it
    was stored (split-K, stream-K),
  * an MMA into, or an epilogue read of, tensor memory that its CTA's warp 1 has not allocated yet (a pair's CTAs
    allocate after their arrival at the set-up barrier, so the pair meets without waiting for it),
  * roles that can no longer move (what would be a hang on the GPU), and CTAs that would leave
    with copies or commits still in flight,
  * anything that reaches a CTA after it has left: an arrival on one of its barriers, a load landing in its ring, an
    MMA reading its slots or writing its tensor memory, a commit reporting to it.  The kernel's full instances hold
    both CTAs of a pair at a cluster barrier until every role of both is done; its simple instances (whole tiles, one
    a CTA or by stride, stored from the registers) let each CTA go when its own roles are done (`teardown="cta"`):
    every word one CTA sends the other is waited for by a role of the receiving CTA before that role ends.

    python -m warpc_public_release_b200.protocol M N K [seed]      # the rule's program for a shape
"""
import random
import sys
from collections import defaultdict

from . import programs

SCHED_ONE, SCHED_STRIDE, SCHED_CLC, SCHED_SPLITK, SCHED_STREAMK = range(5)
RESIDENT_CLUSTERS = 74  # pairs that fit the machine at one CTA an SM


class Violation(Exception):
    pass


class Barrier:
    """An mbarrier: `count` arrivals and a byte count per phase (interp.ml:454-487)."""

    def __init__(self, name, count):
        self.name, self.count = name, count
        self.pending, self.tx, self.phase = count, 0, 0

    def settle(self):
        if self.pending == 0 and self.tx == 0:
            self.phase += 1
            self.pending = self.count

    def arrive(self, tx=0):
        self.tx += tx
        self.pending -= 1
        if self.pending < 0:
            raise Violation("%s: an arrival beyond its %d in phase %d" % (self.name, self.count, self.phase))
        self.settle()

    def complete_tx(self, nbytes):
        self.tx -= nbytes
        self.settle()

    def passed(self, index):
        """Has phase number `index` completed?  A waiter only sees the parity, so the barrier
        being two or more phases past what the waiter means is an error of its own."""
        if self.phase > index + 1:
            raise Violation("%s: a waiter for phase %d finds the barrier in phase %d (parity would alias)" % (self.name, index, self.phase))
        return self.phase > index


class Model:
    def __init__(self, li, m, n, k, seed=0, mutate=None, replicas=0, teardown=None):
        self.li, self.m, self.n, self.k = li, m, n, k
        # when a CTA leaves: "cluster": when every role of every CTA of its cluster is done (a cluster barrier before
        # the exit); "cta": when its own roles are done.  Default: what the kernel that `li` names does.
        self.teardown = teardown or ("cta" if programs.kernel_is_simple(li.kernel_id) else "cluster")
        self.gone = set()
        # further copies of C (wg_plan_set_replicas): the epilogue hands stored tiles to a forwarding warp
        self.replicas = replicas if (not li.direct and li.sched in (SCHED_ONE, SCHED_STRIDE, SCHED_CLC)) else 0
        self.fwd_slot, self.forwarded, self.peer_stored = {}, defaultdict(int), defaultdict(int)
        self.rng = random.Random(seed)
        self.mut = dict(mutate or {})
        self.cg = li.cg
        self.kt = k // 64
        self.tiles = ((m + li.tile_m - 1) // li.tile_m) * ((n + li.tile_n - 1) // li.tile_n)
        self.clusters = li.grid // self.cg
        self.rounds, self.ksub, self.nbuf = li.rounds, li.ksub, li.nbuf
        self.stage_bytes = li.stage_bytes
        self.events = 0
        self.asyncs = []          # callables that complete later: loads landing, commits arriving
        self.commit_queue = defaultdict(list)  # per MMA thread: commits complete in issue order
        self.bars = {}
        self.slots = {}           # (cta, slot) -> None | ("loading"|"full", tile, kstep, bytes_left)
        self.acc = {}             # (cluster, buffer) -> dict(state, tile, ks, readers, complete)
        self.flags = defaultdict(int)
        self.ws = {}              # (CTA, epilogue warp) -> tile whose partial sums that warp has left in the CTA's workspace slot
        self.nbar = defaultdict(set)  # (CTA, use) -> epilogue warps that have reached the named barrier
        self.tile_log = defaultdict(list)  # tile -> [(kind, frozenset(ksteps))]
        self.clc_next = min(self.clusters, RESIDENT_CLUSTERS)  # first cluster not resident at launch
        self.sched_slot = {}
        self.tmem = set()         # CTAs whose tensor memory is allocated (warp 1 of each, after the set-up barrier has its arrival)
        for cta in range(li.grid):
            for r in range(self.rounds):
                self.bars[cta, "full", r] = Barrier("CTA %d full[%d]" % (cta, r), self.mut.get("full_count", 1))
                self.bars[cta, "empty", r] = Barrier("CTA %d empty[%d]" % (cta, r), 1)
            for b in range(2):
                self.bars[cta, "acc_full", b] = Barrier("CTA %d acc_full[%d]" % (cta, b), 1)
                self.bars[cta, "acc_empty", b] = Barrier("CTA %d acc_empty[%d]" % (cta, b), self.mut.get("acc_empty_count", 4 * self.cg))
            for s_ in range(2):
                self.bars[cta, "fwd_full", s_] = Barrier("CTA %d fwd_full[%d]" % (cta, s_), 4)
                self.bars[cta, "fwd_empty", s_] = Barrier("CTA %d fwd_empty[%d]" % (cta, s_), 1)
            self.bars[cta, "tmem_ready", 0] = Barrier("CTA %d tmem_ready" % cta, 1)
            self.bars[cta, "sched_full", 0] = Barrier("CTA %d sched_full" % cta, 1)
            self.bars[cta, "sched_empty", 0] = Barrier("CTA %d sched_empty" % cta, self.cg + 1 + 4 * self.cg)
            for s in range(li.depth):
                self.slots[cta, s] = None
        for c in range(self.clusters):
            for b in range(2):
                self.acc[c, b] = dict(state="free", tile=None, ks=set(), readers=0, complete=False)

    # ------------------------------------------------------------------ the work a CTA walks (Walker)
    def works(self, cta, taker):
        """Yields ('work', tile, kb, ke) items and, for cluster launch control, the waits in between."""
        li, cg, kt = self.li, self.cg, self.kt
        rank, c = cta % cg, cta // cg
        if li.sched == SCHED_SPLITK:
            S = li.split
            s, q, r = c % S, kt // S, kt % S
            yield ("work", (c // S) * cg + rank, s * q + (s * r) // S, (s + 1) * q + ((s + 1) * r) // S, True)
            return
        if li.sched == SCHED_STREAMK:
            # the first sk_dp cluster tiles are walked whole, by stride, after the units of the rest, which are dealt out evenly
            G, dp = self.clusters, li.sk_dp
            units = (self.tiles // cg - dp) * kt
            q, r = units // G, units % G
            b, last = c * q + (c * r) // G, (c + 1) * q + ((c + 1) * r) // G - 1
            if last >= b:
                t_first, kb_first, t_last, ke_last = b // kt, b % kt, last // kt, last % kt + 1
                for seg in range(t_last, t_first - 1, -1):
                    yield ("work", (dp + seg) * cg + rank, kb_first if seg == t_first else 0, ke_last if seg == t_last else kt, seg == t_first and dp == 0)
            whole = list(range(c, dp, G))
            for i, t in enumerate(whole):
                yield ("work", t * cg + rank, 0, kt, i == len(whole) - 1)
            return
        tile = cta
        if tile >= self.tiles:
            return
        if li.sched == SCHED_ONE:
            yield ("work", tile, 0, kt, True)
            return
        if li.sched == SCHED_STRIDE:
            while tile < self.tiles:
                yield ("work", tile, 0, kt, tile + li.grid >= self.tiles)  # the walker knows its last tile
                tile += li.grid
            return
        yield ("work", tile, 0, kt, False)
        index = 0  # cluster launch control: one answer a tile, read by every taker, released on the first CTA
        while True:
            yield ("wait", (cta, "sched_full", 0), index)
            valid, first = self.sched_slot[cta, index]
            yield ("arrive", (c * cg, "sched_empty", 0), 0)
            if not valid:
                return
            yield ("work", first + rank, 0, kt, False)
            index += 1

    # ------------------------------------------------------------------ roles
    def producer(self, cta):
        cg, leader = self.cg, (cta // self.cg) * self.cg
        rnd, use_index = 0, 0  # round of the ring, how often it has gone round
        depth_rounds = self.mut.get("producer_rounds", self.rounds)
        for item in self.works(cta, "producer"):
            if item[0] != "work":
                yield item
                continue
            _, tile, kb, ke, _last = item
            kk = kb
            while kk < ke:
                use = min(self.ksub, ke - kk)
                yield ("wait", (cta, "empty", rnd), use_index - 1)  # the round's previous use has been released
                if cta == leader:
                    yield ("arrive", (leader, "full", rnd), cg * self.stage_bytes * use - self.mut.get("tx_short", 0))
                for g in range(use):
                    slot = rnd * self.ksub + g
                    yield ("load", cta, slot, tile, kk + g, (leader, "full", rnd))
                kk += use
                rnd += 1
                if rnd == depth_rounds:
                    rnd, use_index = 0, use_index + 1
        for _ in range(self.rounds):  # every stage this CTA filled has been released before it leaves
            yield ("wait", (cta, "empty", rnd), use_index - 1)
            rnd += 1
            if rnd == self.rounds:
                rnd, use_index = 0, use_index + 1

    def mma(self, cta):
        cg, c = self.cg, cta // self.cg
        ctas = [c * cg + r for r in range(cg)]
        rnd, use_index, acc, acc_use = 0, 0, 0, 0
        yield ("alloc", cta)   # the issuing warp allocates its own CTA's tensor memory itself
        yield ("tmemwait", cta)
        waited = cg == 1 or bool(self.mut.get("mma_no_tmem_wait"))
        for item in self.works(cta, "mma"):
            if item[0] != "work":
                yield item
                continue
            _, tile, kb, ke, _last = item
            if not waited:   # a pair's MMAs write into both CTAs' tensor memory
                yield ("wait", (cta, "tmem_ready", 0), 0)
                waited = True
            if not self.mut.get("no_acc_empty_wait"):
                yield ("wait", (cta, "acc_empty", acc), acc_use - 1)
            first, kk = True, kb
            while kk < ke:
                use = min(self.ksub, ke - kk)
                yield ("wait", (cta, "full", rnd), use_index)
                for g in range(use):
                    yield ("mma", c, acc, ctas, rnd * self.ksub + g, tile + 0 * g, kk + g, first)
                    first = False
                yield ("commit", cta, [(x, "empty", rnd) for x in ctas], [(x, rnd * self.ksub + g) for x in ctas for g in range(use)], None)
                kk += use
                rnd += 1
                if rnd == self.rounds:
                    rnd, use_index = 0, use_index + 1
            yield ("commit", cta, [(x, "acc_full", acc) for x in ctas], [], (c, acc))
            acc += 1
            if acc == self.nbuf:
                acc, acc_use = 0, acc_use + 1
        for _ in range(0 if self.mut.get("mma_no_final_drain") else self.nbuf):  # every accumulator has been read out in both CTAs before leaving
            yield ("wait", (cta, "acc_empty", acc), acc_use - 1)
            acc += 1
            if acc == self.nbuf:
                acc, acc_use = 0, acc_use + 1

    def allocator(self, cta):
        """Warp 1 of a pair's second CTA: allocates, then tells the leader's MMA lane."""
        yield ("alloc", cta)
        yield ("tmemwait", cta)
        yield ("arrive", (cta - cta % self.cg, "tmem_ready", 0), 0)

    def epilogue(self, cta, warp):
        li, cg, c = self.li, self.cg, cta // self.cg
        leader, rank = c * cg, cta % cg
        acc, acc_use, nth, handed = 0, 0, 0, 0
        if not self.mut.get("epilogue_no_tmem_wait"):
            yield ("tmemwait", cta)   # the named barrier warp 1 arrives at once the CTA's tensor memory exists
        if programs.kernel_is_simple(li.kernel_id) and self.blocks_per_warp() <= 4:
            yield ("rehearse", cta, warp)   # a simple instance's pass through its epilogue on whatever tensor memory holds
        shared_k = (not li.direct) and li.sched in (SCHED_SPLITK, SCHED_STREAMK)
        ws_k = bool(li.direct) and li.sched in (SCHED_SPLITK, SCHED_STREAMK)   # the same sharing through a workspace
        # hand-off words count launches; every epilogue thread reads its CTA's word before any of them
        # moves on (a named barrier in the kernel), so in this first launch they all mean 1
        target = 1 if shared_k else 0
        if shared_k and li.sched == SCHED_STREAMK and warp == 0:
            yield ("flag", ("cta", cta), target)
        for item in self.works(cta, "epilogue"):
            if item[0] != "work":
                yield item
                continue
            _, tile, kb, ke, last = item
            wide = last and li.wide_rows != 0  # the tile is staged in the ring, which has to be drained by then
            if ws_k and li.sched == SCHED_SPLITK:
                # every run leaves its partial in its slot, raises its flag, waits for the tile's other runs' flags, then
                # sums and stores its own share of the tile's blocks (tensor memory is read again: released last)
                S, s = li.split, c % li.split
                base = (c // S) * S
                yield ("wait", (cta, "acc_full", acc), acc_use)
                yield ("peek", c, acc, tile, "partial", warp, cta)
                yield ("nbar", cta, 2 * nth, warp)
                if warp == 0:
                    yield ("flag", ("cta", cta), 1)
                    for j in range(S):
                        if j != s and not self.mut.get("ws_no_flag_wait"):
                            yield ("flagwait", ("cta", (base + j) * cg + rank), 1)
                yield ("nbar", cta, 2 * nth + 1, warp)
                yield ("wsread", tile, [(base + j) * cg + rank for j in range(S) if j != s], warp, cta)
                yield ("share", tile, s, S, warp, cta)
                yield ("read", c, acc, leader, tile, "sum", warp, cta, False)
            elif ws_k and ke < self.kt:
                yield ("wait", (cta, "acc_full", acc), acc_use)
                yield ("read", c, acc, leader, tile, "partial", warp, cta, False)
                yield ("nbar", cta, 2 * nth, warp)
                if warp == 0:
                    yield ("flag", ("cta", cta), 1)
            elif ws_k and kb != 0:
                if warp == 0 and not self.mut.get("ws_no_flag_wait"):
                    yield ("flagwait", ("cta", cta - cg), 1)
                yield ("nbar", cta, 2 * nth, warp)
                if warp == 0:
                    yield ("flag", ("cta", cta - cg), 0)
                yield ("wsread", tile, [cta - cg], warp, cta)
                yield ("wait", (cta, "acc_full", acc), acc_use)
                yield ("read", c, acc, leader, tile, "sum", warp, cta, False)
            elif not shared_k or (li.sched == SCHED_STREAMK and kb == 0 and ke == self.kt):
                # (under stream-K a tile one cluster computes whole has no other part: stored like any tile, no flag)
                yield ("wait", (cta, "acc_full", acc), acc_use)
                yield ("read", c, acc, leader, tile, "store", warp, cta, wide)
                if self.replicas and wide:
                    if warp == 0:
                        yield ("peerstore", tile)        # the last tile, staged whole in the ring: TMA stores to every copy
                elif self.replicas:
                    for ev in self.hand_over(cta, warp, handed, tile):
                        yield ev
                    handed += 1
            elif li.sched == SCHED_SPLITK:
                S, s = li.split, c % li.split
                yield ("zero", tile, s, S, warp, cta)
                yield ("nbar", cta, 2 * nth, warp)   # named barrier of the four epilogue warps
                if warp == 0:
                    yield ("flag", ("cta", cta), target)
                yield ("wait", (cta, "acc_full", acc), acc_use)
                base = (c // S) * S
                if warp == 0:  # the first warp polls the runs' flags, the others meet it at the named barrier
                    for j in range(S):
                        yield ("flagwait", ("cta", (base + j) * cg + rank), target)
                yield ("nbar", cta, 2 * nth + 1, warp)
                yield ("read", c, acc, leader, tile, "add", warp, cta, wide)
            else:
                if kb == 0:
                    yield ("wait", (cta, "acc_full", acc), acc_use)
                    yield ("read", c, acc, leader, tile, "store", warp, cta, wide)
                    yield ("nbar", cta, 2 * nth, warp)   # every warp's stores are complete before the flag goes up
                    if warp == 0:
                        yield ("flag", ("tile", tile), target)
                else:
                    if warp == 0:
                        yield ("flagwait", ("tile", tile), target)
                    yield ("nbar", cta, 2 * nth, warp)
                    yield ("wait", (cta, "acc_full", acc), acc_use)
                    yield ("read", c, acc, leader, tile, "add", warp, cta, wide)
            nth += 1
            acc += 1
            if acc == self.nbuf:
                acc, acc_use = 0, acc_use + 1
        if self.replicas:
            for ev in self.hand_over(cta, warp, handed, None):   # no more tiles: the forwarding warp may leave
                yield ev

    def hand_over(self, cta, warp, count, tile):
        """An epilogue warp's part in handing a stored tile to the forwarding warp (fwd_hand_over): the first warp waits for
        the slot's last use to have been taken and writes the tile into it; all four arrive on the slot's `full` barrier."""
        s, index = count & 1, count >> 1
        if warp == 0:
            if not self.mut.get("fwd_no_empty_wait"):
                yield ("wait", (cta, "fwd_empty", s), index - 1)
            yield ("fwdslot", cta, s, tile)
        yield ("arrive", (cta, "fwd_full", s), 0)

    def forwarder(self, cta):
        taken = 0
        while True:
            s, index = taken & 1, taken >> 1
            yield ("wait", (cta, "fwd_full", s), index)
            tile = self.fwd_slot.get((cta, s), "unset")
            yield ("fwdtake", cta, s)
            yield ("arrive", (cta, "fwd_empty", s), 0)
            if tile is None:
                return
            yield ("fwdcopy", cta, tile)
            for _ in range(self.mut.get("fwd_copy_ticks", 40)):   # the copy crosses NVLink and may take longer than a tile does
                yield ("tick",)
            taken += 1

    def scheduler(self, cta):
        cg = self.cg
        index = 0
        while True:
            yield ("wait", (cta, "sched_empty", 0), index - 1)
            if self.clc_next < self.clusters:
                answer = (True, self.clc_next * cg)
                self.clc_next += 1
            else:
                answer = (False, 0)
            for r in range(cg):
                self.sched_slot[cta + r, index] = answer
                yield ("arrive", (cta + r, "sched_full", 0), 0)
            if not answer[0]:
                return
            index += 1

    # ------------------------------------------------------------------ what the events do
    def step(self, role, ev):
        kind = ev[0]
        self.events += 1
        if kind == "wait":
            _, key, index = ev
            return index < 0 or self.bars[key].passed(index)
        if kind == "flagwait":
            return self.flags[ev[1]] == ev[2]
        if kind == "tmemwait":
            return ev[1] in self.tmem
        if kind == "nbar":
            _, cta, seq, warp = ev
            self.nbar[cta, seq].add(warp)
            return len(self.nbar[cta, seq]) == 4
        if kind == "arrive":
            self.still_here(ev[1][0], "%s arrives on %s" % (role, self.bars[ev[1]].name))
            self.bars[ev[1]].arrive(ev[2])
        elif kind == "flag":
            self.flags[ev[1]] = ev[2]
        elif kind == "alloc":   # tcgen05.alloc returns when the columns are free: at some later time
            self.asyncs.append(lambda cta=ev[1]: self.tmem.add(cta))
        elif kind == "rehearse":
            if ev[1] not in self.tmem:
                raise Violation("CTA %d warp %d rehearses its epilogue on tensor memory that is not allocated yet" % (ev[1], ev[2]))
        elif kind == "load":
            _, cta, slot, tile, kstep, bar = ev
            if self.slots[cta, slot] is not None:
                raise Violation("CTA %d loads k-step %d of tile %d into slot %d, which still holds %r" % (cta, kstep, tile, slot, self.slots[cta, slot]))
            self.slots[cta, slot] = ["loading", tile, kstep]

            def land(cta=cta, slot=slot, bar=bar):
                self.still_here(cta, "a load lands in slot %d of CTA %d" % (slot, cta))
                self.still_here(bar[0], "a load of CTA %d reports its bytes to %s" % (cta, self.bars[bar].name))
                self.slots[cta, slot][0] = "full"
                self.bars[bar].complete_tx(self.stage_bytes)
            self.asyncs.append(land)
        elif kind == "mma":
            _, c, acc, ctas, slot, tile, kstep, first = ev
            for x in ctas:
                self.still_here(x, "cluster %d multiplies k-step %d from CTA %d's ring into its tensor memory" % (c, kstep, x))
                if x not in self.tmem:
                    raise Violation("cluster %d multiplies k-step %d into CTA %d's tensor memory, which is not allocated yet" % (c, kstep, x))
                have = self.slots[x, slot]
                want_tile = tile - tile % self.cg + x % self.cg
                if have is None or have[0] != "full" or have[1] != want_tile or have[2] != kstep:
                    raise Violation("cluster %d multiplies k-step %d of tile %d from slot %d of CTA %d, which holds %r" % (c, kstep, want_tile, slot, x, have))
            a = self.acc[c, acc]
            if first:
                if a["state"] == "live":
                    raise Violation("cluster %d overwrites accumulator %d, which holds tile %r that no load has read" % (c, acc, a["tile"]))
                a.update(state="live", tile=tile - tile % self.cg, ks=set(), readers=0, complete=False)
            elif a["state"] != "live":
                raise Violation("cluster %d adds to accumulator %d, which is %s" % (c, acc, a["state"]))
            if kstep in a["ks"]:
                raise Violation("cluster %d multiplies k-step %d of tile %d twice" % (c, kstep, tile))
            a["ks"].add(kstep)
        elif kind == "commit":
            _, cta, bar_keys, freed, acc_key = ev

            def fire(bar_keys=bar_keys, freed=freed, acc_key=acc_key, cta=cta):
                for key in bar_keys:
                    self.still_here(key[0], "a commit of CTA %d's MMAs reports to %s" % (cta, self.bars[key].name))
                for x, slot in freed:
                    self.slots[x, slot] = None
                if acc_key is not None:
                    self.acc[acc_key]["complete"] = True
                for key in bar_keys:
                    self.bars[key].arrive(0)
            self.commit_queue[cta].append(fire)
        elif kind == "read":
            _, c, acc, leader, tile, how, warp, cta, wide = ev
            if cta not in self.tmem:
                raise Violation("CTA %d warp %d reads tensor memory that is not allocated yet" % (cta, warp))
            if wide:
                busy = [(slot, have) for (x, slot), have in self.slots.items() if x == cta and have is not None]
                if busy:
                    raise Violation("CTA %d stages its last tile %d in the ring while slot %d holds %r" % (cta, tile, busy[0][0], busy[0][1]))
            a = self.acc[c, acc]
            if a["state"] != "live" or not a["complete"] or a["tile"] != tile - tile % self.cg:
                raise Violation("CTA %d warp %d reads accumulator %d for tile %d, which is %s (tile %r, MMAs complete: %s)" % (
                    cta, warp, acc, tile, a["state"], a["tile"], a["complete"]))
            if warp == 0:
                self.tile_log[tile].append((how, frozenset(a["ks"])))
            if how == "partial":
                self.ws[cta, warp] = tile
            a["readers"] += 1
            if a["readers"] == 4 * self.cg:
                a["state"] = "read"
            self.still_here(leader, "CTA %d warp %d releases accumulator %d on the leader's barrier" % (cta, warp, acc))
            self.bars[leader, "acc_empty", acc].arrive(0)
        elif kind == "fwdslot":
            _, cta, s, tile = ev
            if (cta, s) in self.fwd_slot:
                raise Violation("CTA %d puts tile %r into forwarding slot %d, which still holds tile %r the forwarding warp has not taken" % (cta, tile, s, self.fwd_slot[cta, s]))
            self.fwd_slot[cta, s] = tile
        elif kind == "fwdtake":
            _, cta, s = ev
            if (cta, s) not in self.fwd_slot:
                raise Violation("CTA %d's forwarding warp takes slot %d, which nobody has filled" % (cta, s))
            del self.fwd_slot[cta, s]
        elif kind == "fwdcopy":
            _, cta, tile = ev
            if not any(how == "store" for how, _ in self.tile_log.get(tile, [])):
                raise Violation("CTA %d forwards tile %d before it is stored" % (cta, tile))
            self.forwarded[tile] += 1
        elif kind == "peerstore":
            self.peer_stored[ev[1]] += 1
        elif kind in ("zero", "share"):
            _, tile, s, S, warp, cta = ev
            if warp == 0:
                nblk = self.blocks_per_warp()
                self.tile_log[tile].append((kind, frozenset(i for i in range(nblk) if i * S // nblk == s)))
        elif kind == "wsread":
            _, tile, others, warp, cta = ev
            for x in others:
                if self.ws.get((x, warp)) != tile - tile % self.cg + x % self.cg:
                    raise Violation("CTA %d warp %d adds CTA %d's partial sums for tile %d, but that slot holds %r" % (cta, warp, x, tile, self.ws.get((x, warp))))
        elif kind == "peek":   # tensor memory read without giving the accumulator up (its owner reads it again later)
            _, c, acc, tile, how, warp, cta = ev
            self.ws[cta, warp] = tile
            a = self.acc[c, acc]
            if a["state"] != "live" or not a["complete"] or a["tile"] != tile - tile % self.cg:
                raise Violation("CTA %d warp %d reads accumulator %d for tile %d, which is %s (tile %r, MMAs complete: %s)" % (
                    cta, warp, acc, tile, a["state"], a["tile"], a["complete"]))
        return True

    def still_here(self, cta, what):
        if cta in self.gone:
            raise Violation("%s, but CTA %d has left" % (what, cta))

    def role_done(self, cta):
        """A role of `cta` has ended; CTAs whose roles are all done leave (with a cluster barrier before the exit: once the
        whole cluster's are)."""
        self.unfinished[cta] -= 1
        mates = [x for x in range((cta // self.cg) * self.cg, (cta // self.cg + 1) * self.cg) if x in self.unfinished]
        if self.teardown == "cta":
            if self.unfinished[cta] == 0:
                self.gone.add(cta)
        elif all(self.unfinished[x] == 0 for x in mates):
            self.gone.update(mates)

    def blocks_per_warp(self):
        """32-row blocks of C one epilogue warp handles per tile (Cfg::NBLK in gemm_kernel.cuh)."""
        fold = self.cg == 2 and self.li.tile_n == 64
        span = self.li.tile_m // 2 if fold else self.li.tile_m
        return (2 if self.li.tile_n == 256 else 1) * (span // 32)

    # ------------------------------------------------------------------ run
    def run(self):
        roles = []
        # under cluster launch control only the clusters that fit the machine start; the others' tiles are taken by them
        started = self.li.grid if self.li.sched != SCHED_CLC else min(self.clusters, RESIDENT_CLUSTERS) * self.cg
        for cta in range(started):
            leader = cta % self.cg == 0
            roles.append(["CTA %d producer" % cta, self.producer(cta), None, cta])
            if not leader:
                roles.append(["CTA %d warp 1" % cta, self.allocator(cta), None, cta])
            if leader:
                roles.append(["CTA %d MMA issuer" % cta, self.mma(cta), None, cta])
                if self.li.sched == SCHED_CLC:
                    roles.append(["CTA %d scheduler" % cta, self.scheduler(cta), None, cta])
            for w in range(4):
                roles.append(["CTA %d epilogue warp %d" % (cta, w), self.epilogue(cta, w), None, cta])
            if self.replicas:
                roles.append(["CTA %d forwarding warp" % cta, self.forwarder(cta), None, cta])
        self.unfinished = defaultdict(int)
        for role in roles:
            self.unfinished[role[3]] += 1
        live = list(range(len(roles)))
        while live or self.asyncs or any(self.commit_queue.values()):
            progressed = False
            # things in flight complete at arbitrary times: sometimes before, sometimes after the roles move
            if self.asyncs and self.rng.random() < 0.5:
                self.asyncs.pop(self.rng.randrange(len(self.asyncs)))()
                progressed = True
            queues = [q for q in self.commit_queue.values() if q]
            if queues and self.rng.random() < 0.5:
                self.rng.choice(queues).pop(0)()
                progressed = True
            self.rng.shuffle(live)
            still = []
            for i in live:
                role = roles[i]
                moved, turn = 0, self.rng.randint(1, 8)
                while moved < turn:  # a few events at a time (one to eight), so roles interleave at every boundary
                    if role[2] is None:
                        try:
                            role[2] = next(role[1])
                        except StopIteration:
                            role[2] = "done"
                            self.role_done(role[3])
                            break
                    if not self.step(role[0], role[2]):
                        break
                    role[2] = None
                    moved += 1
                progressed = progressed or moved > 0 or role[2] == "done"
                if role[2] != "done":
                    still.append(i)
            live = still
            if not progressed:
                if self.asyncs:
                    self.asyncs.pop(self.rng.randrange(len(self.asyncs)))()
                    continue
                queues = [q for q in self.commit_queue.values() if q]
                if queues:
                    self.rng.choice(queues).pop(0)()
                    continue
                stuck = ["%s at %r" % (roles[i][0], roles[i][2][:3]) for i in live[:6]]
                raise Violation("nothing can move (a hang on the GPU): %d roles wait, e.g. %s" % (len(live), "; ".join(stuck)))
        self.check_end()
        return self.events

    def check_end(self):
        for b in self.bars.values():
            if b.pending != b.count or b.tx != 0:
                raise Violation("%s is left in mid-phase: %d of %d arrivals, %d bytes outstanding" % (b.name, b.count - b.pending, b.count, b.tx))
        for (cta, slot), have in self.slots.items():
            if have is not None:
                raise Violation("CTA %d leaves with slot %d still holding %r" % (cta, slot, have))
        for tile in range(self.tiles):
            log = self.tile_log.get(tile, [])
            pieces = [ks for how, ks in log if how in ("store", "add", "partial", "sum")]
            seen = sorted(k for ks in pieces for k in ks)
            if seen != list(range(self.kt)):
                raise Violation("tile %d: k-steps accumulated %s, wanted each of 0..%d once" % (tile, _ranges(seen), self.kt - 1))
            stores = [how for how, _ in log if how == "store"]
            zeros = sorted(i for how, ks in log if how == "zero" for i in ks)
            if self.li.direct and self.li.sched == SCHED_SPLITK:
                nblk, shares = self.blocks_per_warp(), sorted(i for how, ks in log if how == "share" for i in ks)
                if stores or shares != list(range(nblk)):
                    raise Violation("tile %d: the runs summed and stored blocks %s (wanted each of %d once) and stored it whole %d times" % (tile, shares, nblk, len(stores)))
            elif self.li.direct and self.li.sched == SCHED_STREAMK:
                kinds = [how for how, _ in log]
                if kinds not in (["store"], ["partial", "sum"]):
                    raise Violation("tile %d through the workspace: %s (wanted one store, or a partial left and then summed)" % (tile, kinds))
            elif self.li.sched == SCHED_SPLITK and not self.li.direct:
                nblk = self.blocks_per_warp()
                if stores or zeros != list(range(nblk)):
                    raise Violation("tile %d: split-K zeroed blocks %s (wanted each of %d once) and stored %d times" % (tile, zeros, nblk, len(stores)))
            elif len(stores) != 1:
                raise Violation("tile %d is stored %d times" % (tile, len(stores)))
            elif log[0][0] != "store":
                raise Violation("tile %d is added to before it is stored" % tile)
        if self.replicas:
            for tile in range(self.tiles):
                if self.forwarded[tile] + self.peer_stored[tile] != 1:
                    raise Violation("tile %d reaches the other copies of C %d times" % (tile, self.forwarded[tile] + self.peer_stored[tile]))
            if self.fwd_slot:
                raise Violation("forwarding slots still filled at the end: %r" % self.fwd_slot)
        extra = [t for t in self.tile_log if t >= self.tiles]
        if extra:
            raise Violation("tiles beyond the output were written: %s" % extra[:4])


def _ranges(xs):
    out, i = [], 0
    while i < len(xs):
        j = i
        while j + 1 < len(xs) and xs[j + 1] == xs[j] + 1:
            j += 1
        out.append("%d" % xs[i] if i == j else "%d-%d" % (xs[i], xs[j]))
        i = j + 1
    return ",".join(out) or "none"


def check(variant, m, n, k, seed=0, mutate=None, replicas=0, teardown=None):
    """Run the model for `variant` on an M x N x K problem; returns the number of events, raises
    Violation with the first finding.  `replicas` > 0: with further copies of C (wg_plan_set_replicas).
    `teardown`: "cluster" or "cta" (see the module text); default: what the kernel the variant runs in does."""
    li = programs.realise(variant, m, n, k)
    return Model(li, m, n, k, seed=seed, mutate=mutate, replicas=replicas, teardown=teardown).run()


def main(argv=None):
    args = list(sys.argv[1:] if argv is None else argv)
    if len(args) < 3:
        print(__doc__, file=sys.stderr)
        return 2
    m, n, k = map(int, args[:3])
    seed = int(args[3]) if len(args) > 3 else 0
    v = programs.choose(m, n, k)
    try:
        events = check(v, m, n, k, seed)
    except Violation as e:
        print("protocol: %s" % e)
        return 1
    print("protocol ok: %dx%dx%d, %d events, seed %d" % (m, n, k, events, seed))
    return 0


if __name__ == "__main__":
    sys.exit(main())

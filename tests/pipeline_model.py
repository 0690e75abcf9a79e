"""Host model of the tensor-core kernel's synchronisation protocol (csrc/sgemm_tcgen05.cuh), for checking the
protocol itself — stage/phase parities, barrier counts, who signals whom in a CTA pair — without a GPU.

The reference project verifies its kernel on the CPU with an instruction-level virtual machine
(vm/gcn_virtual_machine.py); an interpreter for compiled sm_100a code is out of reach, so this model restates the
kernel's roles as coroutines over a small mbarrier simulator and lets a seeded random scheduler interleave them:

* ``Mbarrier``   arrival count + transaction bytes + phase bit, ``try_wait(parity)`` as in PTX;
* producer       waits ``empty[s]``, arms ``full[s]`` with the stage bytes, "TMA" completes later and asynchronously;
* transform      (in-kernel split only) waits ``full[s]``, writes the lo tile, arrives on ``ready[s]``;
* MMA issuer     (leader CTA only) waits ``tmem_empty[b]``, then per k-block ``full[s]``/``ready[s]``; its MMAs
                 complete asynchronously and in order, commits fire after them (``empty[s]``, ``tmem_full[b]``, in a
                 pair to both CTAs).  With ``chunk`` > 0 a tile's k-blocks are accumulated in chunks: every chunk
                 starts a fresh accumulator in the next buffer and is handed over on its own;
* epilogue       waits ``tmem_full[b]``, reads the accumulator (adding the chunks of a tile up in chunk order),
                 arrives on the leader's ``tmem_empty[b]``; buffers alternate per hand-over, not per tile.

Shared-memory stages and TMEM buffers carry tags (tile, k-block); every read checks the tag it expects, every
overwrite checks that the previous contents were consumed.  A run fails on a wrong tag, an overwrite of live data, a
barrier that completes a phase twice, or a deadlock (no role can make progress).
"""
from __future__ import annotations

import random
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


class ProtocolError(AssertionError):
    pass


class Mbarrier:
    def __init__(self, count: int, name: str):
        self.count, self.name = count, name
        self.pending, self.tx, self.phase = count, 0, 0

    def _maybe_complete(self):
        if self.pending == 0 and self.tx == 0:
            self.phase ^= 1
            self.pending = self.count

    def arrive(self, tx: int = 0):
        if self.pending <= 0:
            raise ProtocolError(f"{self.name}: more arrivals than its count in one phase")
        self.tx += tx
        self.pending -= 1
        self._maybe_complete()

    def complete_tx(self, nbytes: int):
        self.tx -= nbytes
        self._maybe_complete()

    def try_wait(self, parity: int) -> bool:
        """True once the phase with this parity has completed (a fresh barrier passes parity 1)."""
        return self.phase != parity


@dataclass
class Cta:
    rank: int
    stages: int
    full: List[Mbarrier] = field(default_factory=list)
    empty: List[Mbarrier] = field(default_factory=list)
    ready: List[Mbarrier] = field(default_factory=list)
    tfull: List[Mbarrier] = field(default_factory=list)
    tempty: List[Mbarrier] = field(default_factory=list)
    hi: List[Optional[Tuple[int, int]]] = field(default_factory=list)    # tag of the raw tiles in each stage
    lo: List[Optional[Tuple[int, int]]] = field(default_factory=list)    # tag of the lo tiles
    reads_left: List[int] = field(default_factory=list)                  # MMAs that still have to read the stage
    tmem: List[Optional[Tuple[int, int, int]]] = field(default_factory=list)  # (tile, first k-block, k-blocks accumulated)
    tmem_readers: List[int] = field(default_factory=list)


class Model:
    def __init__(self, tiles: int, kblocks: int, stages: int, cta_group: int = 1, epi_warps: int = 4,
                 inkernel: bool = False, units: int = 2, seed: int = 0, bug: str = "", chunk: int = 0):
        self.tiles, self.kblocks, self.stages = tiles, kblocks, stages
        self.chunk = chunk if chunk > 0 else kblocks      # k-blocks per accumulator hand-over
        self.G, self.E, self.inkernel, self.units, self.bug = cta_group, epi_warps, inkernel, units, bug
        self.rng = random.Random(seed)
        self.pending_async: List = []      # (callable) asynchronous completions (TMA landings, MMA completions)
        self.output: Dict[Tuple[int, int, int], int] = {}   # (tile, cta rank, epilogue warp) -> times written
        self.clusters = []
        for u in range(units):
            ctas = []
            for r in range(cta_group):
                c = Cta(r, stages)
                xf = 4 if inkernel else 1
                for s in range(stages):
                    c.full.append(Mbarrier(1, f"u{u}c{r}.full{s}"))
                    c.empty.append(Mbarrier(1, f"u{u}c{r}.empty{s}"))
                    c.ready.append(Mbarrier(xf * cta_group, f"u{u}c{r}.ready{s}"))
                    c.hi.append(None); c.lo.append(None); c.reads_left.append(0)
                for b in range(2):
                    c.tfull.append(Mbarrier(1, f"u{u}c{r}.tfull{b}"))
                    tempty_count = epi_warps if bug == "tempty_counts_one_cta" else epi_warps * cta_group
                    c.tempty.append(Mbarrier(tempty_count, f"u{u}c{r}.tempty{b}"))
                    c.tmem.append(None); c.tmem_readers.append(0)
                ctas.append(c)
            self.clusters.append(ctas)

    # ------------------------------------------------------------------------------------------------ roles
    def my_tiles(self, unit):
        return range(unit, self.tiles, self.units)

    def producer(self, unit, cta):
        leader = self.clusters[unit][0]
        stage = phase = 0
        for tile in self.my_tiles(unit):
            for kb in range(self.kblocks):
                while not cta.empty[stage].try_wait(phase ^ 1):
                    yield
                if cta.reads_left[stage]:
                    raise ProtocolError(f"producer overwrites stage {stage} that MMAs still read")
                tag = (tile, kb)
                if self.inkernel:   # raw tiles only, reported to this CTA's own barrier
                    cta.full[stage].arrive(tx=1)
                    self.pending_async.append(lambda c=cta, s=stage, t=tag: (c.hi.__setitem__(s, t), c.full[s].complete_tx(1)))
                else:               # four tiles, reported to the leader's barrier; the leader arms it for the pair
                    if cta.rank == 0:
                        leader.full[stage].arrive(tx=self.G)

                    def land(c=cta, s=stage, t=tag):
                        c.hi[s] = t
                        c.lo[s] = t
                        leader.full[s].complete_tx(1)
                    self.pending_async.append(land)
                stage += 1
                if stage == self.stages:
                    stage, phase = 0, phase ^ 1
                yield

    def transform(self, unit, cta, warp):
        leader = self.clusters[unit][0]
        stage = phase = 0
        for tile in self.my_tiles(unit):
            for kb in range(self.kblocks):
                while not cta.full[stage].try_wait(phase):
                    yield
                if cta.hi[stage] != (tile, kb):
                    raise ProtocolError(f"transform reads stage {stage}: {cta.hi[stage]} instead of {(tile, kb)}")
                yield
                cta.lo[stage] = (tile, kb)      # (all four warps write disjoint parts; the tag stands for all)
                leader.ready[stage].arrive()
                stage += 1
                if stage == self.stages:
                    stage, phase = 0, phase ^ 1
                yield

    def chunks_of_tile(self):
        """Chunks of `chunk` k-blocks, the first two twice as long (tc_chunk_span in the kernel)."""
        out, first = [], 0
        while first < self.kblocks:
            span = 2 * self.chunk if first < 4 * self.chunk else self.chunk
            out.append((first, min(self.kblocks, first + span)))
            first += span
        return out

    def mma(self, unit):
        ctas = self.clusters[unit]
        leader = ctas[0]
        stage = phase = 0
        handover = 0
        for tile in self.my_tiles(unit):
            for first, end in self.chunks_of_tile():
                buf, acc_phase = handover & 1, (handover >> 1) & 1
                if self.bug == "buffer_per_tile":
                    local = (tile - unit) // self.units
                    buf, acc_phase = local & 1, (local >> 1) & 1
                while not leader.tempty[buf].try_wait(acc_phase ^ 1):
                    yield
                for c in ctas:
                    if c.tmem_readers[buf]:
                        raise ProtocolError(f"MMA overwrites accumulator {buf} while the epilogue reads it")
                for kb in range(first, end):
                    bar = leader.ready[stage] if self.inkernel else leader.full[stage]
                    while not bar.try_wait(phase):
                        yield
                    for c in ctas:
                        if c.hi[stage] != (tile, kb) or c.lo[stage] != (tile, kb):
                            raise ProtocolError(f"MMA of {(tile, kb)} finds {c.hi[stage]}/{c.lo[stage]} in stage {stage} of CTA {c.rank}")
                        c.reads_left[stage] += 1

                    def done(s=stage, t=tile, k=kb, b=buf, f=first, last=(kb == end - 1)):
                        for c in ctas:      # in-order completion: accumulate, then the commits fire
                            c.reads_left[s] -= 1
                            fresh = k == f   # the first MMA of a chunk overwrites the buffer
                            c.tmem[b] = (t, f, k - f + 1) if (fresh or c.tmem[b] == (t, f, k - f)) else ("corrupt", c.tmem[b], t, k)
                            if self.bug != "no_empty_commit_to_peer" or c.rank == 0:
                                c.empty[s].arrive()
                            if last:
                                c.tfull[b].arrive()
                    self.pending_async.append(("ordered", unit, done))
                    stage += 1
                    if stage == self.stages:
                        stage, phase = 0, phase ^ 1
                    yield
                handover += 1

    def epilogue(self, unit, cta, warp):
        leader = self.clusters[unit][0]
        handover = 0
        for tile in self.my_tiles(unit):
            blocks_summed = 0
            for first, end in self.chunks_of_tile():
                buf, acc_phase = handover & 1, (handover >> 1) & 1
                while not cta.tfull[buf].try_wait(acc_phase):
                    yield
                if cta.tmem[buf] != (tile, first, end - first):
                    raise ProtocolError(f"epilogue of tile {tile} chunk {first} finds {cta.tmem[buf]} in accumulator {buf}")
                cta.tmem_readers[buf] += 1
                yield
                blocks_summed += end - first          # the running sum in registers
                cta.tmem_readers[buf] -= 1
                leader.tempty[buf].arrive()
                handover += 1
                yield
            if blocks_summed != self.kblocks:
                raise ProtocolError(f"tile {tile}: {blocks_summed} of {self.kblocks} k-blocks reached the output")
            key = (tile, cta.rank, warp)
            self.output[key] = self.output.get(key, 0) + 1
            yield

    # -------------------------------------------------------------------------------------------- scheduler
    def run(self, max_steps: int = 2_000_000):
        roles = []
        for u, ctas in enumerate(self.clusters):
            roles.append(self.mma(u))
            for c in ctas:
                roles.append(self.producer(u, c))
                roles += [self.epilogue(u, c, w) for w in range(self.E)]
                if self.inkernel:
                    roles += [self.transform(u, c, w) for w in range(4)]
        idle = 0
        for _ in range(max_steps):
            if not roles and not self.pending_async:
                break
            progressed = False
            # asynchronous completions: TMA landings in any order, MMA completions in issue order per unit
            if self.pending_async and (not roles or self.rng.random() < 0.4):
                i = self.rng.randrange(len(self.pending_async))
                ev = self.pending_async[i]
                if isinstance(ev, tuple):   # the oldest outstanding MMA of that unit goes first
                    i = next(j for j, e in enumerate(self.pending_async) if isinstance(e, tuple) and e[1] == ev[1])
                    ev = self.pending_async[i]
                    ev[2]()
                else:
                    ev()
                del self.pending_async[i]
                progressed = True
            elif roles:
                r = self.rng.choice(roles)
                before = self._state()
                try:
                    next(r)
                except StopIteration:
                    roles.remove(r)
                progressed = self._state() != before or r not in roles
            idle = 0 if progressed else idle + 1
            if idle > 20000:
                raise ProtocolError("deadlock: no role makes progress")
        else:
            raise ProtocolError("did not finish")
        want = {(t, r, w): 1 for t in range(self.tiles) for r in range(self.G) for w in range(self.E)}
        if self.output != want:
            raise ProtocolError("output tiles written: not exactly once each")
        return True

    def _state(self):
        return (len(self.pending_async), sum(len(c.full) for cl in self.clusters for c in cl),
                tuple((b.phase, b.pending, b.tx) for cl in self.clusters for c in cl
                      for b in c.full + c.empty + c.ready + c.tfull + c.tempty),
                len(self.output), tuple(tuple(c.reads_left) + tuple(c.tmem_readers) for cl in self.clusters for c in cl))


# =====================================================================================================================
# The TMA-fed FFMA kernel (csrc/sgemm_ffma_tma.cuh): one block, one tile.
#
# * producer        waits ``empty[s]``, arms ``full[s]``, its two copies land later and asynchronously (A tile; raw B);
# * transposing warps (an untransposed B only) wait ``full[s]``, read the raw buffer, write the B tile, arrive on ``ready[s]``;
# * consumer warps  wait ``full[s]`` (and ``ready[s]``), read the A and B tiles, arrive on ``empty[s]``.
#
# Register hand-over: every scheduler partition holds one warp of the first group and ``consumer_groups`` consumer
# warps, all launched with ``regs_launch`` registers per lane.  ``setmaxnreg.dec`` returns registers to the partition's
# share of the block's allocation, ``setmaxnreg.inc`` waits until that share holds enough — without limit, which is why a
# budget that asks for more than the launch allocation must show up here as a deadlock and not on a GPU.
# =====================================================================================================================
class FfmaModel:
    def __init__(self, steps: int, stages: int, consumer_warps: int = 8, transpose: bool = True, seed: int = 0,
                 bug: str = "", regs_launch: int = 168, regs_small: int = 40, regs_consumer: int = 232, handover: bool = True):
        self.steps, self.stages, self.consumer_warps, self.transpose, self.bug = steps, stages, consumer_warps, transpose, bug
        self.rng = random.Random(seed)
        self.full = [Mbarrier(1, f"full{s}") for s in range(stages)]
        self.ready = [Mbarrier(3, f"ready{s}") for s in range(stages)]
        self.empty = [Mbarrier(consumer_warps - (1 if bug == "empty_count_short" else 0), f"empty{s}") for s in range(stages)]
        self.a_tile: List[Optional[int]] = [None] * stages      # step whose data the buffer holds
        self.raw: List[Optional[int]] = [None] * stages
        self.b_tile: List[Optional[int]] = [None] * stages
        self.xform_parts: List[int] = [0] * stages               # transposing warps that have written their part
        self.readers: List[int] = [0] * stages                   # consumer warps inside the stage
        self.xform_readers: List[int] = [0] * stages
        self.pending_async: List = []
        self.consumed = [0] * consumer_warps
        # registers per lane in one scheduler partition: one warp of the first group + consumer_warps / 4 consumer warps
        self.handover = handover
        self.regs_launch, self.regs_small, self.regs_consumer = regs_launch, regs_small, regs_consumer
        self.free_regs = 0                                        # released and not yet taken (the launch allocation is all in use)

    # ------------------------------------------------------------------------------------------------ roles
    def first_group_warp(self, role):
        """A warp of the first group: shrink, then its role."""
        if self.handover:
            self.free_regs += self.regs_launch - self.regs_small
            yield
        yield from role

    def consumer_warp(self, w):
        if self.handover:
            need = self.regs_consumer - self.regs_launch
            while self.free_regs < need:                          # setmaxnreg.inc: no limit on this wait
                yield
            self.free_regs -= need
            yield
        yield from self.consumer(w)

    def producer(self):
        for t in range(self.steps):
            s, rnd = t % self.stages, t // self.stages
            while not self.empty[s].try_wait((rnd & 1) ^ 1):
                yield
            if self.readers[s] or self.xform_readers[s]:
                raise ProtocolError(f"producer refills stage {s} while it is being read")
            self.full[s].arrive(tx=2)

            def land_a(s=s, t=t):
                self.a_tile[s] = t
                self.full[s].complete_tx(1)

            def land_b(s=s, t=t):
                if self.transpose:
                    self.raw[s] = t
                else:
                    self.b_tile[s] = t
                self.full[s].complete_tx(1)
            self.pending_async += [land_a, land_b]
            yield

    def transposer(self, w):
        for t in range(self.steps):
            s, rnd = t % self.stages, t // self.stages
            while not self.full[s].try_wait(rnd & 1):
                yield
            if self.raw[s] != t:
                raise ProtocolError(f"transposing warp {w} finds step {self.raw[s]} in the raw buffer of stage {s}, wants {t}")
            if self.readers[s]:
                raise ProtocolError(f"transposing warp {w} rewrites the B tile of stage {s} while consumers read it")
            self.xform_readers[s] += 1
            yield
            self.xform_readers[s] -= 1
            self.xform_parts[s] += 1
            if self.xform_parts[s] == 3:
                self.b_tile[s], self.xform_parts[s] = t, 0
            self.ready[s].arrive()
            yield

    def consumer(self, w):
        for t in range(self.steps):
            s, rnd = t % self.stages, t // self.stages
            while not self.full[s].try_wait(rnd & 1):
                yield
            if self.transpose and self.bug != "ready_not_waited":
                while not self.ready[s].try_wait(rnd & 1):
                    yield
            if self.a_tile[s] != t or self.b_tile[s] != t:
                raise ProtocolError(f"consumer warp {w}, step {t}: stage {s} holds A of {self.a_tile[s]}, B of {self.b_tile[s]}")
            self.readers[s] += 1
            yield
            self.readers[s] -= 1
            self.consumed[w] += 1
            self.empty[s].arrive()
            yield

    # -------------------------------------------------------------------------------------------- scheduler
    def run(self, max_steps: int = 1_000_000):
        roles = [self.first_group_warp(self.producer())]
        roles += [self.first_group_warp(self.transposer(w) if self.transpose else iter(())) for w in range(3)]
        # (registers are pooled over the four scheduler partitions here: each holds one warp of the first group and
        # consumer_warps / 4 consumer warps, so the sums scale alike and the block-wide balance is the partition's)
        roles += [self.consumer_warp(w) for w in range(self.consumer_warps)]
        idle = 0
        for _ in range(max_steps):
            if not roles and not self.pending_async:
                break
            progressed = False
            if self.pending_async and (not roles or self.rng.random() < 0.4):
                self.pending_async.pop(self.rng.randrange(len(self.pending_async)))()
                progressed = True
            elif roles:
                r = self.rng.choice(roles)
                before = self._state()
                try:
                    next(r)
                except StopIteration:
                    roles.remove(r)
                progressed = self._state() != before or r not in roles
            idle = 0 if progressed else idle + 1
            if idle > 20000:
                raise ProtocolError("deadlock: no role makes progress")
        else:
            raise ProtocolError("did not finish")
        if self.consumed != [self.steps] * self.consumer_warps:
            raise ProtocolError("not every consumer warp multiplied every step exactly once")
        return True

    def _state(self):
        return (len(self.pending_async), self.free_regs, tuple(self.consumed), tuple(self.readers), tuple(self.xform_readers),
                tuple((b.phase, b.pending, b.tx) for b in self.full + self.ready + self.empty))

"""A CPU model of the barrier protocol of the GEMM kernels (hipkittensp_b200/csrc/gemm_kernel.cuh): the mbarriers,
their phase parities, and the wait / arrive sequence of each warp role, written with the same index arithmetic as
the kernel (stage = n % STAGES, parity = (n / STAGES) & 1, groups of 4 K-blocks per scale slab, two accumulators).
The roles run as coroutines under a seeded random scheduler, so any interleaving the hardware could produce is a
possible trace.  The model checks what the protocol has to guarantee:

  * every role finishes (no deadlock) for any number of tiles / K-blocks / ring depths;
  * a stage is consumed by the MMA only when it holds the K-block the MMA expects, and is never refilled before the
    MMA that read it has completed;
  * scale atoms are consumed only when they belong to the current group of K-blocks, an accumulator is never
    re-used before the epilogue has drained it;
  * when an arrival is withheld, the role that depends on it reports a wait that ran out, with the role code the
    kernel would write to its status word, and every other role still ends (bounded waits), never hangs.

Test infrastructure only: nothing of the product imports it.
"""
from __future__ import annotations

import random

# role codes of the device status word (gemm_kernel.cuh: kStatusTimeout*)
PRODUCER, MMA, SCALE, EPILOGUE = 1, 2, 3, 4


class MBarrier:
    """mbarrier with an arrival count: the phase completes when `count` arrivals have been made."""

    def __init__(self, name, count=1):
        self.name, self.count, self.pending, self.phase = name, count, count, 0

    def arrive(self):
        self.pending -= 1
        assert self.pending >= 0, f"{self.name}: more arrivals than the barrier expects"
        if self.pending == 0:
            self.pending, self.phase = self.count, self.phase + 1

    def done(self, parity):
        """mbarrier.try_wait.parity: true once the phase with this parity has completed."""
        return (self.phase & 1) != parity


class Timeout(Exception):
    def __init__(self, role):
        self.role = role


class Pipeline:
    def __init__(self, tiles, kblocks, stages=4, raw_slots=2, atom_groups=3, drop=None, seed=0, wait_budget=20000):
        self.tiles, self.kblocks, self.S, self.R, self.G = tiles, kblocks, stages, raw_slots, atom_groups
        self.drop = drop                      # (barrier name, n-th arrival) that is withheld
        self.rng = random.Random(seed)
        self.wait_budget = wait_budget
        mk = lambda n, c=1: MBarrier(n, c)
        self.full = [mk(f"full{s}") for s in range(stages)]
        self.empty = [mk(f"empty{s}") for s in range(stages)]
        self.raw_full = [mk(f"raw_full{r}") for r in range(raw_slots)]
        self.raw_empty = [mk(f"raw_empty{r}") for r in range(raw_slots)]
        self.atom_full = [mk(f"atom_full{g}") for g in range(atom_groups)]
        self.atom_empty = [mk(f"atom_empty{g}") for g in range(atom_groups)]
        self.acc_full = [mk("acc_full0"), mk("acc_full1")]
        self.acc_empty = [mk("acc_empty0"), mk("acc_empty1")]
        self.arrivals = {}
        # contents, for the invariants
        self.stage_tag = [None] * stages      # (tile, kb) a stage holds; None while the MMA may still be reading an old one
        self.raw_tag = [None] * raw_slots
        self.atom_tag = [None] * atom_groups
        self.acc_state = ["free", "free"]     # free -> accumulating -> complete -> free
        self.status = 0
        self.abort = False
        self.finished = set()

    # ---- primitives the roles yield
    def _arrive(self, bar):
        n = self.arrivals.get(bar.name, 0)
        self.arrivals[bar.name] = n + 1
        if self.drop == (bar.name, n):
            return                              # the withheld arrival
        bar.arrive()

    def _wait(self, bar, parity, role):
        spins = 0
        while not bar.done(parity):
            if self.abort:
                raise Timeout(role)
            spins += 1
            if spins > self.wait_budget:        # the bounded wait of the kernel: record the role, raise the abort flag
                if self.status == 0:
                    self.status = role
                self.abort = True
                raise Timeout(role)
            yield

    # ---- roles (same loops and index arithmetic as the kernel)
    def producer(self):
        n_stage = n_raw = 0
        for tile in range(self.tiles):
            for kb in range(self.kblocks):
                if kb % 4 == 0:
                    r, ph = n_raw % self.R, (n_raw // self.R) & 1
                    yield from self._wait(self.raw_empty[r], ph ^ 1, PRODUCER)
                    assert self.raw_tag[r] is None, "scale slab overwritten before the scale warp read it"
                    self.raw_tag[r] = (tile, kb // 4)
                    self._arrive(self.raw_full[r])              # TMA completion of the slab
                    n_raw += 1
                s, ph = n_stage % self.S, (n_stage // self.S) & 1
                yield from self._wait(self.empty[s], ph ^ 1, PRODUCER)
                assert self.stage_tag[s] is None, "operand stage refilled while the MMA may still read it"
                self.stage_tag[s] = (tile, kb)
                yield                                           # the copy is in flight
                self._arrive(self.full[s])                      # TMA completion (expect_tx satisfied)
                n_stage += 1

    def scale_warps(self):
        n_grp = 0
        for tile in range(self.tiles):
            for grp in range((self.kblocks + 3) // 4):
                r = n_grp % self.R
                yield from self._wait(self.raw_full[r], (n_grp // self.R) & 1, SCALE)
                assert self.raw_tag[r] == (tile, grp), "scale warp read a slab of another group"
                self.raw_tag[r] = None
                self._arrive(self.raw_empty[r])
                g = n_grp % self.G
                yield from self._wait(self.atom_empty[g], ((n_grp // self.G) & 1) ^ 1, SCALE)
                assert self.atom_tag[g] is None, "scale atoms overwritten before the MMA used them"
                self.atom_tag[g] = (tile, grp)
                self._arrive(self.atom_full[g])
                n_grp += 1

    def mma(self):
        n_kb = n_seg = n_grp = 0
        for tile in range(self.tiles):
            b = n_seg & 1
            yield from self._wait(self.acc_empty[b], ((n_seg >> 1) & 1) ^ 1, MMA)
            assert self.acc_state[b] == "free", "accumulator re-used before the epilogue drained it"
            self.acc_state[b] = "accumulating"
            for kb in range(self.kblocks):
                s, g = n_kb % self.S, n_grp % self.G
                if kb % 4 == 0:
                    yield from self._wait(self.atom_full[g], (n_grp // self.G) & 1, MMA)
                    assert self.atom_tag[g] == (tile, kb // 4), "MMA used the scale atoms of another group"
                yield from self._wait(self.full[s], (n_kb // self.S) & 1, MMA)
                assert self.stage_tag[s] == (tile, kb), "MMA consumed a stage that holds another K-block"
                yield                                           # the MMAs of this K-block execute
                self.stage_tag[s] = None
                self._arrive(self.empty[s])                     # tcgen05.commit
                group_done = kb % 4 == 3 or kb == self.kblocks - 1
                if group_done:
                    self.atom_tag[g] = None
                    self._arrive(self.atom_empty[g])
                    n_grp += 1
                n_kb += 1
            self.acc_state[b] = "complete"
            self._arrive(self.acc_full[b])
            n_seg += 1

    def epilogue(self):
        for n_seg in range(self.tiles):
            b = n_seg & 1
            yield from self._wait(self.acc_full[b], (n_seg >> 1) & 1, EPILOGUE)
            assert self.acc_state[b] == "complete", "epilogue read an accumulator that is not complete"
            yield                                               # TMEM loads and stores
            self.acc_state[b] = "free"
            self._arrive(self.acc_empty[b])

    # ---- scheduler
    def run(self, max_steps=5_000_000):
        roles = {"producer": self.producer(), "scale": self.scale_warps(), "mma": self.mma(), "epilogue": self.epilogue()}
        timed_out = {}
        steps = 0
        while roles:
            steps += 1
            assert steps < max_steps, f"no progress: roles {sorted(roles)} never finished (deadlock)"
            name = self.rng.choice(sorted(roles))
            try:
                next(roles[name])
            except StopIteration:
                self.finished.add(name)
                del roles[name]
            except Timeout as t:
                timed_out[name] = t.role
                del roles[name]
        return timed_out

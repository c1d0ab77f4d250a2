"""A host-side model of the mbarrier protocol inside one CTA of csrc/bwd_sm100.cu, run to
completion under random interleavings.

The kernel's roles (TMA producer, MMA issuer, two compute warpgroups, and at head dim 128 the
dQ^T drain warpgroup) hand tiles to each other through 16 mbarriers whose waits carry a single
phase bit.  A wait with the wrong parity, a barrier that completes twice before its waiter has
looked, or a buffer that is rewritten while the tensor pipe still reads it would show on the
GPU as a hang or as wrong gradients for some timings only.  This file restates, role by role,
which barrier each step waits for (with which parity) and arrives on, which buffer it reads
and writes, and that the MMAs run asynchronously and in issue order on one tensor pipe; it
then advances the roles in random order and checks that

* nothing deadlocks,
* every read finds the tile it expects (a tag written with the data),
* no buffer is written while a reader of its previous contents has not finished.

The buffers: shared memory K/V, Q[2] (with the per-row terms of the stage), dO[2], dS; tensor
memory S/P (P^T overlays S^T), dP/dQ (dQ^T overlays dP^T), dK+dV.
Mutations of the protocol (a wait left out, a parity inverted) must fail: that is what shows
the model can see such faults.  One wait that an earlier kernel had is absent on purpose: the
compute warpgroups do not wait for the MMAs that read dS^T of the previous tile before they
overwrite it, because dP^T of the current tile was issued behind those MMAs and its commit
covers them (in-order tensor pipe); the model shows no overwrite under a reader.
"""
import random

import pytest


class Barrier:
    """mbarrier with `count` arrivals per phase; `phase` = parity of the phase in progress."""

    def __init__(self, count):
        self.count, self.pending, self.phase = count, count, 0

    def arrive(self):
        self.pending -= 1
        assert self.pending >= 0
        if self.pending == 0:
            self.pending, self.phase = self.count, self.phase ^ 1

    def done(self, parity):  # try_wait.parity: has the phase with this parity completed?
        return self.phase != parity


class Buffer:
    def __init__(self, name):
        self.name, self.tag, self.readers = name, None, 0

    def write(self, tag):
        assert self.readers == 0, f"{self.name}: written ({tag}) while {self.readers} reader(s) of {self.tag} are active"
        self.tag = tag

    def begin_read(self, want):
        assert self.tag == want, f"{self.name}: holds {self.tag}, reader expected {want}"
        self.readers += 1

    def end_read(self):
        self.readers -= 1


class Cta:
    """One CTA walking `tiles` query tiles.  drain=True: head dim 128 (a drain warpgroup);
    drain=False: head dim 64 (the compute warpgroups drain dQ themselves)."""

    def __init__(self, tiles, drain, rng, mutate=None):
        self.T, self.drain, self.rng, self.mutate = tiles, drain, rng, mutate
        wg = 2  # compute warpgroups; each arrives once where the kernel has 128 thread arrivals
        names = ["KV_FULL", "Q_FULL0", "Q_FULL1", "Q_EMPTY0", "Q_EMPTY1", "DO_FULL0", "DO_FULL1", "DO_EMPTY0",
                 "DO_EMPTY1", "S_FULL", "DP_FULL", "P_READY", "DS_READY", "DQ_FULL", "DQ_DRAINED",
                 "DKDV_FULL"]
        self.bar = {n: Barrier(1) for n in names}
        self.bar["P_READY"] = Barrier(wg)
        self.bar["DS_READY"] = Barrier(wg)
        self.bar["DQ_DRAINED"] = Barrier(1 if drain else wg)
        self.buf = {n: Buffer(n) for n in ["KV", "Q0", "Q1", "dO0", "dO1", "dS", "S", "dP", "dKdV"]}
        self.pipe = []      # tensor pipe: MMAs and commits, executed in issue order
        self.loads = []     # TMA loads in flight: complete in any order
        self.dkdv_tiles = 0

    # ---- the asynchronous units -------------------------------------------------------
    def run_pipe(self):
        """Generator: executes queued MMAs one at a time, in order; a commit arrives when
        everything issued before it has completed (which in-order execution implies)."""
        while True:
            if not self.pipe:
                yield "idle"
                continue
            op = self.pipe.pop(0)
            if op[0] == "commit":
                self.bar[op[1]].arrive()
                yield "ran"
                continue
            _, reads, writes = op
            for name, tag in reads:
                self.buf[name].begin_read(tag)
            yield "ran"  # the MMA is executing: other roles run meanwhile
            for name, _ in reads:
                self.buf[name].end_read()
            for name, tag in writes:
                if name == "dKdV":
                    self.dkdv_tiles += 1
                else:
                    self.buf[name].write(tag)
            yield "ran"

    def run_loads(self):
        while True:
            if not self.loads:
                yield "idle"
                continue
            name, tag, bar = self.loads.pop(self.rng.randrange(len(self.loads)))
            self.buf[name].write(tag)
            self.bar[bar].arrive()
            yield "ran"

    def wait(self, name, parity):
        while not self.bar[name].done(parity):
            yield "blocked"

    # ---- roles ------------------------------------------------------------------------
    def producer(self):
        self.loads.append(("KV", "KV", "KV_FULL"))
        yield "ran"
        # two independently polled streams: Q (with the row terms) and dO
        qn = don = 0
        while qn < self.T or don < self.T:
            progressed = False
            if qn < self.T and self.bar[f"Q_EMPTY{qn & 1}"].done(((qn >> 1) & 1) ^ 1):
                self.loads.append((f"Q{qn & 1}", ("Q", qn), f"Q_FULL{qn & 1}"))
                qn += 1
                progressed = True
            if don < self.T and self.bar[f"DO_EMPTY{don % 2}"].done(((don // 2) & 1) ^ 1):
                self.loads.append((f"dO{don % 2}", ("dO", don), f"DO_FULL{don % 2}"))
                don += 1
                progressed = True
            yield "ran" if progressed else "blocked"

    def issue(self, reads, writes):
        self.pipe.append(("mma", reads, writes))

    def commit(self, name):
        self.pipe.append(("commit", name))

    def mma(self):
        T = self.T

        def s(n):
            self.issue([("KV", "KV"), (f"Q{n & 1}", ("Q", n))], [("S", ("S", n))])
            self.commit("S_FULL")

        def dp(n):
            self.issue([("KV", "KV"), (f"dO{n % 2}", ("dO", n))], [("dP", ("dP", n))])
            self.commit("DP_FULL")

        def dv(n):
            self.issue([("S", ("P", n)), (f"dO{n % 2}", ("dO", n))], [("dKdV", n)])

        yield from self.wait("KV_FULL", 0)
        yield from self.wait("Q_FULL0", 0)
        yield from self.wait("DO_FULL0", 0)
        s(0)
        dp(0)
        yield "ran"
        yield from self.wait("P_READY", 0)
        dv(0)
        self.commit("DO_EMPTY0")
        yield "ran"
        for n in range(T):
            par, has_next = n & 1, n + 1 < T
            if has_next:
                yield from self.wait(f"Q_FULL{(n + 1) & 1}", ((n + 1) >> 1) & 1)
                s(n + 1)
                yield "ran"
            yield from self.wait("DS_READY", par)
            self.issue([("KV", "KV"), ("dS", ("dS", n))], [("dP", ("dQ", n))])
            self.commit("DQ_FULL")
            self.issue([("dS", ("dS", n)), (f"Q{n & 1}", ("Q", n))], [("dKdV", n)])
            self.commit(f"Q_EMPTY{n & 1}")
            yield "ran"
            if not has_next:
                break
            if self.mutate != "no_drained_wait":
                yield from self.wait("DQ_DRAINED", par)
            yield from self.wait(f"DO_FULL{(n + 1) % 2}", ((n + 1) // 2) & 1)
            dp(n + 1)
            yield "ran"
            if self.mutate != "no_p_ready_wait":
                yield from self.wait("P_READY", par ^ 1)
            dv(n + 1)
            self.commit(f"DO_EMPTY{(n + 1) % 2}")
            yield "ran"
        self.commit("DKDV_FULL")
        yield "ran"

    def read(self, name, tag):
        """A warpgroup's read of a buffer: other roles may run while it is in progress."""
        self.buf[name].begin_read(tag)
        yield "ran"
        self.buf[name].end_read()

    def compute(self, g):
        """One compute warpgroup: step k forms dS^T(k-1), then P^T(k) (then, at head dim 64,
        drains dQ(k-1)).  Buffer writes shared by the two warpgroups (dS, P^T) are modelled
        as done by the warpgroup that arrives last on the barrier."""
        T = self.T
        for k in range(T + 1):
            if k > 0:
                n = k - 1
                yield from self.wait("DP_FULL", (n & 1) ^ (1 if self.mutate == "dp_full_parity" else 0))
                yield from self.read("dP", ("dP", n))
                yield from self.read(f"Q{n & 1}", ("Q", n))  # -delta * scale of the tile's rows
                if self.bar["DS_READY"].pending == 1:
                    self.buf["dS"].write(("dS", n))
                else:
                    assert self.buf["dS"].readers == 0, f"dS: warpgroup {g} writes tile {n} under a reader"
                self.bar["DS_READY"].arrive()
                yield "ran"
            if k < T:
                n = k
                yield from self.wait(f"Q_FULL{n & 1}", (n >> 1) & 1)
                yield from self.wait("S_FULL", n & 1)
                yield from self.read("S", ("S", n))
                yield from self.read(f"Q{n & 1}", ("Q", n))  # -L * log2(e) of the tile's rows
                if self.bar["P_READY"].pending == 1:
                    self.buf["S"].write(("P", n))
                self.bar["P_READY"].arrive()
                yield "ran"
            if k > 0 and not self.drain:
                n = k - 1
                yield from self.wait("DQ_FULL", n & 1)
                yield from self.read("dP", ("dQ", n))
                self.bar["DQ_DRAINED"].arrive()
                yield "ran"
        yield from self.wait("DKDV_FULL", 0)
        assert self.dkdv_tiles == 2 * T, (self.dkdv_tiles, T)

    def drain_wg(self):
        for n in range(self.T):
            yield from self.wait("DQ_FULL", n & 1)
            yield from self.read("dP", ("dQ", n))
            self.bar["DQ_DRAINED"].arrive()
            yield "ran"


def run(tiles, drain, seed, mutate=None, max_steps=200000):
    rng = random.Random(seed)
    cta = Cta(tiles, drain, rng, mutate)
    roles = {"producer": cta.producer(), "mma": cta.mma(), "compute0": cta.compute(0), "compute1": cta.compute(1)}
    if drain:
        roles["drain"] = cta.drain_wg()
    units = {"pipe": cta.run_pipe(), "loads": cta.run_loads()}
    live = dict(roles)
    # speeds differ per run: in some runs a role or a unit is ten times slower than the others
    weight = {n: rng.choice([1, 1, 3, 10]) for n in list(roles) + list(units)}
    stuck = set()  # roles and units that could not move since anything last moved
    for _ in range(max_steps):
        if not live:
            break
        names = list(live) + list(units)
        name = rng.choices(names, weights=[weight[n] for n in names])[0]
        gen = live.get(name) or units[name]
        try:
            state = next(gen)
        except StopIteration:
            del live[name]
            stuck.clear()
            continue
        if state == "ran":
            stuck.clear()
        else:
            stuck.add(name)
            if stuck >= set(names):  # every role waits and both units are empty
                raise AssertionError(f"deadlock: {sorted(live)} still waiting; "
                                     f"{ {n: (b.phase, b.pending) for n, b in cta.bar.items()} }")
    assert not live, f"did not finish: {sorted(live)}"
    assert not cta.pipe and not cta.loads


@pytest.mark.parametrize("drain", [True, False], ids=["head_dim_128", "head_dim_64"])
@pytest.mark.parametrize("tiles", [1, 2, 3, 4, 5, 9])
def test_protocol_completes_under_random_interleavings(tiles, drain):
    for seed in range(60):
        run(tiles, drain, seed)


@pytest.mark.parametrize("mutate", ["no_drained_wait", "dp_full_parity", "no_p_ready_wait"])
def test_model_sees_protocol_faults(mutate):
    failures = 0
    for seed in range(40):
        try:
            run(6, True, seed, mutate)
        except AssertionError:
            failures += 1
    assert failures >= 10, f"{mutate}: only {failures} of 40 runs failed"

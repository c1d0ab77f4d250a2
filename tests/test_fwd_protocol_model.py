"""A host-side model of the mbarrier protocol inside one CTA of csrc/fwd_sm100.cu, run to
completion under random interleavings (the forward counterpart of
test_bwd_protocol_model.py, whose barrier and buffer models it uses).

Roles: the TMA producer (Q tiles once, then K and V of every visited K/V tile through two
stages each), the MMA issuer (S = Q K^T for both query tiles of the CTA, O += P V), one
softmax warpgroup per query tile.  The tensor pipe executes in issue order, so a commit
covers everything issued before it: the softmax of step i may rescale O because S(i) was
issued behind P V of step i-1 -- there is no barrier of its own for that, and the model checks
that no rescale lands under a running P V.
"""
import random

import pytest

from tests.test_bwd_protocol_model import Barrier, Buffer


class FwdCta:
    def __init__(self, steps, ntile, rng, mutate=None):
        self.n, self.ntile, self.rng, self.mutate = steps, ntile, rng, mutate
        names = ["K_FULL0", "K_FULL1", "K_EMPTY0", "K_EMPTY1", "V_FULL0", "V_FULL1", "V_EMPTY0", "V_EMPTY1", "O_FULL"]
        for t in range(ntile):
            names += [f"Q_FULL{t}", f"S_FULL{t}", f"P_FULL{t}"]
        self.bar = {n: Barrier(1) for n in names}
        bufs = ["K0", "K1", "V0", "V1"] + [f"{x}{t}" for t in range(ntile) for x in ("Q", "S", "O")]
        self.buf = {n: Buffer(n) for n in bufs}
        for t in range(ntile):
            self.buf[f"O{t}"].tag = ("O", t, -1)
        self.pipe, self.loads = [], []

    def run_pipe(self):
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
            yield "ran"
            for name, _ in reads:
                self.buf[name].end_read()
            for name, tag in writes:
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

    def producer(self):
        for t in range(self.ntile):
            self.loads.append((f"Q{t}", ("Q", t), f"Q_FULL{t}"))
        yield "ran"
        for i in range(self.n):
            s, ph = i & 1, (i >> 1) & 1
            if self.mutate != "no_k_empty_wait":
                yield from self.wait(f"K_EMPTY{s}", ph ^ 1)
            self.loads.append((f"K{s}", ("K", i), f"K_FULL{s}"))
            yield "ran"
            yield from self.wait(f"V_EMPTY{s}", ph ^ 1)
            self.loads.append((f"V{s}", ("V", i), f"V_FULL{s}"))
            yield "ran"

    def mma(self):
        n, ntile = self.n, self.ntile

        def issue_s(t, i):
            self.pipe.append(("mma", [(f"Q{t}", ("Q", t)), (f"K{i & 1}", ("K", i))], [(f"S{t}", ("S", t, i))]))
            self.pipe.append(("commit", f"S_FULL{t}"))

        def issue_pv(t, i):
            # accumulates into O: it reads the O that the softmax of this step left, and writes
            self.pipe.append(("mma", [(f"S{t}", ("P", t, i)), (f"V{i & 1}", ("V", i)), (f"O{t}", ("O", t, i - 1))],
                              [(f"O{t}", ("O", t, i))]))

        for t in range(ntile):
            yield from self.wait(f"Q_FULL{t}", 0)
        yield from self.wait("K_FULL0", 0)
        for t in range(ntile):
            issue_s(t, 0)
        self.pipe.append(("commit", "K_EMPTY0"))
        yield "ran"
        for i in range(n):
            s, sn, ph, phn = i & 1, (i + 1) & 1, (i >> 1) & 1, ((i + 1) >> 1) & 1
            has_next = i + 1 < n
            if has_next:
                yield from self.wait(f"K_FULL{sn}", phn)
            yield from self.wait(f"V_FULL{s}", ph)
            for t in range(ntile):
                if self.mutate != "no_p_full_wait":
                    yield from self.wait(f"P_FULL{t}", i & 1)
                issue_pv(t, i)
                if t == ntile - 1:
                    self.pipe.append(("commit", f"V_EMPTY{s}"))
                if has_next:
                    issue_s(t, i + 1)
                    if t == ntile - 1:
                        self.pipe.append(("commit", f"K_EMPTY{sn}"))
                yield "ran"
        self.pipe.append(("commit", "O_FULL"))
        yield "ran"

    def softmax(self, t):
        for i in range(self.n):
            par = (i & 1) ^ (1 if self.mutate == "s_full_parity" else 0)
            yield from self.wait(f"S_FULL{t}", par)
            self.buf[f"S{t}"].begin_read(("S", t, i))
            yield "ran"
            self.buf[f"S{t}"].end_read()
            # rescale of O (in the kernel only when the row max grew enough; here always): the
            # tile must hold P V of every earlier step and no P V may be running on it
            o = self.buf[f"O{t}"]
            assert o.tag == ("O", t, i - 1), f"O{t}: rescale at step {i} finds {o.tag}"
            o.write(("O", t, i - 1))
            self.buf[f"S{t}"].write(("P", t, i))
            self.bar[f"P_FULL{t}"].arrive()
            yield "ran"
        yield from self.wait("O_FULL", 0)
        assert self.buf[f"O{t}"].tag == ("O", t, self.n - 1)


def run(steps, ntile, seed, mutate=None, max_steps=200000):
    rng = random.Random(seed)
    cta = FwdCta(steps, ntile, rng, mutate)
    roles = {"producer": cta.producer(), "mma": cta.mma()}
    for t in range(ntile):
        roles[f"softmax{t}"] = cta.softmax(t)
    units = {"pipe": cta.run_pipe(), "loads": cta.run_loads()}
    weight = {n: rng.choice([1, 1, 3, 10]) for n in list(roles) + list(units)}
    live = dict(roles)
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
                raise AssertionError(f"deadlock: {sorted(live)} still waiting")
    assert not live, f"did not finish: {sorted(live)}"
    assert not cta.pipe and not cta.loads


@pytest.mark.parametrize("ntile", [1, 2])
@pytest.mark.parametrize("steps", [1, 2, 3, 4, 7])
def test_protocol_completes_under_random_interleavings(steps, ntile):
    for seed in range(60):
        run(steps, ntile, seed)


@pytest.mark.parametrize("mutate", ["no_k_empty_wait", "no_p_full_wait", "s_full_parity"])
def test_model_sees_protocol_faults(mutate):
    failures = 0
    for seed in range(40):
        try:
            run(6, 2, seed, mutate)
        except AssertionError:
            failures += 1
    assert failures >= 10, f"{mutate}: only {failures} of 40 runs failed"

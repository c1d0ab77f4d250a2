"""A host-side model of the peer-copy ring protocol of csrc/ring.cu, run to completion under
random interleavings.

The CUDA schedule cannot run without GPUs, and at most 4 of them are ever available to the
tests, so this file restates its ordering rules -- which stream an operation is enqueued on,
which flag counter it waits for or publishes, which event ties two streams of a rank together,
which buffer a copy overwrites -- and executes them for 2 to 8 ranks with every stream of every
rank advancing in random order.  It checks that nothing deadlocks, that every block step reads
the K/V block (or the dK/dV contribution) of the rank and step it should, and that no buffer is
overwritten while its reader has not finished; with and without a plan that leaves out
(query shard, K/V block) pairs, over several calls in a row (the flag counters carry over).

Counters (one page per rank, written by peers): KV_READY[slot], PART_READY[slot],
PROGRESS0[rank], PROGRESS1[rank], ADDED[rank]; `epoch` advances by the ring size per call.

Block steps alternate between two compute lanes of a rank (even steps on the caller's stream,
odd steps on the ring's second compute stream), so that the tail of one block kernel overlaps
the head of the next.  Staging slot, contribution buffer, forward state and PROGRESS counter of
a step are those of its lane (slot = lane = step parity); steps of one lane stay ordered.
"""
import random

import pytest

SLOTS = 4  # staging slots, contribution buffers and receive buffers per rank (slot = step % SLOTS)


class Event:
    def __init__(self):
        self.enqueued = 0
        self.done = 0


class Rank:
    def __init__(self, me, n):
        self.me, self.n = me, n
        self.flags = {}  # (name, index) -> value, this rank's page
        self.stage = [None] * SLOTS  # K/V staging slots: (owner, step, call)
        self.rpart = [None] * SLOTS  # received contributions: (giver, step, call)
        self.part = [None] * SLOTS  # own contribution buffers: (step, call) being built / sent
        self.streams = {"main": [], "lane": [], "push": [], "give": [], "reduce": [], "flag": []}
        self.state = [None, None]  # forward state of each lane: (call, steps folded in)
        self.events = {}
        self.log = []

    def flag(self, name, index):
        return self.flags.get((name, index), 0)

    def event(self, name):
        return self.events.setdefault(name, Event())


class Model:
    def __init__(self, n, need):
        self.n, self.need = n, need
        self.ranks = [Rank(r, n) for r in range(n)]
        self.epoch = 0
        self.call = 0

    # ---- enqueue helpers (host side, program order) -------------------------------------
    def op(self, r, stream, fn, what):
        self.ranks[r].streams[stream].append((fn, what))

    def record(self, r, stream, name):
        ev = self.ranks[r].event(name)
        ev.enqueued += 1
        ticket = ev.enqueued

        def run():
            ev.done = max(ev.done, ticket)
            return True

        self.op(r, stream, run, f"record {name}")

    def wait_event(self, r, stream, name):
        ev = self.ranks[r].event(name)
        ticket = ev.enqueued  # the most recent record at the time of the call; none: no wait
        self.op(r, stream, lambda: ev.done >= ticket, f"wait {name}")

    def wait_flag(self, r, stream, name, index, target):
        rk = self.ranks[r]
        self.op(r, stream, lambda: rk.flag(name, index) >= target, f"wait {name}[{index}] >= {target}")

    def set_flag(self, r, stream, peer, name, index, value):
        targets = [j for j in range(self.n) if (j == peer if peer >= 0 else j != r)]

        def run():
            for j in targets:
                key = (name, index)
                assert self.ranks[j].flags.get(key, 0) <= value, f"counter {name}[{index}] of rank {j} went backwards"
                self.ranks[j].flags[key] = value
            return True

        self.op(r, stream, run, f"set {name}[{index}] = {value} at {targets}")

    def needed(self, q_rank, kv_rank):
        return self.need is None or self.need[q_rank][kv_rank]

    # ---- the schedule: mirrors send_kv / wait_kv / step_done / ra_ring_fwd / ra_ring_bwd ----
    def send_kv(self, me, t):
        n, E, slot, call = self.n, self.epoch, t % SLOTS, self.call
        to = (me + t) % n
        if not self.needed(to, me):
            return
        # the consumer's stage[slot] was last read by its step t - SLOTS (same lane: SLOTS is even)
        self.wait_flag(me, "push", f"PROGRESS{t & 1}", to, E + t - SLOTS + 1 if t > SLOTS else E)

        def copy():
            old = self.ranks[to].stage[slot]
            if old is not None:  # the slot's previous block must have been consumed
                owner, step, c = old
                assert ("done", owner, step, c) in self.ranks[to].log, f"rank {to} stage[{slot}] overwritten before use"
            self.ranks[to].stage[slot] = (me, t, call)
            return True

        self.op(me, "push", copy, f"push K/V to {to} slot {slot}")
        self.set_flag(me, "push", to, "KV_READY", slot, E + t)

    def block(self, me, stream, t, kind):
        n, call = self.n, self.call
        src = (me - t) % n

        def run():
            rk = self.ranks[me]
            if t > 0:
                assert rk.stage[t % SLOTS] == (src, t, call), f"rank {me} step {t} ({kind}) reads {rk.stage[t % SLOTS]}, wants {(src, t, call)}"
            rk.log.append(("block", kind, t, call))
            return True

        self.op(me, stream, run, f"{kind} block step {t}")

    @staticmethod
    def lane(t):
        return "main" if t % 2 == 0 else "lane"

    def step_done(self, me, t):
        src, call = (me - t) % self.n, self.call

        def run():
            self.ranks[me].log.append(("done", src, t, call))
            return True

        self.op(me, self.lane(t), run, f"step {t} done")
        # published from a high-priority stream behind an event: a one-thread kernel on the lane
        # itself would queue behind the other lane's block kernel until its last wave
        self.record(me, self.lane(t), f"ev_done{t % SLOTS}")
        self.wait_event(me, "flag", f"ev_done{t % SLOTS}")
        self.set_flag(me, "flag", -1, f"PROGRESS{t & 1}", me, self.epoch + t + 1)

    def begin_call(self, me):
        self.record(me, "main", "ev_start")
        self.wait_event(me, "push", "ev_start")
        self.wait_event(me, "reduce", "ev_start")
        self.wait_event(me, "lane", "ev_start")
        self.wait_event(me, "give", "ev_start")

    def end_call(self, me):
        # both lanes' counters end the call at epoch + n: the next call's first pushes wait for that
        self.record(me, "main", "ev_main_end")
        self.wait_event(me, "flag", "ev_main_end")
        self.set_flag(me, "flag", -1, "PROGRESS0", me, self.epoch + self.n)
        self.record(me, "push", "ev_push_tail")
        self.wait_event(me, "main", "ev_push_tail")
        self.record(me, "give", "ev_give_tail")
        self.wait_event(me, "main", "ev_give_tail")

    def join_lane(self, me):
        self.record(me, "lane", "ev_lane_done")
        self.wait_event(me, "main", "ev_lane_done")
        self.wait_event(me, "flag", "ev_lane_done")
        self.set_flag(me, "flag", -1, "PROGRESS1", me, self.epoch + self.n)

    def forward(self):
        n, E = self.n, self.epoch
        for me in range(n):
            self.begin_call(me)
            for t in range(n):
                if t + 1 < n:
                    self.send_kv(me, t + 1)
                if t > 0 and not self.needed(me, (me - t) % n):
                    self.step_done(me, t)
                    continue
                ln = self.lane(t)
                if t > 0:
                    self.wait_flag(me, ln, "KV_READY", t % SLOTS, E + t)
                self.block(me, ln, t, "fwd")

                def fold(me=me, t=t, call=self.call):
                    st = self.ranks[me].state
                    prev = st[t & 1]
                    st[t & 1] = (call, (prev[1] if prev and prev[0] == call else ()) + (t,))
                    return True

                self.op(me, ln, fold, f"fold step {t} into state {t & 1}")
                self.step_done(me, t)
            self.join_lane(me)

            def merge(me=me, call=self.call):
                st = self.ranks[me].state
                got = sorted(sum((x[1] for x in st if x and x[0] == call), ()))
                want = [t for t in range(n) if t == 0 or self.needed(me, (me - t) % n)]
                assert got == want, f"rank {me} merges states holding steps {got}, wants {want}"
                return True

            self.op(me, "main", merge, "merge the two lanes' states")
            self.set_flag(me, "main", -1, "ADDED", me, E + n)
            self.end_call(me)
        self.epoch += n
        self.call += 1

    def backward(self):
        n, E, call = self.n, self.epoch, self.call
        for me in range(n):
            rk = self.ranks[me]
            self.begin_call(me)
            self.record(me, "main", "ev_lane_start")  # delta computed, dQ accumulator cleared
            self.wait_event(me, "lane", "ev_lane_start")
            for t in range(n):
                ln = self.lane(t)
                if t + 1 < n:
                    self.send_kv(me, t + 1)
                if t == 0:
                    self.block(me, "main", 0, "bwd own part 1")
                    self.step_done(me, 0)
                    self.record(me, "main", "ev_step0")
                    self.wait_event(me, "reduce", "ev_step0")
                    continue
                slot = t % SLOTS
                owner, giver = (me - t) % n, (me + t) % n
                compute, receive = self.needed(me, owner), self.needed(giver, me)
                if compute:
                    self.wait_flag(me, ln, "KV_READY", slot, E + t)
                    if t > SLOTS:
                        self.wait_event(me, ln, f"ev_sent{slot}")

                    def clear(slot=slot, t=t, rk=rk, me=me):
                        old = rk.part[slot]
                        assert old is None or old[2] == "sent", f"rank {me} part[{slot}] cleared while {old} is in flight"
                        rk.part[slot] = (t, call, "built")
                        return True

                    self.op(me, ln, clear, f"first store into part[{slot}]")
                    self.block(me, ln, t, "bwd")
                self.step_done(me, t)
                if compute:
                    self.record(me, ln, f"ev_part{slot}")
                    # contributions travel on a stream of their own: a K/V block for a later step must
                    # not queue behind a contribution that waits for its block kernel
                    self.wait_event(me, "give", f"ev_part{slot}")
                    self.wait_flag(me, "give", "ADDED", owner, E + t - SLOTS + 1 if t > SLOTS else E)

                    def give(slot=slot, t=t, owner=owner, rk=rk, me=me):
                        assert rk.part[slot] == (t, call, "built"), (me, rk.part[slot])
                        old = self.ranks[owner].rpart[slot]
                        assert old is None or old[3] == "added", f"rank {owner} rpart[{slot}] overwritten while {old} is unread"
                        self.ranks[owner].rpart[slot] = (me, t, call, "fresh")
                        rk.part[slot] = (t, call, "sent")
                        return True

                    self.op(me, "give", give, f"push contribution to {owner}")
                    self.set_flag(me, "give", owner, "PART_READY", slot, E + t)
                    self.record(me, "give", f"ev_sent{slot}")
                if receive:
                    self.wait_flag(me, "reduce", "PART_READY", slot, E + t)

                    def add(slot=slot, t=t, giver=giver, rk=rk, me=me):
                        assert rk.rpart[slot] == (giver, t, call, "fresh"), f"rank {me} adds {rk.rpart[slot]}, wants {(giver, t, call)}"
                        rk.rpart[slot] = (giver, t, call, "added")
                        rk.log.append(("added", giver, t, call))
                        return True

                    self.op(me, "reduce", add, f"add contribution of {giver}")
                self.set_flag(me, "reduce", -1, "ADDED", me, E + t + 1)
            self.record(me, "reduce", "ev_tail")
            self.block(me, self.lane(n - 1), 0, "bwd own part 2")  # behind the last remote step, on its lane
            self.join_lane(me)
            self.wait_event(me, "main", "ev_tail")
            self.op(me, "main", lambda me=me: self.ranks[me].log.append(("finished", call)) or True, "casts")
            self.end_call(me)
        self.epoch += n
        self.call += 1

    # ---- execution: any stream whose head operation can run, in random order ------------------
    def run(self, rng):
        heads = [(r, s) for r in range(self.n) for s in ("main", "lane", "push", "give", "reduce", "flag")]
        pos = {h: 0 for h in heads}
        while True:
            rng.shuffle(heads)
            progressed, left = False, 0
            for h in heads:
                ops = self.ranks[h[0]].streams[h[1]]
                burst = rng.randint(1, 4)
                while pos[h] < len(ops) and burst > 0:
                    fn, _ = ops[pos[h]]
                    if not fn():
                        break
                    pos[h] += 1
                    burst -= 1
                    progressed = True
                left += len(ops) - pos[h]
            if left == 0:
                return
            if not progressed:
                stuck = {h: self.ranks[h[0]].streams[h[1]][pos[h]][1] for h in heads
                         if pos[h] < len(self.ranks[h[0]].streams[h[1]])}
                raise AssertionError(f"deadlock: {stuck}")


def _random_plan(n, rng, density):
    need = [[r == o or rng.random() < density for o in range(n)] for r in range(n)]
    return need


def _check(model, n, calls):
    for r in range(n):
        log = model.ranks[r].log
        for call, kind in enumerate(calls):
            want = [t for t in range(n) if t == 0 or model.needed(r, (r - t) % n)]
            got = [e[2] for e in log if e[0] == "block" and e[3] == call and e[1] in ("fwd", "bwd")]
            if kind == "fwd":  # steps of different lanes may finish in either order
                assert sorted(got) == want, (r, call, got, want)
            else:
                assert sorted(got) == want[1:], (r, call, got, want)
                givers = sorted(e[1] for e in log if e[0] == "added" and e[3] == call)
                assert givers == sorted((r + t) % n for t in range(1, n) if model.needed((r + t) % n, r)), (r, call, givers)
                assert ("finished", call) in log


@pytest.mark.parametrize("n", [2, 3, 4, 5, 8, 11])
@pytest.mark.parametrize("plan", ["none", "dense", "sparse", "diagonal"])
def test_protocol_runs_to_completion_under_random_interleavings(n, plan):
    calls = ["fwd", "bwd", "fwd", "fwd", "bwd", "bwd"]
    for seed in range(6):
        rng = random.Random(1000 * n + seed)
        need = {"none": None, "dense": _random_plan(n, rng, 0.8), "sparse": _random_plan(n, rng, 0.3),
                "diagonal": _random_plan(n, rng, 0.0)}[plan]
        model = Model(n, need)
        for kind in calls:  # the host enqueues whole calls without waiting for the device
            model.forward() if kind == "fwd" else model.backward()
        model.run(rng)
        _check(model, n, calls)

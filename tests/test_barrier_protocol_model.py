"""CPU: host-only models of the barrier protocols of the single-pass backward kernel
(dadgpt_b200/csrc/flash_bwd_fused_sm100.cu) and of the head-size-64 forward kernel
(dadgpt_b200/csrc/flash_fwd64_sm100.cu), run under adversarial schedules.

The kernel's roles (TMA producer, MMA issuer, the compute warps and the accumulator drain warps
each taken as one agent, the dQ reducer) are written down as the sequences of waits and arrivals they execute, per work item and tile, in
the order of the CUDA source. Barriers behave like mbarriers waited by PARITY: a wait for the
k-th completion passes iff the number of completed phases is odd/even as k + 1 is, so it is only
correct while that number is k (blocks) or k + 1 (passes). The model checks, at every evaluation
of every wait, that the count is one of those two: a barrier that has run two phases ahead of its
waiter would leave the waiter blocked for ever (on the GPU: until the bounded wait expires), one
that is behind by a phase would let it through too early.

TMA completions arrive after arbitrary delays and in any order; tensor-core commits arrive after
arbitrary delays but in issue order; which runnable agent moves next is chosen at random, with
one agent at a time slowed down heavily. Item lists include the shapes that matter: single-tile
items behind longer ones.

With one `dkv_staged` barrier for all items, and the compute warps draining the accumulators
themselves (the layout the kernel had first), the model finds the violation that showed up as
intermittent timeouts on some GPUs; with one barrier per K/V buffer no schedule produces one, in
that role split or in the committed one (separate drain warps).
"""
import random

import pytest

STAGES = 2


class Violation(Exception):
    pass


class Sim:
    def __init__(self, items, per_buffer_dkv, rng, drain_warps=True):
        self.items, self.per_buffer, self.rng = items, per_buffer_dkv, rng
        # drain_warps=False: the kernel's earlier role split, in which the compute warps took
        # dQ / dK / dV out of tensor memory themselves (kept to show what the model catches)
        self.drain_warps = drain_warps
        self.done = {}          # barrier name -> completed phases
        self.count = {}         # barrier name -> arrivals in the current phase
        self.need = {}          # barrier name -> arrivals per phase (default 1)
        self.tma = []           # pending TMA completions (any order)
        self.queues = {"tensor": []}   # pending tensor-pipe commits, in order per issuing thread

    # ---- primitives ----
    def arrive(self, name):
        self.count[name] = self.count.get(name, 0) + 1
        if self.count[name] == self.need.get(name.split("[")[0], 1):
            self.count[name] = 0
            self.done[name] = self.done.get(name, 0) + 1

    def ready(self, name, k):
        """Parity wait for the k-th completion (0-based). Raises when the count is outside {k, k+1}."""
        c = self.done.get(name, 0)
        if c - k not in (0, 1):
            raise Violation(f"{name}: waiter wants completion {k}, barrier has completed {c}")
        return c == k + 1

    def dkv(self, j):
        return (f"dkv_staged[{j & 1}]", j >> 1) if self.per_buffer else ("dkv_staged", j)

    # ---- roles: generators yielding ('wait', name, k) | ('arrive', name) | ('tma', name) | ('commit', name)
    def producer(self):
        g = 0
        for j, n_it in enumerate(self.items):
            kb = j & 1
            if j >= 2:
                yield ("wait", f"dkv_sent[{kb}]", (j >> 1) - 1)
            yield ("tma", f"kv_full[{kb}]")
            for _ in range(n_it):
                s, use = g % STAGES, g // STAGES
                if use > 0:
                    yield ("wait", f"qdo_empty[{s}]", use - 1)
                yield ("tma", f"q_full[{s}]")
                yield ("tma", f"do_full[{s}]")
                yield ("tma", f"vec_full[{s}]")           # the tile's row scalars ride the same ring
                g += 1

    def issuer(self):
        def issue_x(g):
            s, use = g % STAGES, g // STAGES
            yield ("wait", f"q_full[{s}]", use)
            yield ("wait", f"do_full[{s}]", use)
            yield ("commit", "x_full")

        yield ("wait", "kv_full[0]", 0)
        yield from issue_x(0)
        g = 0
        for j, n_it in enumerate(self.items):
            for i in range(n_it):
                if i + 1 < n_it:
                    yield ("wait", "x_free", g)
                    yield from issue_x(g + 1)
                elif j + 1 < len(self.items):
                    kbn = (j + 1) & 1
                    yield ("wait", "x_free", g)
                    yield ("wait", f"kv_full[{kbn}]", (j + 1) >> 1)
                    yield from issue_x(g + 1)
                # issue_acc(g)
                yield ("wait", "w_full", g)
                if i == 0 and j > 0 and self.drain_warps:
                    yield ("wait", "dkv_drained", j - 1)
                yield ("commit", f"qdo_empty[{g % STAGES}]")     # after dV / dK, before dQ
                if g > 0:
                    yield ("wait", "dq_drained", g - 1)
                yield ("commit", "acc_done")
                g += 1

    def compute(self):
        g = 0
        for j, n_it in enumerate(self.items):
            for i in range(n_it):
                yield ("wait", f"vec_full[{g % STAGES}]", g // STAGES)
                yield ("wait", "x_full", g)
                yield ("arrive", "x_free")
                if g > 0:
                    yield ("wait", "acc_done", g - 1)
                yield ("arrive", "w_full")
                g += 1

    def compute_and_drain(self):
        """The earlier role split: the compute warps drain the accumulators between tiles."""
        def drain_dq(t):
            yield ("arrive", "dq_drained")
            if t > 0:
                yield ("wait", "dq_sent", t - 1)
            yield ("arrive", "dq_staged")

        g = 0
        j = 0
        for j, n_it in enumerate(self.items):
            for i in range(n_it):
                yield ("wait", f"vec_full[{g % STAGES}]", g // STAGES)
                yield ("wait", "x_full", g)
                yield ("arrive", "x_free")
                if g > 0:
                    yield ("wait", "acc_done", g - 1)
                if i == 0 and j > 0:
                    yield ("arrive", self.dkv(j - 1)[0])      # stage dK / dV of the finished item
                yield ("arrive", "w_full")
                if g > 0:
                    yield from drain_dq(g - 1)
                g += 1
        if g > 0:
            yield ("wait", "acc_done", g - 1)
            yield ("arrive", self.dkv(j)[0])
            yield from drain_dq(g - 1)

    def drain(self):
        """The accumulator drain warps: each tile's dQ, each finished item's dK / dV."""
        g = 0
        for j, n_it in enumerate(self.items):
            for i in range(n_it):
                if g > 0:
                    yield ("wait", "dq_sent", g - 1)
                yield ("wait", "acc_done", g)
                if i + 1 == n_it:
                    yield ("arrive", "dkv_drained")
                    yield ("arrive", self.dkv(j)[0])
                yield ("arrive", "dq_drained")
                yield ("arrive", "dq_staged")
                g += 1

    def reducer(self):
        g = 0
        for j, n_it in enumerate(self.items):
            for i in range(n_it):
                yield ("wait", "dq_staged", g)
                if i + 1 < n_it:
                    yield ("arrive", "dq_sent")
                else:
                    name, k = self.dkv(j)
                    yield ("wait", name, k)
                    yield ("arrive", "dq_sent")
                    yield ("arrive", f"dkv_sent[{j & 1}]")
                g += 1

    def roles(self):
        if not self.drain_warps:
            return {"producer": self.producer(), "issuer": self.issuer(),
                    "compute": self.compute_and_drain(), "reducer": self.reducer()}
        return {"producer": self.producer(), "issuer": self.issuer(), "compute": self.compute(),
                "drain": self.drain(), "reducer": self.reducer()}

    # ---- scheduler ----
    def run(self, max_steps=400000):
        roles = self.roles()
        pending = {n: None for n in roles}   # a wait the role is blocked on
        alive = set(roles)
        others = ["tma"] + list(self.queues) + [None]
        slow = self.rng.choice(list(roles) + others)
        for _ in range(max_steps):
            movable = []
            for n in sorted(alive):   # a fixed order, so that a seed names one schedule
                op = pending[n]
                if op is None or self.ready(op[1], op[2]):   # ready() also audits the wait
                    movable.append(n)
            if self.tma:
                movable.append("tma")
            movable += [qn for qn, q in self.queues.items() if q]
            if not movable:
                if alive:
                    raise Violation(f"deadlock: {sorted(alive)} blocked on "
                                    f"{ {n: pending[n][1:] for n in alive if pending[n]} }")
                return
            who = self.rng.choice(movable)
            if who == slow and self.rng.random() < 0.9 and len(movable) > 1:
                continue
            if who == "tma":
                self.arrive(self.tma.pop(self.rng.randrange(len(self.tma))))
                continue
            if who in self.queues:
                self.arrive(self.queues[who].pop(0))
                continue
            pending[who] = None
            try:
                op = next(roles[who])
            except StopIteration:
                alive.discard(who)
                continue
            if op[0] == "wait":
                pending[who] = op
            elif op[0] == "arrive":
                self.arrive(op[1])
            elif op[0] == "tma":
                self.tma.append(op[1])
            elif op[0] == "commit":
                self.queues[op[2] if len(op) > 2 else "tensor"].append(op[1])
            if self.rng.random() < 0.02:
                slow = self.rng.choice(list(roles) + others)
        raise Violation("did not finish")


ITEM_LISTS = [
    [3, 1, 1, 2],          # a single-tile item behind another: the case that failed
    [8, 7, 1, 1, 1, 4, 1],
    [1, 1, 1, 1, 1, 1],
    [2, 2, 2, 2],
    [5],
    [1, 6, 1, 6, 1],
]


def first_violation(per_buffer, seeds=range(300), drain_warps=True):
    for items in ITEM_LISTS:
        for seed in seeds:
            try:
                Sim(items, per_buffer, random.Random(seed), drain_warps).run()
            except Violation as e:
                return items, seed, str(e)
    return None


def test_one_dkv_staged_barrier_per_buffer_survives_every_schedule():
    assert first_violation(per_buffer=True) is None


def test_the_earlier_role_split_survives_too():
    assert first_violation(per_buffer=True, drain_warps=False) is None


def test_a_single_dkv_staged_barrier_is_caught():
    # the failure belonged to the earlier role split: there the compute warps could stage the
    # next item's dK / dV without needing the reducer
    found = first_violation(per_buffer=False, drain_warps=False)
    assert found is not None, "the model no longer reproduces the double-advancing barrier"
    assert "dkv_staged" in found[2] or "deadlock" in found[2]


# ---------------------------------------------------------------------------------------------
# The head-size-64 forward (dadgpt_b200/csrc/flash_fwd64_sm100.cu): TMA producer, one MMA issuer
# per softmax group, each group as two agents (its two halves). Work items are (tiles of group A,
# tiles of group B): B has one tile more than A, or none when the pair's second tile lies beyond
# the sequence. Every K/V tile is two sub-steps with two score buffers per group.
# ---------------------------------------------------------------------------------------------
KV_STAGES = 4


class FwdSim(Sim):
    def __init__(self, items, rng, rescale_prob=0.3):
        super().__init__(items, True, rng)
        self.need = {"kv_empty": 2, "q_empty": 2, "p_full": 2, "o_free": 2, "stat_full": 2}
        self.queues = {"tensor_A": [], "tensor_B": []}
        self.rescale_prob = rescale_prob

    @staticmethod
    def n_of(item, X):
        return item[X]

    @staticmethod
    def n_kv(item):
        return item[1] if item[1] else item[0]

    def producer(self):
        g = 0
        for k, item in enumerate(self.items):
            qb = k & 1
            if k >= 2:
                yield ("wait", f"q_empty[{qb}]", (k >> 1) - 1)
            yield ("tma", f"q_full[{qb}]")
            for _ in range(self.n_kv(item)):
                s, use = g % KV_STAGES, g // KV_STAGES
                if use > 0:
                    yield ("wait", f"kv_empty[{s}]", use - 1)
                yield ("tma", f"k_full[{s}]")
                yield ("tma", f"v_full[{s}]")
                g += 1

    def issuer_x(self, X):
        q = f"tensor_{'AB'[X]}"
        items = self.items
        cur = items[0]
        yield ("wait", "q_full[0]", 0)
        yield ("wait", "k_full[0]", 0)
        if self.n_of(cur, X) > 0:
            yield ("commit", f"s_full[{X}][0]", q)
            yield ("commit", f"s_full[{X}][1]", q)
        if self.n_of(cur, X) <= 1:
            yield ("commit", "q_empty[0]", q) if self.n_of(cur, X) == 1 else ("arrive", "q_empty[0]")
        g = n_pv = n_done = 0
        for k, item in enumerate(items):
            qb, n_x, n_kv = k & 1, self.n_of(item, X), self.n_kv(item)
            for j in range(n_kv):
                s = g % KV_STAGES
                last = j + 1 == n_kv
                have_next = (not last) or k + 1 < len(items)
                ni = items[k + 1] if (last and have_next) else item
                nj, nqb = (0, qb ^ 1) if last else (j + 1, qb)
                yield ("wait", f"v_full[{s}]", g // KV_STAGES)
                n_next = self.n_of(ni, X) if have_next else 0
                s_next = have_next and nj < n_next
                next_ready = issued = False
                for c in (0, 1):
                    if j < n_x:
                        if j == 0 and c == 0 and n_done > 0:
                            yield ("wait", f"o_free[{X}]", n_done - 1)
                        yield ("wait", f"p_full[{X}][{c}]", n_pv >> 1)
                        yield ("commit", f"o_done[{X}][{n_pv & 1}]", q)
                        n_pv += 1
                        issued = True
                    if s_next:
                        if not next_ready:
                            if last:
                                yield ("wait", f"q_full[{nqb}]", (k + 1) >> 1)
                            yield ("wait", f"k_full[{(g + 1) % KV_STAGES}]", (g + 1) // KV_STAGES)
                            next_ready = True
                        yield ("commit", f"s_full[{X}][{c}]", q)
                        issued = True
                        if c == 1 and nj + 1 == n_next:
                            yield ("commit", f"q_empty[{nqb}]", q)
                if have_next and not s_next and nj == 0:
                    if last:
                        yield ("wait", f"q_full[{nqb}]", (k + 1) >> 1)
                    yield ("arrive", f"q_empty[{nqb}]")
                yield ("commit", f"kv_empty[{s}]", q) if issued else ("arrive", f"kv_empty[{s}]")
                g += 1
            if n_x > 0:
                n_done += 1

    def softmax(self, X):
        t = n_item = 0
        for item in self.items:
            n_x = self.n_of(item, X)
            if n_x == 0:
                continue
            for v in range(2 * n_x):
                c = v & 1
                yield ("wait", f"s_full[{X}][{c}]", t >> 1)
                if v > 0 and self.rng.random() < self.rescale_prob:   # the lazy rescale looks at O
                    yield ("wait", f"o_done[{X}][{(t - 1) & 1}]", (t - 1) >> 1)
                yield ("arrive", f"p_full[{X}][{c}]")
                t += 1
            yield ("arrive", f"stat_full[{X}]")
            yield ("wait", f"stat_full[{X}]", n_item)
            yield ("wait", f"o_done[{X}][{(t - 1) & 1}]", (t - 1) >> 1)
            yield ("arrive", f"o_free[{X}]")
            n_item += 1

    def roles(self):
        return {"producer": self.producer(), "issuer_A": self.issuer_x(0), "issuer_B": self.issuer_x(1),
                "A0": self.softmax(0), "A1": self.softmax(0), "B0": self.softmax(1), "B1": self.softmax(1)}


FWD_ITEM_LISTS = [
    [(7, 8), (5, 6), (3, 4), (1, 2)],             # the GPT-2 shape's pairs, heaviest first
    [(1, 2)] * 7,
    [(1, 0)] * 9,                                 # S = 128: lone tiles, group B and its issuer idle throughout
    [(9, 0), (7, 8), (1, 0), (3, 4)],             # odd tile count: a lone last tile longer than the ring
    [(5, 0), (1, 2), (5, 0)],
    [(1, 2), (1, 0), (1, 2), (1, 0), (3, 4)],
]


def test_forward_protocol_survives_every_schedule():
    for items in FWD_ITEM_LISTS:
        for seed in range(150):
            FwdSim(items, random.Random(seed)).run()


def test_forward_model_catches_an_ungated_idle_issuer():
    """The rule the idle issuer follows (wait for the stage's data before releasing it) is what
    keeps it from arriving twice within one phase of kv_empty; a model without that wait must
    trip the audit, or the model is not looking."""
    class Ungated(FwdSim):
        def issuer_x(self, X):
            for op in super().issuer_x(X):
                if X == 1 and op[0] == "wait" and op[1].startswith("v_full"):
                    continue
                yield op
    caught = False
    for seed in range(200):
        try:
            Ungated([(9, 0), (9, 0), (9, 0)], random.Random(seed)).run()
        except Violation:
            caught = True
            break
    assert caught

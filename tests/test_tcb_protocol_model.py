"""A model of the small-batch kernel's intra-CTA protocol (csrc/linear_tcb.cu), run under random interleavings on the CPU.

Agents: the producer warp (digit stages, released per warpgroup and stage), one issuer per warpgroup (weight stages, MMAs,
commits) and the compute warps (reads of step i + 1 hoisted into iteration i, sums read two steps behind).  Barriers are
mbarriers waited on by PARITY, as on the device, so a waiter that fell two phases behind would be caught as aliasing.
The test checks: no deadlock, no parity aliasing, no stage refilled before all of its readers are done, every reader sees
the step it expects; and that the same checks do flag a protocol whose producer does not wait for the release.
"""
import random


class MBar:
    def __init__(self, count): self.count = count; self.pending = count; self.ph = 0
    def arrive(self):
        self.pending -= 1
        assert self.pending >= 0, "too many arrivals"
        if self.pending == 0: self.ph += 1; self.pending = self.count
    def done(self, k):                      # hardware test for "phase k complete" through its parity
        alias = self.ph - k >= 2
        return ((self.ph & 1) != (k & 1)), alias

def simulate(n, NWG, AST, BST, CW, seed, single_empty=False, producer_waits=True):
    rnd = random.Random(seed)
    a_full = [[MBar(1) for _ in range(AST)] for _ in range(NWG)]
    b_full = [MBar(1) for _ in range(BST)]
    b_empty = [MBar(NWG) for _ in range(BST)] if single_empty else [[MBar(1) for _ in range(BST)] for _ in range(NWG)]
    mma_bar = [[MBar(1), MBar(1)] for _ in range(NWG)]
    nb = [[0, 0] for _ in range(NWG)]        # named barrier arrival counts (compute warps)
    nb_gen = [[0, 0] for _ in range(NWG)]    # completed generations
    a_content = [[None] * AST for _ in range(NWG)]; b_content = [None] * BST
    a_readers = [[set() for _ in range(AST)] for _ in range(NWG)]; b_readers = [set() for _ in range(BST)]
    pending = []                             # asynchronous completions: (kind, args)
    errors = []
    def prod():
        for i in range(n):
            s = i % BST
            if producer_waits and i >= BST:
                k = i // BST - 1
                bars = [b_empty[s]] if single_empty else [b_empty[w][s] for w in range(NWG)]
                for b in bars:
                    while True:
                        ok, alias = b.done(k)
                        if alias: errors.append(("alias b_empty", i))
                        if ok: break
                        yield
            # refill: every reader of the previous content must be done
            if b_content[s] is not None and len(b_readers[s]) < NWG * (CW + 1):
                errors.append(("B stage reused early", i, s, len(b_readers[s])))
            b_content[s] = ("loading", i); b_readers[s] = set()
            pending.append(("b", s, i)); yield
    def issuer(w):
        issued = 0
        def load():
            nonlocal issued
            s = issued % AST
            if a_content[w][s] is not None and len(a_readers[w][s]) < CW: errors.append(("A stage reused early", w, issued))
            a_content[w][s] = ("loading", issued); a_readers[w][s] = set(); pending.append(("a", w, s, issued)); issued += 1
        for _ in range(min(n, AST)): load(); yield
        for i in range(n):
            buf = i & 1
            while nb_gen[w][buf] <= i // 2 - 0 - 0 and not (nb[w][buf] >= CW): yield      # wait for the CW arrivals of step i
            nb[w][buf] -= CW; nb_gen[w][buf] += 1
            s = i % BST
            while True:
                ok, alias = b_full[s].done(i // BST)
                if alias: errors.append(("alias b_full (issuer)", i))
                if ok: break
                yield
            if b_content[s] != ("ready", i): errors.append(("issuer reads wrong B", i, b_content[s]))
            pending.append(("mma", w, buf, s, i)); yield
            if issued < n: load(); yield
    def compute(w, c):
        def fetch(i):
            s = i % AST
            while True:
                ok, alias = a_full[w][s].done(i // AST)
                if alias: errors.append(("alias a_full", w, i))
                if ok: break
                yield
            if a_content[w][s] != ("ready", i): errors.append(("compute reads wrong A", w, i, a_content[w][s]))
            a_readers[w][s].add(c)
            sb = i % BST
            while True:
                ok, alias = b_full[sb].done(i // BST)
                if alias: errors.append(("alias b_full (compute)", w, i))
                if ok: break
                yield
            if b_content[sb] != ("ready", i): errors.append(("compute reads wrong SF", w, i, b_content[sb]))
            b_readers[sb].add((w, c))
        if n > 0: yield from fetch(0)
        for i in range(n + 2):
            buf = i & 1
            if i >= 2:
                k = (i >> 1) - 1
                while True:
                    ok, alias = mma_bar[w][buf].done(k)
                    if alias: errors.append(("alias mma_bar", w, i))
                    if ok: break
                    yield
            if i < n:
                yield
                if i + 1 < n: yield from fetch(i + 1)
                nb[w][buf] += 1                      # bar.arrive
            yield
    agents = [prod()] + [issuer(w) for w in range(NWG)] + [compute(w, c) for w in range(NWG) for c in range(CW)]
    alive = list(range(len(agents)))
    idle_rounds = 0
    while alive:
        progressed = False
        # asynchronous completions happen at random times
        if pending and rnd.random() < 0.5:
            ev = pending.pop(rnd.randrange(len(pending)))
            if ev[0] == "b": _, s, i = ev; b_content[s] = ("ready", i); b_full[s].arrive()
            elif ev[0] == "a": _, w, s, i = ev; a_content[w][s] = ("ready", i); a_full[w][s].arrive()
            else:
                _, w, buf, s, i = ev
                mma_bar[w][buf].arrive()
                b_readers[s].add((w, "mma"))
                (b_empty[s] if single_empty else b_empty[w][s]).arrive()
            progressed = True
        a = rnd.choice(alive)
        before = (tuple(x.ph for row in a_full for x in row), tuple(x.ph for x in b_full), len(pending), tuple(map(tuple, nb)))
        try:
            next(agents[a])
        except StopIteration:
            alive.remove(a); progressed = True
        after = (tuple(x.ph for row in a_full for x in row), tuple(x.ph for x in b_full), len(pending), tuple(map(tuple, nb)))
        if before != after: progressed = True
        idle_rounds = 0 if progressed else idle_rounds + 1
        if idle_rounds > 20000 and not pending:
            errors.append(("deadlock", [x for x in alive])); break
    return errors


def _sweep(trials, **kw):
    found = []
    for trial in range(trials):
        rnd = random.Random(trial)
        n = rnd.randint(1, 30)
        NWG = rnd.choice([2, 3])
        AST, BST = rnd.randint(2, 6), rnd.randint(2, 6)
        e = simulate(n, NWG, AST, BST, 2, trial, **kw)
        if e:
            found.append((dict(n=n, NWG=NWG, AST=AST, BST=BST), e[:3]))
    return found


def test_protocol_has_no_deadlock_aliasing_or_early_reuse():
    assert _sweep(200) == []
    assert _sweep(100, single_empty=True) == []           # the earlier form: one release barrier of count NWG per stage


def test_model_flags_a_producer_that_does_not_wait_for_the_release():
    assert _sweep(40, producer_waits=False) != []

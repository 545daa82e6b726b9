"""Discrete-event model of the mbarrier protocol of the key-loop tcgen05 kernels
(llsa_b200/csrc/attn_pooled_loop_tc.cu, attn_pooled_bwd_loop_tc.cu, attn_pooled_dkv_loop_tc.cu) and of the
single-shot pooled backward with its two MMA-issuing threads (attn_pooled_bwd_tc.cu).

Test infrastructure: nothing in the package imports it.  Every role of a CTA
(TMA producer, the threads that issue MMAs, the eight softmax warps) is a Python
generator that waits on barriers, spends random time and arrives, exactly in the
order the kernel's role does.  The model keeps the hardware's semantics where
they matter for correctness:

* a barrier has an arrival count and a phase; a wait names a PARITY and passes
  when the barrier's current (incomplete) phase has the other parity.  A wait
  for "completion number u" therefore also passes when completion u - 1 has
  not happened yet -- the case a protocol must exclude by construction;
* `tcgen05.commit` arrives when the MMAs the committing thread issued before
  it have completed; MMAs of all threads share one in-order pipe;
* a TMA load arrives on its barrier after a random latency.

On top of that the model tracks who owns each tensor-memory buffer and each
operand ring stage and asserts at every read and overwrite, so that a protocol
error shows as a failed assertion or as a deadlock (roles left waiting with no
event pending), not as a wrong number.
"""
import heapq
import random


class Barrier:
    def __init__(self, name, count):
        self.name, self.count, self.pending, self.phase = name, count, count, 0

    def parity(self):                     # parity of the current, incomplete phase
        return self.phase & 1

    def arrive(self, sim):
        self.pending -= 1
        assert self.pending >= 0, self.name
        if self.pending == 0:
            self.phase += 1
            self.pending = self.count
            sim.wake(self)


class Sim:
    def __init__(self, seed):
        self.t, self.queue, self.serial = 0, [], 0
        self.rng = random.Random(seed)
        self.waiting = []                 # (role, barrier, parity)
        self.roles = {}
        self.pipe_free = 0                # the tensor pipe executes in issue order
        self.last_mma_done = {}           # per issuing thread

    def at(self, t, fn):
        self.serial += 1
        heapq.heappush(self.queue, (t, self.serial, fn))

    def spawn(self, name, gen):
        self.roles[name] = gen
        self.at(0, lambda: self.step(name))

    def step(self, name):
        gen = self.roles.get(name)
        if gen is None:
            return
        try:
            op = next(gen)
        except StopIteration:
            del self.roles[name]
            return
        if op[0] == "delay":
            self.at(self.t + op[1], lambda: self.step(name))
        else:                             # ("wait", barrier, parity)
            _, bar, par = op
            if bar.parity() != par:
                self.at(self.t + self.rng.randint(20, 120), lambda: self.step(name))
            else:
                self.waiting.append((name, bar, par))

    def wake(self, bar):
        still = []
        for name, b, par in self.waiting:
            if b is bar and b.parity() != par:
                self.at(self.t + self.rng.randint(20, 150), (lambda nm: (lambda: self.step(nm)))(name))
            else:
                still.append((name, b, par))
        self.waiting = still

    def run(self):
        while self.queue:
            self.t, _, fn = heapq.heappop(self.queue)
            fn()
        return "deadlock" if self.roles else "ok"

    def mma(self, thread, cycles):        # -> (start, done) on the shared pipe
        start = max(self.pipe_free, self.t)
        self.pipe_free = start + cycles
        self.last_mma_done[thread] = self.pipe_free
        return start, self.pipe_free

    def commit(self, thread, bar):
        done = max(self.last_mma_done.get(thread, 0), self.t) + self.rng.randint(20, 100)
        self.at(done, lambda: bar.arrive(self))

    def tma(self, bar, fn=None):
        def land():
            if fn:
                fn()
            bar.arrive(self)
        self.at(self.t + self.rng.randint(500, 1500), land)

    def r(self, a, b):
        return self.rng.randint(a, b)


def key_major_kernel(seed, units, score_threads=1, score_barriers=3, stages=8, buffers=3):
    """attn_dkv_pooled_loop_tc_kernel.  `units`: job counts of the (head, chunk) units of one CTA's piece.
    score_threads: threads that issue S^T / dP^T (1 = the kernel; 2 = even and odd jobs on two threads).
    score_barriers: sdp_ready / buf_free barriers (3 = one per buffer, the kernel; 6 = one per job number mod 6)."""
    sim = Sim(seed)
    nb = score_barriers
    kv_full, kv_empty = Barrier("kv_full", 1), Barrier("kv_empty", score_threads)
    q_full = [Barrier("q_full%d" % i, 1) for i in range(stages)]
    q_empty = [Barrier("q_empty%d" % i, 1) for i in range(stages)]
    sdp = [Barrier("sdp_ready%d" % i, 1) for i in range(nb)]
    pds = [Barrier("pds_ready%d" % i, 4) for i in range(buffers)]
    free = [Barrier("buf_free%d" % i, 1) for i in range(nb)]
    acc_ready, acc_free = Barrier("acc_ready", 1), Barrier("acc_free", 8)
    owner = [None] * buffers              # None: free; ("s", job): scores; ("p", job): probabilities

    def producer():
        job = 0
        for i, n in enumerate(units):
            yield ("wait", kv_empty, (i & 1) ^ 1)
            sim.tma(kv_full)
            for _ in range(n):
                st = job % stages
                yield ("wait", q_empty[st], ((job // stages) & 1) ^ 1)
                yield ("delay", sim.r(20, 80))
                sim.tma(q_full[st])
                job += 1

    def score_issuer(mine):
        job, first = mine, 0
        for i, n in enumerate(units):
            yield ("wait", kv_full, i & 1)
            while job < first + n:
                st, buf = job % stages, job % buffers
                if job >= buffers:
                    prev = job - buffers
                    yield ("wait", free[prev % nb], (prev // nb) & 1)
                yield ("wait", q_full[st], (job // stages) & 1)
                if sim.rng.random() < 0.15:
                    yield ("delay", sim.r(500, 4000))          # one thread falls behind the other
                assert owner[buf] is None, ("scores written over a live buffer", buf, owner[buf], job)
                start, done = sim.mma(("score", mine), 384)
                sim.at(done, (lambda b=buf, j=job: owner.__setitem__(b, ("s", j))))
                yield ("delay", max(0, start - sim.t) + sim.r(50, 200))
                sim.commit(("score", mine), sdp[job % nb])
                yield ("delay", sim.r(30, 80))
                job += score_threads
            first += n
            sim.commit(("score", mine), kv_empty)
            yield ("delay", sim.r(30, 80))

    def out_issuer():
        job = 0
        for i, n in enumerate(units):
            for j in range(n):
                st, buf = job % stages, job % buffers
                yield ("wait", pds[buf], (job // buffers) & 1)
                if j == 0 and i > 0:
                    yield ("wait", acc_free, (i - 1) & 1)
                assert owner[buf] == ("p", job), ("dV / dK read", buf, owner[buf], job)
                start, done = sim.mma("out", 384)
                sim.at(done, (lambda b=buf: owner.__setitem__(b, None)))
                yield ("delay", max(0, start - sim.t) + sim.r(50, 200))
                sim.commit("out", q_empty[st])
                sim.commit("out", free[job % nb])
                yield ("delay", sim.r(60, 160))
                job += 1
            sim.commit("out", acc_ready)
            yield ("delay", sim.r(30, 80))

    def softmax(group, warp):
        job, first = group, 0
        for i, n in enumerate(units):
            while job < first + n:
                buf = job % buffers
                yield ("wait", sdp[job % nb], (job // nb) & 1)
                assert owner[buf] is not None and owner[buf][1] == job, ("softmax read", buf, owner[buf], job)
                yield ("delay", sim.r(500, 1200))
                if warp == 0:
                    owner[buf] = ("p", job)
                pds[buf].arrive(sim)
                job += 2
            first += n
            yield ("wait", acc_ready, i & 1)
            yield ("delay", sim.r(200, 600))
            acc_free.arrive(sim)

    sim.spawn("producer", producer())
    for t in range(score_threads):
        sim.spawn("score%d" % t, score_issuer(t))
    sim.spawn("out", out_issuer())
    for g in range(2):
        for w in range(4):
            sim.spawn("softmax%d%d" % (g, w), softmax(g, w))
    return sim.run()


def query_major_kernel(seed, tiles, jobs, score_threads=1, score_barriers=3, stages=8, buffers=3):
    """attn_dq_pooled_loop_tc_kernel: `tiles` query tiles of `jobs` key chunks (even); Q / dO in two stages, K and V
    chunks in rings, S / dP into three buffers, dQ accumulated per tile."""
    sim = Sim(seed)
    nb = score_barriers
    q_full = [Barrier("q_full%d" % i, 1) for i in range(2)]
    q_empty = [Barrier("q_empty%d" % i, score_threads) for i in range(2)]
    k_full = [Barrier("k_full%d" % i, 1) for i in range(stages)]
    k_empty = [Barrier("k_empty%d" % i, 1) for i in range(stages)]
    v_full = [Barrier("v_full%d" % i, 1) for i in range(stages)]
    v_empty = [Barrier("v_empty%d" % i, 1) for i in range(stages)]
    sdp = [Barrier("sdp_ready%d" % i, 1) for i in range(nb)]
    ds = [Barrier("ds_ready%d" % i, 4) for i in range(buffers)]
    free = [Barrier("buf_free%d" % i, 1) for i in range(nb)]
    dq_ready, dq_free = Barrier("dq_ready", 1), Barrier("dq_free", 8)
    owner = [None] * buffers
    held = [None] * stages                # chunk number a K ring stage holds

    def producer():
        job = 0
        for i in range(tiles):
            yield ("wait", q_empty[i & 1], ((i >> 1) & 1) ^ 1)
            sim.tma(q_full[i & 1])
            for _ in range(jobs):
                st, par = job % stages, ((job // stages) & 1) ^ 1
                yield ("wait", k_empty[st], par)
                assert held[st] is None, ("keys loaded over a live stage", st, held[st], job)
                sim.tma(k_full[st], (lambda s=st, j=job: held.__setitem__(s, j)))
                yield ("wait", v_empty[st], par)
                sim.tma(v_full[st])
                job += 1

    def score_issuer(mine):
        job = mine
        for i in range(tiles):
            yield ("wait", q_full[i & 1], (i >> 1) & 1)
            for _ in range(mine, jobs, score_threads):
                st, par, buf = job % stages, (job // stages) & 1, job % buffers
                if job >= buffers:
                    prev = job - buffers
                    yield ("wait", free[prev % nb], (prev // nb) & 1)
                yield ("wait", k_full[st], par)
                yield ("wait", v_full[st], par)
                if sim.rng.random() < 0.15:
                    yield ("delay", sim.r(500, 4000))
                assert owner[buf] is None, ("scores written over a live buffer", buf, owner[buf], job)
                assert held[st] == job, ("S read the wrong keys", st, held[st], job)
                start, done = sim.mma(("score", mine), 384)
                sim.at(done, (lambda b=buf, j=job: owner.__setitem__(b, ("s", j))))
                yield ("delay", max(0, start - sim.t) + sim.r(50, 200))
                sim.commit(("score", mine), sdp[job % nb])
                sim.commit(("score", mine), v_empty[st])
                yield ("delay", sim.r(30, 80))
                job += score_threads
            sim.commit(("score", mine), q_empty[i & 1])
            yield ("delay", sim.r(30, 80))

    def dq_issuer():
        job = 0
        for i in range(tiles):
            for j in range(jobs):
                st, buf = job % stages, job % buffers
                yield ("wait", ds[buf], (job // buffers) & 1)
                if j == 0 and i > 0:
                    yield ("wait", dq_free, (i - 1) & 1)
                assert owner[buf] == ("p", job), ("dQ read", buf, owner[buf], job)
                assert held[st] == job, ("dQ read the wrong keys", st, held[st], job)
                start, done = sim.mma("dq", 192)

                def release(b=buf, s=st):
                    owner[b] = None
                    held[s] = None
                sim.at(done, release)
                yield ("delay", max(0, start - sim.t) + sim.r(50, 200))
                sim.commit("dq", k_empty[st])
                sim.commit("dq", free[job % nb])
                yield ("delay", sim.r(60, 160))
                job += 1
            sim.commit("dq", dq_ready)
            yield ("delay", sim.r(30, 80))

    def softmax(group, warp):
        job = group
        for i in range(tiles):
            for _ in range(group, jobs, 2):
                buf = job % buffers
                yield ("wait", sdp[job % nb], (job // nb) & 1)
                assert owner[buf] is not None and owner[buf][1] == job, ("softmax read", buf, owner[buf], job)
                yield ("delay", sim.r(400, 1000))
                if warp == 0:
                    owner[buf] = ("p", job)
                ds[buf].arrive(sim)
                job += 2
            yield ("wait", dq_ready, i & 1)
            yield ("delay", sim.r(200, 600))
            dq_free.arrive(sim)

    sim.spawn("producer", producer())
    for t in range(score_threads):
        sim.spawn("score%d" % t, score_issuer(t))
    sim.spawn("dq", dq_issuer())
    for g in range(2):
        for w in range(4):
            sim.spawn("softmax%d%d" % (g, w), softmax(g, w))
    return sim.run()


def forward_kernel(seed, tiles, chunks, passes, k_stages=4, v_stages=4, buffers=3):
    """attn_fwd_pooled_loop_tc_kernel: `tiles` query tiles of `chunks` key chunks; one pass (jobs = chunks, every job
    feeds P.V) or two (jobs = 2 * chunks: row maxima first, then the exponentials; the two groups exchange their maxima
    before their first second-pass job).  One thread issues S, one issues P.V and hands every job's buffer back; the two
    softmax groups take the jobs of one parity of the CTA-wide job number each (with an odd job count the parity of a
    tile's first job alternates) and exchange their row sums at the end of a tile."""
    sim = Sim(seed)
    jobs, first_p2 = passes * chunks, (passes - 1) * chunks
    q_full = [Barrier("q_full%d" % i, 1) for i in range(2)]
    q_empty = [Barrier("q_empty%d" % i, 1) for i in range(2)]
    k_full = [Barrier("k_full%d" % i, 1) for i in range(k_stages)]
    k_empty = [Barrier("k_empty%d" % i, 1) for i in range(k_stages)]
    v_full = [Barrier("v_full%d" % i, 1) for i in range(v_stages)]
    v_empty = [Barrier("v_empty%d" % i, 1) for i in range(v_stages)]
    s_ready = [Barrier("s_ready%d" % i, 1) for i in range(buffers)]
    wg_done = [Barrier("wg_done%d" % i, 4) for i in range(buffers)]
    free = [Barrier("buf_free%d" % i, 1) for i in range(buffers)]
    o_ready, o_free, xchg = Barrier("o_ready", 1), Barrier("o_free", 8), Barrier("xchg", 8)
    owner = [None] * buffers
    v_held = [None] * v_stages
    o_busy = [False]                      # the O accumulator holds a finished tile that has not been read yet

    def producer():
        kjob = vjob = 0
        for i in range(tiles):
            yield ("wait", q_empty[i & 1], ((i >> 1) & 1) ^ 1)
            sim.tma(q_full[i & 1])
            for j in range(jobs):
                ks = kjob % k_stages
                yield ("wait", k_empty[ks], ((kjob // k_stages) & 1) ^ 1)
                sim.tma(k_full[ks])
                kjob += 1
                if j >= first_p2:
                    vs = vjob % v_stages
                    yield ("wait", v_empty[vs], ((vjob // v_stages) & 1) ^ 1)
                    assert v_held[vs] is None, ("values loaded over a live stage", vs, v_held[vs], vjob)
                    sim.tma(v_full[vs], (lambda s=vs, j=vjob: v_held.__setitem__(s, j)))
                    vjob += 1

    def s_issuer():
        n = 0
        for i in range(tiles):
            yield ("wait", q_full[i & 1], (i >> 1) & 1)
            for _ in range(jobs):
                buf, ks = n % buffers, n % k_stages
                if n >= buffers:
                    yield ("wait", free[buf], ((n // buffers) & 1) ^ 1)
                yield ("wait", k_full[ks], (n // k_stages) & 1)
                assert owner[buf] is None, ("scores written over a live buffer", buf, owner[buf], n)
                start, done = sim.mma("s", 256)
                sim.at(done, (lambda b=buf, j=n: owner.__setitem__(b, ("s", j))))
                yield ("delay", max(0, start - sim.t) + sim.r(50, 200))
                sim.commit("s", s_ready[buf])
                sim.commit("s", k_empty[ks])
                yield ("delay", sim.r(30, 80))
                n += 1
            sim.commit("s", q_empty[i & 1])
            yield ("delay", sim.r(30, 80))

    def pv_issuer():
        n = vjob = 0
        for i in range(tiles):
            for j in range(jobs):
                buf = n % buffers
                yield ("wait", wg_done[buf], (n // buffers) & 1)
                if j >= first_p2:
                    vs = vjob % v_stages
                    yield ("wait", v_full[vs], (vjob // v_stages) & 1)
                    if j == first_p2 and i > 0:
                        yield ("wait", o_free, (i - 1) & 1)
                    if j == first_p2:
                        assert not o_busy[0], ("O overwritten before it was read", i)
                    assert owner[buf] == ("p", n), ("P.V read", buf, owner[buf], n)
                    assert v_held[vs] == vjob, ("P.V read the wrong values", vs, v_held[vs], vjob)
                    start, done = sim.mma("pv", 384)

                    def release(b=buf, s=vs):
                        owner[b] = None
                        v_held[s] = None
                    sim.at(done, release)
                    yield ("delay", max(0, start - sim.t) + sim.r(50, 200))
                    sim.commit("pv", v_empty[vs])
                    vjob += 1
                else:
                    assert owner[buf] == ("m", n), ("first-pass buffer handed back early", buf, owner[buf], n)
                    owner[buf] = None
                sim.commit("pv", free[buf])
                yield ("delay", sim.r(30, 80))
                n += 1
            last = max(sim.last_mma_done.get("pv", 0), sim.t)
            sim.at(last, (lambda: o_busy.__setitem__(0, True)))
            sim.commit("pv", o_ready)
            yield ("delay", sim.r(30, 80))

    def softmax(group, warp):
        n_x = 0
        state = {"n": group}              # this group's next job, numbered over the CTA

        def exchange():
            nonlocal n_x
            xchg.arrive(sim)
            yield ("wait", xchg, n_x & 1)
            n_x += 1

        for i in range(tiles):
            j = (group - i * jobs) & 1
            assert i * jobs + j == state["n"], ("job numbering", i, j, state["n"])
            while j < jobs:
                n, buf = state["n"], state["n"] % buffers
                if passes == 2 and j >= first_p2 and j - 2 < first_p2:
                    yield from exchange()                  # row maxima of the two groups
                yield ("wait", s_ready[buf], (n // buffers) & 1)
                assert owner[buf] is not None and owner[buf][1] == n, ("softmax read", buf, owner[buf], n)
                yield ("delay", sim.r(400, 1400))
                if warp == 0:
                    owner[buf] = ("p" if j >= first_p2 else "m", n)
                wg_done[buf].arrive(sim)
                state["n"] += 2
                j += 2
            yield from exchange()                          # row sums
            yield ("wait", o_ready, i & 1)
            yield ("delay", sim.r(200, 600))
            if group == 0 and warp == 0:
                o_busy[0] = False
            o_free.arrive(sim)

    sim.spawn("producer", producer())
    sim.spawn("s", s_issuer())
    sim.spawn("pv", pv_issuer())
    for g in range(2):
        for w in range(4):
            sim.spawn("softmax%d%d" % (g, w), softmax(g, w))
    return sim.run()


class Resource:
    """A buffer with one content tag; reads must see the expected tag, and an overwrite must come after the last read
    (an MMA reads until it completes) has ended."""
    def __init__(self, name):
        self.name, self.tag, self.busy_until = name, None, 0

    def read(self, sim, tag, until=None):
        assert self.tag == tag, ("%s read" % self.name, self.tag, tag)
        self.busy_until = max(self.busy_until, sim.t if until is None else until)

    def write(self, sim, tag, at=None):
        assert sim.t >= self.busy_until, ("%s overwritten while it is read" % self.name, self.tag, tag, sim.t, self.busy_until)
        if at is None:
            self.tag = tag
        else:
            self.tag = ("in flight", tag)
            sim.at(at, (lambda: setattr(self, "tag", tag)))


def single_shot_backward_kernel(seed, t_begin, n_tiles, tiles_per_head, mma_done_count=2, softmax_waits_for_products=True):
    """attn_bwd_pooled_tc_kernel: tiles [t_begin, t_begin + n_tiles) of one CTA; a parent is two tiles (even, odd), a head is
    tiles_per_head tiles (even).  Two MMA-issuing threads: A = S, dP, dQ; B = the three transposed products.
    The last two arguments break the protocol on purpose (tests of the model itself): mma_done counting only thread A's
    commit, and softmax warps that overwrite P / dS without waiting for the previous tile's products."""
    sim = Sim(seed)
    full = [Barrier("full%d" % i, 1) for i in range(2)]
    mma_done = [Barrier("mma_done%d" % i, mma_done_count) for i in range(2)]
    v_free = [Barrier("v_free%d" % i, 1) for i in range(2)]
    s_ready, dp_ready, out_ready = Barrier("s_ready", 1), Barrier("dp_ready", 1), Barrier("out_ready", 2)
    s_consumed, pds_ready = Barrier("s_consumed", 12), Barrier("pds_ready", 12)
    dq_free, acc_free = Barrier("dq_free", 4), Barrier("acc_free", 4)
    stage = [Resource("Q/dO stage %d" % i) for i in range(2)]
    k1 = [Resource("K1 buffer %d" % i) for i in range(2)]
    v1, kv2 = Resource("V1"), Resource("K2/V2")
    scores, pds, dq = Resource("S/dP columns"), Resource("P/dS tiles"), Resource("dQ columns")
    acc1, acc2 = Resource("level-1 accumulators"), Resource("level-2 accumulators")
    tile_of = lambda i: t_begin + i
    parent_of = lambda i: tile_of(i) >> 1
    head_of = lambda i: tile_of(i) // tiles_per_head

    def producer():
        for i in range(n_tiles):
            s, tile = i & 1, tile_of(i)
            new_parent = i == 0 or tile % 2 == 0
            new_head = i == 0 or tile % tiles_per_head == 0
            if i >= 2:
                yield ("wait", mma_done[s], ((i - 2) >> 1) & 1)
            if i >= 1 and new_head:
                yield ("wait", mma_done[(i - 1) & 1], ((i - 1) >> 1) & 1)
            land = sim.t + sim.r(500, 1500)
            stage[s].write(sim, tile, at=land)
            if new_head:
                kv2.write(sim, head_of(i), at=land)
            if new_parent:
                k1[parent_of(i) & 1].write(sim, parent_of(i), at=land)
                if i >= 1:
                    yield ("wait", v_free[(i - 1) & 1], ((i - 1) >> 1) & 1)
                land = max(land, sim.t + sim.r(500, 1500))
                v1.write(sim, parent_of(i), at=land)
            sim.at(land, (lambda b=full[s]: b.arrive(sim)))
            yield ("delay", sim.r(20, 80))

    def issuer_a():
        def issue_s(i):
            s = i & 1
            yield ("wait", full[s], (i >> 1) & 1)
            start, done = sim.mma("A", 384)
            stage[s].read(sim, tile_of(i), done)
            k1[parent_of(i) & 1].read(sim, parent_of(i), done)
            kv2.read(sim, head_of(i), done)
            scores.write(sim, ("S", i), at=done)
            yield ("delay", max(0, start - sim.t) + sim.r(50, 200))
            sim.commit("A", s_ready)

        if n_tiles > 0:
            yield from issue_s(0)
        for i in range(n_tiles):
            s, tile = i & 1, tile_of(i)
            yield ("wait", s_consumed, i & 1)
            start, done = sim.mma("A", 384)
            stage[s].read(sim, tile, done)
            v1.read(sim, parent_of(i), done)
            kv2.read(sim, head_of(i), done)
            scores.write(sim, ("dP", i), at=done)
            yield ("delay", max(0, start - sim.t) + sim.r(50, 200))
            sim.commit("A", dp_ready)
            sim.commit("A", v_free[s])
            yield ("wait", pds_ready, i & 1)
            next_early = i + 1 < n_tiles and (tile + 1) % tiles_per_head != 0
            if next_early:
                yield from issue_s(i + 1)
            if i > 0:
                yield ("wait", dq_free, (i - 1) & 1)
            start, done = sim.mma("A", 576)
            pds.read(sim, i, done)
            k1[parent_of(i) & 1].read(sim, parent_of(i), done)
            kv2.read(sim, head_of(i), done)
            dq.write(sim, i, at=done)
            yield ("delay", max(0, start - sim.t) + sim.r(50, 200))
            sim.commit("A", out_ready)
            sim.commit("A", mma_done[s])
            if not next_early and i + 1 < n_tiles:
                yield from issue_s(i + 1)

    def issuer_b():
        parents_done = 0
        for i in range(n_tiles):
            s, tile = i & 1, tile_of(i)
            yield ("wait", pds_ready, i & 1)
            fresh1 = not (i > 0 and tile % 2 == 1)
            fresh2 = not (i > 0 and tile % tiles_per_head != 0)
            if fresh1 and parents_done > 0:
                yield ("wait", acc_free, (parents_done - 1) & 1)
            start, done = sim.mma("B", 1280)
            pds.read(sim, i, done)
            stage[s].read(sim, tile, done)
            if fresh1:
                acc1.write(sim, parent_of(i))
            else:
                acc1.read(sim, parent_of(i))
            if fresh2:
                acc2.write(sim, head_of(i))
            else:
                acc2.read(sim, head_of(i))
            acc1.busy_until = max(acc1.busy_until, 0)
            yield ("delay", max(0, start - sim.t) + sim.r(50, 300))
            sim.commit("B", out_ready)
            if mma_done_count == 2:
                sim.commit("B", mma_done[s])
            if tile % 2 == 1 or i == n_tiles - 1:
                parents_done += 1

    def drain(warp):
        for i in range(n_tiles):
            tile = tile_of(i)
            parent_end = tile % 2 == 1 or i == n_tiles - 1
            yield ("wait", out_ready, i & 1)
            dq.read(sim, i)
            yield ("delay", sim.r(150, 400))
            dq.busy_until = max(dq.busy_until, sim.t)
            dq_free.arrive(sim)
            if not parent_end:
                continue
            acc1.read(sim, parent_of(i))
            if i == n_tiles - 1 or (tile + 1) % tiles_per_head == 0:
                acc2.read(sim, head_of(i))
            yield ("delay", sim.r(300, 900))
            acc1.busy_until = max(acc1.busy_until, sim.t)
            acc2.busy_until = max(acc2.busy_until, sim.t)
            acc_free.arrive(sim)

    def softmax(warp):
        for i in range(n_tiles):
            yield ("wait", s_ready, i & 1)
            scores.read(sim, ("S", i))
            yield ("delay", sim.r(200, 500))
            scores.busy_until = max(scores.busy_until, sim.t)
            s_consumed.arrive(sim)
            if i > 0 and softmax_waits_for_products:
                yield ("wait", out_ready, (i - 1) & 1)
            if warp == 0:
                pds.write(sim, ("being written", i))
            yield ("delay", sim.r(100, 300))
            yield ("wait", dp_ready, i & 1)
            scores.read(sim, ("dP", i))
            yield ("delay", sim.r(300, 700))
            scores.busy_until = max(scores.busy_until, sim.t)
            if warp == 0:
                pds.tag = i
            pds_ready.arrive(sim)

    sim.spawn("producer", producer())
    sim.spawn("A", issuer_a())
    sim.spawn("B", issuer_b())
    for w in range(4):
        sim.spawn("drain%d" % w, drain(w))
    for w in range(12):
        sim.spawn("softmax%d" % w, softmax(w))
    return sim.run()


def outcome(fn, *args, **kw):
    try:
        return fn(*args, **kw)
    except AssertionError as e:
        return "hazard: %s" % (e.args[0],)

"""Host model of the barrier protocols of the head_dim-128 attention kernels.

The kernels (csrc/attention.cu: ``attn_fwd2_kernel``, ``attn_bwd_dq2_kernel``, ``attn_bwd_dkv2_kernel``) are warp-specialised: a TMA
producer, a single-thread MMA issuer and eight softmax warps hand shared-memory stages and tensor-memory regions
to one another through mbarriers that are waited on by phase parity.  This file restates each role's sequence of
waits, arrivals, loads and MMAs, runs the roles under randomly chosen interleavings (loads and MMAs complete
asynchronously, MMAs in issue order) and checks for every step count that

* nothing deadlocks (a parity wait that can never be satisfied would show up as one), and
* every read sees the data it is meant to see: each write tags its buffer with (what, step), each read asserts
  the tag - an MMA that overwrites S before the threads have read it, or a load that lands in a stage an MMA
  still needs, fails the assertion.

It is a model of the protocol, not of the arithmetic; the kernels themselves are tested on the GPU against fp32
PyTorch (tests/test_gpu_ops.py).
"""
import random

import pytest

WARPS = range(8)      # softmax warps: warp w owns the 32 rows of quarter w % 4 in column half w // 4


class Bar:
    def __init__(self, count):
        self.count, self.pending, self.phase = count, count, 0

    def arrive(self):
        self.pending -= 1
        assert self.pending >= 0, "more arrivals than the barrier expects in one phase"
        if self.pending == 0:
            self.pending, self.phase = self.count, self.phase + 1

    def passed(self, parity):          # mbarrier.try_wait.parity: true once the phase with this parity completed
        return (self.phase & 1) != parity


class Machine:
    """Roles are generators that yield ('wait', bar, parity) or None (a scheduling point).  ``pipe`` is the
    in-order tensor pipe, ``loads`` the TMA requests in flight."""

    def __init__(self, seed):
        self.rng = random.Random(seed)
        self.mem = {}
        self.pipe, self.loads = [], []

    def write(self, buf, tag):
        self.mem[buf] = tag

    def read(self, buf, tag):
        assert self.mem.get(buf) == tag, f"{buf}: expected {tag}, found {self.mem.get(buf)}"

    def mma(self, reads, writes):
        self.pipe.append(("mma", reads, writes))

    def commit(self, *bars):
        for b in bars:
            self.pipe.append(("commit", b))

    def load(self, buf, tag, bar):
        self.loads.append((buf, tag, bar))

    def run(self, roles):
        roles = [[r, None] for r in roles]
        for r in roles:
            r[1] = next(r[0], "done")
        steps = 0
        while True:
            steps += 1
            assert steps < 200000, "model did not terminate"
            choices = []
            for i, (gen, st) in enumerate(roles):
                if st == "done":
                    continue
                if st is None or (st[0] == "wait" and st[1].passed(st[2])):
                    choices.append(("role", i))
            if self.pipe:
                choices.append(("pipe", 0))
            for i in range(len(self.loads)):
                choices.append(("load", i))
            if not choices:
                assert all(st == "done" for _, st in roles), \
                    "deadlock: " + str([st for _, st in roles if st != "done"][0][2:])
                return
            kind, i = self.rng.choice(choices)
            if kind == "role":
                roles[i][1] = next(roles[i][0], "done")
            elif kind == "pipe":
                item = self.pipe.pop(0)
                if item[0] == "mma":
                    for buf, tag in item[1]:
                        self.read(buf, tag)
                    for buf, tag in item[2]:
                        self.write(buf, tag)
                else:
                    item[1].arrive()
            else:
                buf, tag, bar = self.loads.pop(i)
                self.write(buf, tag)
                bar.arrive()


def run_dq2(nblk, seed, ds_barriers=2):
    """TMEM: S | dP x 2 | dQ.  K: 3 stages (held until the step's dQ MMAs), V: 2 stages.  ``ds_barriers`` is the
    number of barriers on which the threads announce dS: the kernel has one per dP buffer."""
    m = Machine(seed)
    qdo = Bar(1)
    k_full, k_empty = [Bar(1) for _ in range(3)], [Bar(1) for _ in range(3)]
    v_full, v_empty = [Bar(1) for _ in range(2)], [Bar(1) for _ in range(2)]
    s_full, s_free, dq_full = Bar(1), Bar(8), Bar(1)
    dp_full = [Bar(1), Bar(1)]
    ds_full = [Bar(8) for _ in range(ds_barriers)]
    NB = ds_barriers

    def producer():
        m.load("QdO", ("QdO", 0), qdo)
        for j in range(nblk):
            ks, st = j % 3, j & 1
            yield ("wait", k_empty[ks], ((j // 3) & 1) ^ 1)
            m.load(("K", ks), ("K", j), k_full[ks])
            yield ("wait", v_empty[st], ((j >> 1) & 1) ^ 1)
            m.load(("V", st), ("V", j), v_full[st])

    def issuer():
        yield ("wait", qdo, 0)
        yield ("wait", k_full[0], 0)
        m.mma([("QdO", ("QdO", 0)), (("K", 0), ("K", 0))], [("S", ("S", 0))])
        m.commit(s_full)
        yield ("wait", v_full[0], 0)
        m.mma([("QdO", ("QdO", 0)), (("V", 0), ("V", 0))], [(("dP", 0, w), ("dP", 0)) for w in WARPS])
        m.commit(dp_full[0], v_empty[0])
        for j in range(nblk):
            st, nx, ks, kn = j & 1, (j & 1) ^ 1, j % 3, (j + 1) % 3
            if j + 1 < nblk:
                yield ("wait", k_full[kn], ((j + 1) // 3) & 1)
                yield ("wait", v_full[nx], ((j + 1) >> 1) & 1)
                yield ("wait", s_free, j & 1)
                m.mma([(("K", kn), ("K", j + 1))], [("S", ("S", j + 1))])
                m.commit(s_full)
                m.mma([(("V", nx), ("V", j + 1))], [(("dP", nx, w), ("dP", j + 1)) for w in WARPS])
                m.commit(dp_full[nx], v_empty[nx])
            yield ("wait", ds_full[j % NB], (j // NB) & 1)
            m.mma([(("dP", st, w), ("dS", j)) for w in WARPS] + [(("K", ks), ("K", j))], [("dQ", ("dQ", j))])
            m.commit(k_empty[ks])
        m.commit(dq_full)

    def softmax(h):                                   # warp h owns its rows and column half of every accumulator
        for j in range(nblk):
            yield ("wait", s_full, j & 1)
            m.read("S", ("S", j))
            s_free.arrive()
            yield None
            yield ("wait", dp_full[j & 1], (j >> 1) & 1)
            m.read(("dP", j & 1, h), ("dP", j))
            yield None
            m.write(("dP", j & 1, h), ("dS", j))
            ds_full[j % NB].arrive()
        yield ("wait", dq_full, 0)
        m.read("dQ", ("dQ", nblk - 1))

    m.run([producer(), issuer()] + [softmax(w) for w in WARPS])


def run_dkv2(niter, seed, q_stages=2):
    """TMEM: S^T | dP^T | dV | dK (single buffers).  Q: ``q_stages`` stages with the row statistics, dO: 2."""
    m = Machine(seed)
    NQ = q_stages
    kv = Bar(1)
    q_full, q_empty, stat_full = ([Bar(1) for _ in range(NQ)] for _ in range(3))
    do_full, do_empty = [Bar(1), Bar(1)], [Bar(1), Bar(1)]
    st_full, dpt_full, p_full, ds_full, acc_full = Bar(1), Bar(1), Bar(8), Bar(8), Bar(1)

    def producer():
        m.load("KV", ("KV", 0), kv)
        for it in range(niter):
            qs, os_ = it % NQ, it & 1
            yield ("wait", q_empty[qs], ((it // NQ) & 1) ^ 1)
            m.load(("Q", qs), ("Q", it), q_full[qs])
            m.write(("stat", qs), ("stat", it))
            stat_full[qs].arrive()
            yield ("wait", do_empty[os_], ((it >> 1) & 1) ^ 1)
            m.load(("dO", os_), ("dO", it), do_full[os_])

    def issuer():
        yield ("wait", kv, 0)
        yield ("wait", q_full[0], 0)
        m.mma([(("Q", 0), ("Q", 0))], [(("ST", w), ("ST", 0)) for w in WARPS])
        m.commit(st_full)
        yield ("wait", do_full[0], 0)
        m.mma([(("dO", 0), ("dO", 0))], [(("DPT", w), ("DPT", 0)) for w in WARPS])
        m.commit(dpt_full)
        for it in range(niter):
            qs, qn, os_, on = it % NQ, (it + 1) % NQ, it & 1, (it & 1) ^ 1
            yield ("wait", p_full, it & 1)
            m.mma([(("ST", w), ("PT", it)) for w in WARPS] + [(("dO", os_), ("dO", it))], [("dV", ("dV", it))])
            m.commit(do_empty[os_])
            if it + 1 < niter:
                yield ("wait", q_full[qn], ((it + 1) // NQ) & 1)
                m.mma([(("Q", qn), ("Q", it + 1))], [(("ST", w), ("ST", it + 1)) for w in WARPS])
                m.commit(st_full)
            yield ("wait", ds_full, it & 1)
            m.mma([(("DPT", w), ("dST", it)) for w in WARPS] + [(("Q", qs), ("Q", it))], [("dK", ("dK", it))])
            m.commit(q_empty[qs])
            if it + 1 < niter:
                yield ("wait", do_full[on], ((it + 1) >> 1) & 1)
                m.mma([(("dO", on), ("dO", it + 1))], [(("DPT", w), ("DPT", it + 1)) for w in WARPS])
                m.commit(dpt_full)
        m.commit(acc_full)

    def softmax(h):                                   # warp h owns its rows and column half of S^T and dP^T
        for it in range(niter):
            qs = it % NQ
            yield ("wait", stat_full[qs], (it // NQ) & 1)
            yield ("wait", st_full, it & 1)
            m.read(("ST", h), ("ST", it))
            m.read(("stat", qs), ("stat", it))
            yield None
            m.write(("ST", h), ("PT", it))
            p_full.arrive()
            yield ("wait", dpt_full, it & 1)
            m.read(("DPT", h), ("DPT", it))
            m.read(("stat", qs), ("stat", it))
            yield None
            m.write(("DPT", h), ("dST", it))
            ds_full.arrive()
        yield ("wait", acc_full, 0)
        m.read("dV", ("dV", niter - 1))
        m.read("dK", ("dK", niter - 1))

    m.run([producer(), issuer()] + [softmax(w) for w in WARPS])


def run_fwd2(nb, seed):
    """Forward, two 128-query tiles per CTA (``attn_fwd2_kernel``).  TMEM: S_0 | S_1 | O_0 | O_1; K and V: 2 stages
    shared by the tiles.  ``nb[t]`` = key blocks tile t visits (tile 0 may visit fewer).  Warps 4t..4t+3 own tile t."""
    m = Machine(seed)
    nblk = max(nb)
    q_full = Bar(1)
    k_full, k_empty, v_full, v_empty = ([Bar(1), Bar(1)] for _ in range(4))
    s_full, pv_done = [Bar(1), Bar(1)], [Bar(1), Bar(1)]
    p_full = [Bar(4), Bar(4)]
    tile_warps = lambda t: range(4 * t, 4 * t + 4)

    def producer():
        m.load("Q", ("Q", 0), q_full)
        for j in range(nblk):
            st, par = j & 1, ((j >> 1) & 1) ^ 1
            yield ("wait", k_empty[st], par)
            m.load(("K", st), ("K", j), k_full[st])
            yield ("wait", v_empty[st], par)
            m.load(("V", st), ("V", j), v_full[st])

    def issue_s(t, j):
        m.mma([("Q", ("Q", 0)), (("K", j & 1), ("K", j))], [(("S", w), ("S", j)) for w in tile_warps(t)])
        m.commit(s_full[t])

    def issuer():
        yield ("wait", q_full, 0)
        yield ("wait", k_full[0], 0)
        for t in range(2):
            if nb[t] > 0:
                issue_s(t, 0)
        m.commit(k_empty[0])
        for j in range(nblk):
            st = j & 1
            yield ("wait", v_full[st], (j >> 1) & 1)
            if j + 1 < nblk:
                yield ("wait", k_full[(j + 1) & 1], ((j + 1) >> 1) & 1)
            for t in range(2):
                if j >= nb[t]:
                    continue
                yield ("wait", p_full[t], j & 1)
                # O_t += P_t V_j: reads the rows the threads rescaled for this step, leaves O(j)
                reads = [(("S", w), ("P", j)) for w in tile_warps(t)] + [(("V", st), ("V", j))]
                reads += [(("O", w), ("O scaled", j)) for w in tile_warps(t)] if j > 0 else []
                m.mma(reads, [(("O", w), ("O", j)) for w in tile_warps(t)])
                m.commit(pv_done[t])
                if j + 1 < nb[t]:
                    issue_s(t, j + 1)
            if j + 1 < nblk:
                m.commit(k_empty[(j + 1) & 1])
            m.commit(v_empty[st])

    def softmax(w):
        t = w // 4
        for j in range(nb[t]):
            yield ("wait", s_full[t], j & 1)
            m.read(("S", w), ("S", j))
            yield None
            if j > 0:                              # rescale of O: PV(j - 1) must be complete, PV(j) not issued
                m.read(("O", w), ("O", j - 1))
                m.write(("O", w), ("O scaled", j))
                yield None
            m.write(("S", w), ("P", j))
            p_full[t].arrive()
        if nb[t] > 0:
            yield ("wait", pv_done[t], (nb[t] - 1) & 1)
            m.read(("O", w), ("O", nb[t] - 1))

    m.run([producer(), issuer()] + [softmax(w) for w in WARPS])


@pytest.mark.parametrize("nblk", list(range(1, 10)) + [16])
def test_dq_kernel_protocol_has_no_deadlock_and_no_stale_read(nblk):
    for seed in range(40):
        run_dq2(nblk, seed)


@pytest.mark.parametrize("niter", list(range(1, 10)) + [16, 64])
def test_dkv_kernel_protocol_has_no_deadlock_and_no_stale_read(niter):
    for seed in range(40):
        run_dkv2(niter, seed)


@pytest.mark.parametrize("nb1", list(range(1, 10)) + [17])
def test_forward_kernel_protocol_has_no_deadlock_and_no_stale_read(nb1):
    for nb0 in sorted({max(nb1 - 1, 0), nb1}):     # tile 0 ends one key block earlier, or the sequence end cuts both
        for seed in range(25):
            run_fwd2((nb0, nb1), seed)
    for seed in range(25):                         # the sequence ends inside tile 0: tile 1 has no rows
        run_fwd2((nb1, 0), seed)


def test_one_ds_barrier_for_two_dp_buffers_would_mix_phases():
    """Why the dQ kernel has a dS barrier per dP buffer: dS(j + 1) depends only on the threads having read S(j), so
    a fast warpgroup can announce dS(j + 1) before a slow one has announced dS(j).  On a single barrier the two
    arrivals complete one phase and the dQ MMAs would read a half of dS(j) that is not written yet."""
    with pytest.raises(AssertionError):
        for seed in range(200):
            run_dq2(4, seed, ds_barriers=1)


def test_the_model_notices_a_missing_stage():
    """Sanity of the model itself: with the Q stage released too early (one stage, as if the release were
    signalled before the dK MMAs), a load overwrites a tile that is still needed and the tag check fires."""
    with pytest.raises(AssertionError):
        for seed in range(200):
            run_dkv2(6, seed, q_stages=1)

"""Host model of the barrier protocols of the warp-specialised kernels.

The attention kernels (csrc/attention.cu: ``attn_fwd2_kernel``, ``attn_bwd_dq2_kernel``, ``attn_bwd_dkv2_kernel`` and
the 64-key-wide ``attn_fwd_kernel``, ``attn_bwd_dq_kernel``, ``attn_bwd_dkv_kernel``) and the persistent GEMMs
(csrc/gemm_umma.cu: ``umma_gemm_kernel``, ``umma_gemm_pair_kernel``) are warp-specialised: a TMA producer, a
single-thread MMA issuer and softmax / epilogue warps hand shared-memory stages and tensor-memory regions to one
another through mbarriers that are waited on by phase parity.  This file restates each role's sequence of waits,
arrivals, loads and MMAs, runs the roles under randomly chosen interleavings (loads and MMAs complete
asynchronously, MMAs in issue order) and checks for every step count that

* nothing deadlocks (a parity wait that can never be satisfied would show up as one), and
* every read sees the data it is meant to see: each write tags its buffer with (what, step), each read asserts
  the tag - an MMA that overwrites S before the threads have read it, a load that lands in a stage an MMA still
  needs, or a barrier phase completed by arrivals that belong to two different steps, fails the assertion.

It is a model of the protocol, not of the arithmetic; the kernels themselves are tested on the GPU against fp32
PyTorch (tests/test_gpu_ops.py, tests/test_gpu_gemm.py).
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
        # uneven speeds: every other seed makes some roles, the tensor pipe or the loads very slow or very fast,
        # so that one warp can run a whole step ahead of another
        skew = self.rng.random() < 0.5
        speed = lambda: self.rng.choice([0.02, 0.2, 1.0, 1.0, 5.0, 50.0]) if skew else 1.0
        w_role = [speed() for _ in roles]
        w_pipe, w_load = speed(), speed()
        steps = 0
        while True:
            steps += 1
            assert steps < 200000, "model did not terminate"
            choices, weights = [], []
            for i, (gen, st) in enumerate(roles):
                if st == "done":
                    continue
                if st is None or (st[0] == "wait" and st[1].passed(st[2])):
                    choices.append(("role", i))
                    weights.append(w_role[i])
            if self.pipe:
                choices.append(("pipe", 0))
                weights.append(w_pipe)
            for i in range(len(self.loads)):
                choices.append(("load", i))
                weights.append(w_load)
            if not choices:
                assert all(st == "done" for _, st in roles), \
                    "deadlock: " + str([st for _, st in roles if st != "done"][0][2:])
                return
            kind, i = self.rng.choices(choices, weights)[0]
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


# ---------------------------------------------------------------- the 64-key-wide kernels (head_dim 64 path)
W4 = range(4)         # these kernels have four softmax warps (thread = accumulator row)


def run_fwd64(nblk, seed):
    """``attn_fwd_kernel``: TMEM S x 2 | O; K, V: 2 stages; P goes through one shared-memory panel."""
    m = Machine(seed)
    q_full, p_full, pv_full = Bar(1), Bar(4), Bar(1)
    k_full, k_empty, v_full, v_empty, s_full = ([Bar(1), Bar(1)] for _ in range(5))
    s_free = [Bar(4), Bar(4)]

    def producer():
        m.load("Q", ("Q", 0), q_full)
        for j in range(nblk):
            st, par = j & 1, ((j >> 1) & 1) ^ 1
            yield ("wait", k_empty[st], par)
            m.load(("K", st), ("K", j), k_full[st])
            yield ("wait", v_empty[st], par)
            m.load(("V", st), ("V", j), v_full[st])

    def issue_s(j):
        st = j & 1
        yield ("wait", k_full[st], (j >> 1) & 1)
        yield ("wait", s_free[st], ((j >> 1) & 1) ^ 1)
        m.mma([("Q", ("Q", 0)), (("K", st), ("K", j))], [(("S", st, w), ("S", j)) for w in W4])
        m.commit(s_full[st], k_empty[st])

    def issuer():
        yield ("wait", q_full, 0)
        yield from issue_s(0)
        for j in range(nblk):
            if j + 1 < nblk:
                yield from issue_s(j + 1)
            st = j & 1
            yield ("wait", v_full[st], (j >> 1) & 1)
            yield ("wait", p_full, j & 1)
            reads = [(("P", w), ("P", j)) for w in W4] + [(("V", st), ("V", j))]
            reads += [(("O", w), ("O scaled", j)) for w in W4] if j > 0 else []
            m.mma(reads, [(("O", w), ("O", j)) for w in W4])
            m.commit(pv_full, v_empty[st])

    def softmax(w):
        for j in range(nblk):
            st = j & 1
            yield ("wait", s_full[st], (j >> 1) & 1)
            m.read(("S", st, w), ("S", j))
            s_free[st].arrive()
            yield None
            if j > 0:
                yield ("wait", pv_full, (j - 1) & 1)
                m.read(("O", w), ("O", j - 1))
                m.write(("O", w), ("O scaled", j))
                yield None
            m.write(("P", w), ("P", j))             # the panel PV(j - 1) read: free since pv_full
            p_full.arrive()
        yield ("wait", pv_full, (nblk - 1) & 1)
        m.read(("O", w), ("O", nblk - 1))

    m.run([producer(), issuer()] + [softmax(w) for w in W4])


def run_dq64(nblk, seed):
    """``attn_bwd_dq_kernel``: TMEM (S | dP) x 2 | dQ; K, V: 2 stages; dS goes through one shared-memory panel
    that ``ds_free`` hands back after the step's dQ MMAs."""
    m = Machine(seed)
    qdo, ds_full, ds_free, dq_full = Bar(1), Bar(4), Bar(1), Bar(1)
    k_full, k_empty, v_full, v_empty, sdp_full = ([Bar(1), Bar(1)] for _ in range(5))

    def producer():
        m.load("QdO", ("QdO", 0), qdo)
        for j in range(nblk):
            st, par = j & 1, ((j >> 1) & 1) ^ 1
            yield ("wait", k_empty[st], par)
            m.load(("K", st), ("K", j), k_full[st])
            yield ("wait", v_empty[st], par)
            m.load(("V", st), ("V", j), v_full[st])

    def issue_sdp(j):
        st, ph = j & 1, (j >> 1) & 1
        yield ("wait", k_full[st], ph)
        yield ("wait", v_full[st], ph)
        m.mma([("QdO", ("QdO", 0)), (("K", st), ("K", j)), (("V", st), ("V", j))],
              [(("SdP", st, w), ("SdP", j)) for w in W4])
        m.commit(sdp_full[st], v_empty[st])

    def issuer():
        yield ("wait", qdo, 0)
        yield from issue_sdp(0)
        for j in range(nblk):
            st = j & 1
            if j + 1 < nblk:
                yield from issue_sdp(j + 1)
            yield ("wait", ds_full, j & 1)
            m.mma([(("dS", w), ("dS", j)) for w in W4] + [(("K", st), ("K", j))], [("dQ", ("dQ", j))])
            m.commit(ds_free, k_empty[st])
        m.commit(dq_full)

    def softmax(w):
        for j in range(nblk):
            yield ("wait", sdp_full[j & 1], (j >> 1) & 1)
            m.read(("SdP", j & 1, w), ("SdP", j))
            yield None
            yield ("wait", ds_free, (j & 1) ^ 1)
            m.write(("dS", w), ("dS", j))
            ds_full.arrive()
        yield ("wait", dq_full, 0)
        m.read("dQ", ("dQ", nblk - 1))

    m.run([producer(), issuer()] + [softmax(w) for w in W4])


def run_dkv64(niter, seed):
    """``attn_bwd_dkv_kernel``: TMEM (S^T | dP^T) x 2 | dV | dK; Q / dO: 2 stages; P^T and dS^T go through
    shared-memory panels that ``pds_free`` hands back; the threads stage the row statistics themselves between
    two CTA-local barriers of the four warps."""
    m = Machine(seed)
    kv, pds_full, pds_free, acc_full = Bar(1), Bar(4), Bar(1), Bar(1)
    q_full, q_empty, st_full = ([Bar(1), Bar(1)] for _ in range(3))
    sync = [Bar(4) for _ in range(2 * niter)]          # bar.sync 1, 128: one single-use barrier per use

    def producer():
        m.load("KV", ("KV", 0), kv)
        for it in range(niter):
            st = it & 1
            yield ("wait", q_empty[st], ((it >> 1) & 1) ^ 1)
            m.load(("QdO", st), ("QdO", it), q_full[st])

    def issue_st(it):
        st = it & 1
        yield ("wait", q_full[st], (it >> 1) & 1)
        m.mma([("KV", ("KV", 0)), (("QdO", st), ("QdO", it))], [(("ST", st, w), ("ST", it)) for w in W4])
        m.commit(st_full[st])

    def issuer():
        yield ("wait", kv, 0)
        yield from issue_st(0)
        for it in range(niter):
            st = it & 1
            if it + 1 < niter:
                yield from issue_st(it + 1)
            yield ("wait", pds_full, it & 1)
            m.mma([(("PdS", w), ("PdS", it)) for w in W4] + [(("QdO", st), ("QdO", it))], [("dKV", ("dKV", it))])
            m.commit(pds_free, q_empty[st])
        m.commit(acc_full)

    def softmax(w):
        for it in range(niter):
            yield ("wait", st_full[it & 1], (it >> 1) & 1)
            sync[2 * it].arrive()
            yield ("wait", sync[2 * it], 0)
            if w < 2:                                  # rows 0-63 stage the statistics of the step's 64 queries
                m.write(("stat", w), ("stat", it))
            sync[2 * it + 1].arrive()
            yield ("wait", sync[2 * it + 1], 0)
            m.read(("ST", it & 1, w), ("ST", it))
            m.read(("stat", 0), ("stat", it))
            yield None
            m.read(("stat", 1), ("stat", it))
            yield ("wait", pds_free, (it & 1) ^ 1)
            m.write(("PdS", w), ("PdS", it))
            pds_full.arrive()
        yield ("wait", acc_full, 0)
        m.read("dKV", ("dKV", niter - 1))

    m.run([producer(), issuer()] + [softmax(w) for w in W4])


# ---------------------------------------------------------------- persistent GEMMs (csrc/gemm_umma.cu)
def run_gemm(k_blocks, stages, seed, ctas=1):
    """``umma_gemm_kernel`` (ctas=1) and ``umma_gemm_pair_kernel`` (ctas=2) for the tiles one CTA (pair) works
    through: ``k_blocks[i]`` reduction blocks for tile i (0 = a group without rows in a batched product: the
    epilogue writes zeros / the addend and the issuer arrives by itself).  Ring of ``stages`` shared-memory
    stages, two accumulators, four epilogue warps per CTA.  In the pair the ``full`` and ``tmem_empty`` barriers
    live in the leader, ``empty`` and ``tmem_full`` exist in both CTAs and get the leader's commits."""
    m = Machine(seed)
    C = range(ctas)
    full = [Bar(1 + ctas) for _ in range(stages)]         # the leader's expect_tx + one load group per CTA
    empty = [[Bar(1) for _ in range(stages)] for _ in C]
    tmem_full = [[Bar(1), Bar(1)] for _ in C]
    tmem_empty = [Bar(4 * ctas), Bar(4 * ctas)]

    def producer(c):
        s, ph, n = 0, 0, 0
        for i, kb_n in enumerate(k_blocks):
            for kb in range(kb_n):
                yield ("wait", empty[c][s], ph ^ 1)
                if c == 0:
                    full[s].arrive()                      # arrive.expect_tx
                m.load(("stage", c, s), ("AB", n), full[s])
                n += 1
                s += 1
                if s == stages:
                    s, ph = 0, ph ^ 1

    def issuer():
        s, ph, n = 0, 0, 0
        for i, kb_n in enumerate(k_blocks):
            acc, acc_ph = i & 1, (i >> 1) & 1
            yield ("wait", tmem_empty[acc], acc_ph ^ 1)
            for kb in range(kb_n):
                yield ("wait", full[s], ph)
                reads = [(("stage", c, s), ("AB", n)) for c in C]
                if kb > 0:
                    reads += [(("acc", c, acc, w), ("acc", i, kb - 1)) for c in C for w in W4]
                m.mma(reads, [(("acc", c, acc, w), ("acc", i, kb)) for c in C for w in W4])
                m.commit(*[empty[c][s] for c in C])
                n += 1
                s += 1
                if s == stages:
                    s, ph = 0, ph ^ 1
            if kb_n > 0:
                m.commit(*[tmem_full[c][acc] for c in C])
            else:
                for c in C:
                    tmem_full[c][acc].arrive()

    def epilogue(c, w):
        for i, kb_n in enumerate(k_blocks):
            acc, acc_ph = i & 1, (i >> 1) & 1
            yield ("wait", tmem_full[c][acc], acc_ph)
            if kb_n > 0:
                m.read(("acc", c, acc, w), ("acc", i, kb_n - 1))
                yield None
                m.read(("acc", c, acc, w), ("acc", i, kb_n - 1))      # later slabs of the same tile
            tmem_empty[acc].arrive()

    m.run([producer(c) for c in C] + [issuer()] + [epilogue(c, w) for c in C for w in W4])


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


@pytest.mark.parametrize("n", list(range(1, 8)) + [12, 33])
def test_the_64_wide_kernels_have_no_deadlock_and_no_stale_read(n):
    for seed in range(25):
        run_fwd64(n, seed)
        run_dq64(n, seed)
        run_dkv64(n, seed)


@pytest.mark.parametrize("ctas", [1, 2])
@pytest.mark.parametrize("stages", [2, 4, 6])
def test_gemm_ring_and_accumulator_hand_off(ctas, stages):
    rng = random.Random(stages * 10 + ctas)
    shapes = [[1], [3], [1, 1, 1, 1, 1], [2, 0, 5, 0, 0, 1], [0], [0, 0, 0], [32, 2, 32], [7] * 9]
    shapes += [[rng.choice([0, 1, 2, 3, 9]) for _ in range(rng.randint(1, 8))] for _ in range(6)]
    for kbs in shapes:
        for seed in range(12):
            run_gemm(kbs, stages, seed, ctas=ctas)


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

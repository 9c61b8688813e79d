"""A CPU model of the hand-off protocol of the int4 TMEM kernel (csrc/w4gemm_tmem.cu): the roles of one CTA
(two dequant sets, two MMA issuers, the activation producer, the epilogue) run as coroutines under a random
scheduler, with mbarriers that behave like the hardware's (a phase counter; a parity wait passes when the
barrier's current phase parity differs from the one asked for). Every wait names the completion it means
(barrier, phase index); the model fails if a wait ever passes before that completion has happened, which is
what a parity wait does when its waiter skipped a phase of the barrier.

The index arithmetic is the kernel's: chunks visited in the order tail segment, head segment, whole
super-strips; chunk i belongs to set i % 2, TMEM / activation stage i % 3, barrier set i % 6; accumulator
(set, segment-of-the-set % buffers). The test also runs the arrangement the kernel had first (one barrier per
stage) and checks that the model catches it: a set that runs ahead of the other passes a wait early.
"""

import random

import pytest

STAGES, SETS = 3, 2


class Barrier:
    def __init__(self, count):
        self.count, self.pending, self.phase = count, count, 0  # phase = completed phases so far

    def arrive(self):
        self.pending -= 1
        if self.pending == 0:
            self.pending, self.phase = self.count, self.phase + 1

    def parity_wait_passes(self, parity):
        return (self.phase & 1) != parity  # the phase of that parity is not the one in progress


def visit_order(f0, f1, chunks):
    """The kernel's Visit: (order of chunk ids, set of positions that end a K segment)."""
    h_end = f0 if f0 % chunks == 0 else min(f1, (f0 // chunks + 1) * chunks)
    t_start = f1 if f1 % chunks == 0 else max(h_end, (f1 // chunks) * chunks)
    order = list(range(t_start, f1)) + list(range(f0, h_end)) + list(range(h_end, t_start))
    lt, lh, n = f1 - t_start, h_end - f0, f1 - f0
    ends = {i for i in range(n) if order[i] % chunks == chunks - 1 or i in (n - 1, lt - 1, lt + lh - 1)}
    return order, ends


def run_model(n, ends, acc_bufs, bars_per_stage, seed):
    """Returns None, or a description of the first wait that passed before its completion."""
    rng = random.Random(seed)
    nb = STAGES * bars_per_stage                       # 3 (one barrier per stage) or 6 (per stage and set)
    a_ready = [Barrier(1) for _ in range(nb)]          # one arrival stands for the set's eight warps
    a_free = [Barrier(1) for _ in range(nb)]
    act_full = [Barrier(1) for _ in range(nb)]
    acc_ready = [[Barrier(1) for _ in range(acc_bufs)] for _ in range(SETS)]
    acc_free = [[Barrier(1) for _ in range(acc_bufs)] for _ in range(SETS)]
    uses = {}                                          # (id(barrier)) -> completions requested so far, to name phases
    fault = []

    def bar_index(i):
        return i % nb

    def wait(bar, k, what):
        """Generator: wait for completion number k (0-based) of `bar`, the way the kernel does: by parity."""
        while not bar.parity_wait_passes(k & 1):
            yield
        if bar.phase < k + 1 and not fault:
            fault.append(f"{what}: passed at phase {bar.phase}, meant completion {k}")

    def segments_of(s):
        """For set s: list of (first, last) positions of its chunks per segment it contributes to."""
        out, start, mine = [], 0, []
        for i in range(n):
            if i % SETS == s:
                mine.append(i)
            if i in ends:
                if mine:
                    out.append((mine[0], mine[-1]))
                mine = []
                start = i + 1
        return out

    def dequant(s):
        for i in range(s, n, SETS):
            yield                                          # codes land, arithmetic
            if i >= STAGES:
                yield from wait(a_free[bar_index(i - STAGES)], (i - STAGES) // nb, f"dequant set {s} chunk {i} a_free")
            yield                                          # TMEM stores
            a_ready[bar_index(i)].arrive()

    def producer():
        for i in range(n):
            if i >= STAGES:
                yield from wait(a_free[bar_index(i - STAGES)], (i - STAGES) // nb, f"producer chunk {i} a_free")
            yield
            act_full[bar_index(i)].arrive()

    def mma(s):
        segs = segments_of(s)
        seg_first = {a: k for k, (a, _) in enumerate(segs)}
        seg_last = {b: k for k, (_, b) in enumerate(segs)}
        for i in range(s, n, SETS):
            if i in seg_first:
                k = seg_first[i]
                if k >= acc_bufs:
                    yield from wait(acc_free[s][k % acc_bufs], k // acc_bufs - 1, f"mma {s} segment {k} acc_free")
            yield from wait(a_ready[bar_index(i)], i // nb, f"mma {s} chunk {i} a_ready")
            yield from wait(act_full[bar_index(i)], i // nb, f"mma {s} chunk {i} act_full")
            yield                                          # the MMAs run
            a_free[bar_index(i)].arrive()
            if i in seg_last:
                acc_ready[s][seg_last[i] % acc_bufs].arrive()

    def epilogue():
        counts, i0 = [0] * SETS, 0
        for i in range(n):
            if i not in ends:
                continue
            for s in range(SETS):
                mine = (i + 2 - s) // 2 - (i0 + 1 - s) // 2       # the kernel's count of chunks of parity s in i0 .. i
                assert mine == len([j for j in range(i0, i + 1) if j % SETS == s])
                if mine == 0:
                    continue
                k = counts[s]
                yield from wait(acc_ready[s][k % acc_bufs], k // acc_bufs, f"epilogue segment {k} of set {s} acc_ready")
                yield
                acc_free[s][k % acc_bufs].arrive()
                counts[s] += 1
            i0 = i + 1

    tasks = [dequant(0), dequant(1), producer(), mma(0), mma(1), epilogue()]
    weights = [rng.choice((1, 1, 1, 8)) for _ in tasks]     # some roles run much faster than others
    alive = list(range(len(tasks)))
    for _ in range(200000):
        if not alive or fault:
            break
        t = rng.choices(alive, [weights[a] for a in alive])[0]
        try:
            next(tasks[t])
        except StopIteration:
            alive.remove(t)
    assert fault or not alive, "the model deadlocked"
    return fault[0] if fault else None


CASES = [(0, 24, 16), (5, 29, 16), (9, 33, 16), (15, 40, 16), (3, 12, 16), (7, 8, 16), (2, 120, 56), (31, 47, 8)]


@pytest.mark.parametrize("f0,f1,chunks", CASES)
@pytest.mark.parametrize("acc_bufs", [1, 2])
def test_barrier_sets_indexed_by_chunk_mod_6_never_pass_a_wait_early(f0, f1, chunks, acc_bufs):
    order, ends = visit_order(f0, f1, chunks)
    assert sorted(order) == list(range(f0, f1))
    for seed in range(40):
        assert run_model(len(order), ends, acc_bufs, SETS, seed) is None


def test_one_barrier_per_stage_is_caught_by_the_model():
    """The first arrangement: the two sets each see every other phase of a stage's barriers, and a parity wait
    then passes one phase early for a set that runs ahead (on the GPU: stale weights in one 128-column tile)."""
    order, ends = visit_order(5, 29, 16)
    faults = [run_model(len(order), ends, 1, 1, seed) for seed in range(200)]
    assert any(f is not None for f in faults), "the model should reproduce the early pass"

"""A host-side model of the GEMM kernel's barrier protocol (coda_kernels_b200/csrc/gemm_core.cuh).

The kernel's three roles (TMA producer, MMA issuer, epilogue) talk through phase-tracked mbarriers: `full[s]` /
`empty[s]` per shared-memory stage, `acc_full[a]` / `acc_empty[a]` per TMEM accumulator stage.  This model restates
the index and parity arithmetic of those loops over a tiny mbarrier simulator and runs the roles as interleaved
coroutines.  It checks, without a GPU and without hanging anything, that

* for any number of tiles, k-blocks and stages every stage is filled and consumed in order and every role finishes,
  including the tail waits that keep a CTA from leaving while arrivals are still on their way to it;
* when one role stops making progress (the failure the bounded waits exist for), every other role gives up at a
  wait, the abort code of the wait that really expired survives, and the other CTA of a pair is told once
  (`kErrPeerAbort`) without echoing the signal back.
"""

import itertools

import pytest

K_ERR_EMPTY, K_ERR_FULL, K_ERR_ACC_EMPTY, K_ERR_ACC_FULL, K_ERR_PEER = 1, 2, 3, 4, 5


class MBarrier:
    """Phase bit + pending arrival count, as `mbarrier.init count` / `arrive` / `try_wait.parity` behave."""

    def __init__(self, count: int):
        self.count, self.pending, self.phase = count, count, 0

    def arrive(self):
        self.pending -= 1
        assert self.pending >= 0, "more arrivals than the barrier expects in one phase"
        if self.pending == 0:
            self.pending, self.phase = self.count, self.phase ^ 1

    def done(self, parity: int) -> bool:
        # try_wait.parity succeeds once the phase with that parity has completed
        return self.phase != parity


class Cta:
    def __init__(self, stages: int):
        self.full = [MBarrier(1) for _ in range(stages)]
        self.empty = [MBarrier(1) for _ in range(stages)]
        self.acc_full = [MBarrier(1) for _ in range(2)]
        self.acc_empty = [MBarrier(1) for _ in range(2)]  # one epilogue "warp" in the model
        self.abort = 0
        self.peer = None
        self.log = []


def wait(cta: Cta, bar: MBarrier, parity: int, code: int, limit: int):
    """Bounded wait as a coroutine: yields while spinning; returns False on abort or when the limit runs out."""
    spins = 0
    while not bar.done(parity):
        if cta.abort:
            return False
        spins += 1
        if spins > limit:
            cta.abort = code
            return False
        yield
    return True


def notify_and_drain(cta: Cta):
    if cta.peer is not None and cta.abort != K_ERR_PEER:
        if cta.peer.abort == 0:
            cta.peer.abort = K_ERR_PEER
        cta.log.append("notified peer")


def producer(cta: Cta, tiles: int, num_kb: int, stages: int, limit: int, stall_after=None):
    s = ph = 0
    ok = True
    issued = 0
    for _tile in range(tiles):
        for _kb in range(num_kb):
            if stall_after is not None and issued >= stall_after:
                while True:  # this role is stuck: it never issues another load
                    if cta.abort:
                        return
                    yield
            ok = yield from wait(cta, cta.empty[s], ph ^ 1, K_ERR_EMPTY, limit)
            if not ok:
                break
            cta.log.append(("load", s))
            cta.full[s].arrive()  # the TMA transaction completes the phase
            issued += 1
            s += 1
            if s == stages:
                s, ph = 0, ph ^ 1
            yield
        if not ok:
            break
    for _ in range(stages):  # tail: wait until the last commits have arrived
        if not ok:
            break
        ok = yield from wait(cta, cta.empty[s], ph ^ 1, K_ERR_EMPTY, limit)
        s += 1
        if s == stages:
            s, ph = 0, ph ^ 1
    if not ok:
        notify_and_drain(cta)
    cta.log.append("producer done")


def mma(cta: Cta, tiles: int, num_kb: int, stages: int, limit: int, dead: bool = False):
    s = ph = 0
    ok = True
    it = 0
    for _tile in range(tiles):
        acc, aph = it & 1, (it >> 1) & 1
        ok = yield from wait(cta, cta.acc_empty[acc], aph ^ 1, K_ERR_ACC_EMPTY, limit)
        if not ok:
            break
        for _kb in range(num_kb):
            if dead:
                while True:
                    if cta.abort:
                        return
                    yield
            ok = yield from wait(cta, cta.full[s], ph, K_ERR_FULL, limit)
            if not ok:
                break
            cta.log.append(("mma", s))
            cta.empty[s].arrive()  # tcgen05.commit once the MMAs that read the stage retire
            s += 1
            if s == stages:
                s, ph = 0, ph ^ 1
            yield
        if not ok:
            break
        cta.acc_full[acc].arrive()
        it += 1
    for _ in range(2):  # tail: both accumulator stages drained
        if not ok:
            break
        acc, aph = it & 1, (it >> 1) & 1
        ok = yield from wait(cta, cta.acc_empty[acc], aph ^ 1, K_ERR_ACC_EMPTY, limit)
        it += 1
    if not ok:
        notify_and_drain(cta)
    cta.log.append("mma done")


def epilogue(cta: Cta, tiles: int, limit: int):
    for it in range(tiles):
        acc, aph = it & 1, (it >> 1) & 1
        ok = yield from wait(cta, cta.acc_full[acc], aph, K_ERR_ACC_FULL, limit)
        if not ok:
            notify_and_drain(cta)
            break
        cta.log.append(("drain", acc))
        yield
        cta.acc_empty[acc].arrive()
    cta.log.append("epilogue done")


def run(roles, max_steps=200000):
    live = list(roles)
    steps = 0
    while live:
        for r in list(live):
            try:
                next(r)
            except StopIteration:
                live.remove(r)
        steps += 1
        assert steps < max_steps, "the model did not terminate: a role waits forever"


@pytest.mark.parametrize("tiles,num_kb,stages", list(itertools.product([1, 2, 3, 7], [1, 5, 12], [2, 4, 6])))
def test_every_stage_is_filled_and_consumed_in_order(tiles, num_kb, stages):
    cta = Cta(stages)
    run([producer(cta, tiles, num_kb, stages, 10**6), mma(cta, tiles, num_kb, stages, 10**6), epilogue(cta, tiles, 10**6)])
    assert cta.abort == 0
    loads = [e[1] for e in cta.log if isinstance(e, tuple) and e[0] == "load"]
    mmas = [e[1] for e in cta.log if isinstance(e, tuple) and e[0] == "mma"]
    expect = [i % stages for i in range(tiles * num_kb)]
    assert loads == expect and mmas == expect
    assert [e[1] for e in cta.log if isinstance(e, tuple) and e[0] == "drain"] == [i & 1 for i in range(tiles)]
    for done in ("producer done", "mma done", "epilogue done"):
        assert done in cta.log


def test_a_dead_mma_role_ends_every_other_role_and_keeps_the_first_code():
    a, b = Cta(4), Cta(4)
    a.peer, b.peer = b, a
    # CTA a: the MMA issuer never consumes a stage; CTA b is healthy but depends on nothing of a in this model, so
    # the only way it stops early is the peer notification
    roles = [producer(a, 3, 8, 4, 50), mma(a, 3, 8, 4, 50, dead=True), epilogue(a, 3, 50),
             producer(b, 10**4, 8, 4, 10**6), mma(b, 10**4, 8, 4, 10**6), epilogue(b, 10**4, 10**6)]
    run(roles)
    assert a.abort in (K_ERR_EMPTY, K_ERR_ACC_FULL), "the code of a wait that really expired survives in the CTA where it happened"
    assert b.abort == K_ERR_PEER, "the other CTA of the pair learns of the abort instead of running into its own limits"
    assert "notified peer" in a.log and "notified peer" not in b.log, "a CTA that only follows its peer does not echo the signal"


def test_a_stalled_producer_is_reported_by_the_mma_role():
    cta = Cta(3)
    run([producer(cta, 4, 6, 3, 10**6, stall_after=5), mma(cta, 4, 6, 3, 40), epilogue(cta, 4, 10**6)])
    assert cta.abort == K_ERR_FULL
    assert sum(1 for e in cta.log if isinstance(e, tuple) and e[0] == "mma") == 5


# ------------------------------------------------------------------------------------------------ tail-split schedule
# Host restatement of `plan_tail_split` (coda_kernels_b200/csrc/gemm_host.cuh), `WorkSchedule::next`
# (csrc/gemm_core.cuh) and the slab arithmetic of `split_finalize_kernel`: every k-block of every tile is done exactly
# once, whole tiles stay whole, each part of a tail tile has its own workspace slab, and the follow-up kernel reads
# exactly the slabs the GEMM wrote.

SPLIT_OVERHEAD_KB = 12


def plan_tail_split(num_tiles: int, num_kb: int, clusters: int):
    tail = num_tiles % clusters
    if tail == 0 or clusters < 2 or num_kb < 16:
        return tail, 1
    best, best_cost = 1, num_kb
    for s in range(2, min(2 * clusters // tail, num_kb // 8, 64) + 1):
        rounds = -(-(tail * s) // clusters)
        cost = rounds * -(-num_kb // s) + SPLIT_OVERHEAD_KB
        if cost < best_cost:
            best, best_cost = s, cost
    return tail, (best if best > 1 and best_cost * 100 <= num_kb * 85 else 1)


def schedule(cluster: int, clusters: int, num_tiles: int, num_kb: int, tail: int, split: int):
    """Items (tile, kb0, kb1, slab) of one cluster, as the kernel's roles enumerate them."""
    split = max(split, 1)
    tail = tail if split > 1 else 0
    full = num_tiles - tail
    items = []
    for i in range(cluster, full + tail * split, clusters):
        if i < full:
            items.append((i, 0, num_kb, -1))
        else:
            j = i - full
            part = j // tail
            items.append((full + j % tail, part * num_kb // split, (part + 1) * num_kb // split, j))
    return items


@pytest.mark.parametrize("num_tiles,num_kb,clusters", [
    (48, 256, 74), (224, 256, 74), (448, 256, 74), (1792, 256, 74), (8, 128, 74), (12, 64, 74), (6, 129, 74), (76, 32, 74),
    (1, 700, 74), (20, 40, 148), (3, 1000, 148), (1, 64, 4),
])
def test_tail_split_schedule_covers_every_k_block_once(num_tiles, num_kb, clusters):
    tail, split = plan_tail_split(num_tiles, num_kb, clusters)
    assert split > 1, "these shapes leave most clusters idle in their last round"
    assert tail * split <= 2 * clusters, "the workspace holds two partial tiles per cluster"
    done, written = {}, {}
    for c in range(clusters):
        for tile, kb0, kb1, slab in schedule(c, clusters, num_tiles, num_kb, tail, split):
            assert 0 <= tile < num_tiles and 0 <= kb0 < kb1 <= num_kb
            assert (slab < 0) == (tile < num_tiles - tail), "whole tiles stay whole; every tail item is a part"
            for kb in range(kb0, kb1):
                assert (tile, kb) not in done
                done[(tile, kb)] = c
            if slab >= 0:
                assert slab < tail * split and slab not in written
                written[slab] = tile
    assert len(done) == num_tiles * num_kb
    # the follow-up kernel adds slabs part * tail + t for tail tile t
    for t in range(tail):
        for part in range(split):
            assert written[part * tail + t] == num_tiles - tail + t
    # what it buys: the last round, in k-blocks
    last_round = -(-(tail * split) // clusters) * -(-num_kb // split)
    assert last_round + SPLIT_OVERHEAD_KB <= 0.85 * num_kb


def test_tail_split_is_left_off_when_it_cannot_pay():
    assert plan_tail_split(1024, 448, 74)[1] == 1   # 62 tail tiles: cutting them in two fills two rounds of half length
    assert plan_tail_split(60, 512, 74)[1] == 1     # same
    assert plan_tail_split(148, 256, 74)[1] == 1    # no tail at all
    assert plan_tail_split(48, 8, 74)[1] == 1       # contraction too short to cut
    assert schedule(3, 74, 200, 10, 52, 1) == [(3, 0, 10, -1), (77, 0, 10, -1), (151, 0, 10, -1)]

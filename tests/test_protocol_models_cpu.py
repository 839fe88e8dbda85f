"""Executable models of the synchronisation protocols the kernels rely on, run on CPU threads with random delays.

The kernels cannot be run under a race detector on this platform, so the protocols themselves are modelled and
exercised here: a schedule that breaks the model's invariant would break the kernel's too.

* low-latency all-reduce with per-CALL epochs (``csrc/comm/allreduce.cu``): every 8-byte unit carries
  ``{data, epoch}``; ranks push into slot ``[epoch & 1][source]`` of every peer and collect only units stamped with
  the current epoch; calls of different sizes follow one another with no other synchronisation;
* mbarrier parity waits (``csrc/attention/*_umma.cu``): a wait for "phase k done" expressed through the phase's
  parity is only correct while the barrier is at most one phase behind k - the model reproduces the early wake-up
  that a barrier two phases behind gives, and shows that the two-step wait used by the kernels does not have it;
* the last-arriver ticket of the split-KV merge (``atomicAdd`` on a per-unit counter that the last arriver resets).
"""
import random
import threading
import time

import pytest


class LLSlots:
    """Receive slots of one rank: ``[parity][source][unit] = (data, epoch)``; a unit is written atomically."""

    def __init__(self, world, units):
        self.s = [[[(0, 0)] * units for _ in range(world)] for _ in range(2)]


def _ll_allreduce_rank(rank, world, slots, calls, out, jitter, rng_seed):
    rng = random.Random(rng_seed)
    epoch = 0
    for call, n in enumerate(calls):
        epoch += 1                      # epochs[0] + 1: one epoch per call, whatever its size
        mine = [(rank + 1) * 1000 + call * 10 + u for u in range(n)]
        par = epoch & 1
        for peer in range(world):       # push
            if peer == rank:
                continue
            for u in range(n):
                if jitter:
                    time.sleep(rng.random() * 1e-5)
                slots[peer].s[par][rank][u] = (mine[u], epoch)
        total = list(mine)              # collect: spin until the unit carries THIS call's epoch
        for src in range(world):
            if src == rank:
                continue
            for u in range(n):
                spins = 0
                while True:
                    data, ep = slots[rank].s[par][src][u]
                    if ep == epoch:
                        break
                    spins += 1
                    assert spins < 2_000_000, "wait ran out"
                    if spins % 64 == 0:
                        time.sleep(0)
                total[u] += data
        out[rank].append(total)


@pytest.mark.parametrize("world", [2, 4])
def test_ll_allreduce_epochs_mixed_sizes(world):
    """Calls of changing size back to back, ranks running at different speeds: every rank gets the sums of the
    right call.  Two parities suffice: a rank can be at most one call ahead of the slowest peer, because it cannot
    finish call c before every peer has pushed call c."""
    units = 8
    calls = [random.Random(7).randint(1, units) for _ in range(60)]
    slots = [LLSlots(world, units) for _ in range(world)]
    out = [[] for _ in range(world)]
    th = [threading.Thread(target=_ll_allreduce_rank, args=(r, world, slots, calls, out, r % 2 == 0, 100 + r))
          for r in range(world)]
    [t.start() for t in th]
    [t.join(60) for t in th]
    assert all(not t.is_alive() for t in th)
    for call, n in enumerate(calls):
        want = [sum((r + 1) * 1000 + call * 10 + u for r in range(world)) for u in range(n)]
        for r in range(world):
            assert out[r][call] == want, (call, r)


def test_ll_allreduce_single_parity_would_mix_calls():
    """The reason for the parity bit, shown on the model: with ONE slot set a fast rank's push for call c + 1 may
    overwrite a unit that a slow rank has not collected for call c yet - the slow rank then never sees epoch c."""
    slot = {"u": (0, 0)}
    # fast rank pushes call 1, then (having collected the slow rank's call 1) pushes call 2 into the same unit
    slot["u"] = (11, 1)
    slot["u"] = (22, 2)
    data, ep = slot["u"]
    assert ep != 1, "the unit of call 1 is gone: a single slot set cannot work"
    # with two parities the unit of call 1 is still there
    slots = {1: (11, 1), 0: (22, 2)}
    assert slots[1 & 1] == (11, 1) and slots[2 & 1] == (22, 2)


class Mbarrier:
    """Phase-parity barrier with one expected arrival per phase (what ``tcgen05.commit`` arrives on)."""

    def __init__(self):
        self.phase = 0          # index of the phase in progress
        self.lock = threading.Lock()

    def arrive(self):
        with self.lock:
            self.phase += 1

    def try_wait_parity(self, parity):
        """True when the phase with this parity is NOT the one in progress - the hardware's test."""
        with self.lock:
            return (self.phase & 1) != parity


def test_parity_wait_two_phases_behind_wakes_early():
    bar = Mbarrier()
    # phases 0 .. k-2 done, the barrier is in phase k-1 (one arrival still missing for it, two for phase k)
    k = 5
    for _ in range(k - 1):
        bar.arrive()
    assert bar.phase == k - 1
    # waiting for "phase k done" by parity alone passes at once - although phase k has not even started
    assert bar.try_wait_parity(k & 1) is True
    # the rule the kernels follow: first wait for phase k-1 (valid: the barrier is at most one phase behind it) ...
    assert bar.try_wait_parity((k - 1) & 1) is False
    bar.arrive()                                   # phase k-1 completes
    assert bar.try_wait_parity((k - 1) & 1) is True
    # ... then for phase k, which now blocks until it really completes
    assert bar.try_wait_parity(k & 1) is False
    bar.arrive()
    assert bar.try_wait_parity(k & 1) is True


def test_parity_wait_pipeline_random_schedule():
    """Producer commits phases 0 .. n-1 with random delays; a consumer that is never more than one phase behind when
    it starts a wait (the kernels guarantee this with a second barrier) observes every phase exactly once, in order."""
    n = 200
    bar = Mbarrier()
    seen = []
    done_flag = threading.Event()
    credit = threading.Semaphore(1)    # the producer may run at most one phase ahead (p_free / s_empty in the kernels)

    def producer():
        rng = random.Random(1)
        for _ in range(n):
            credit.acquire()
            if rng.random() < 0.3:
                time.sleep(rng.random() * 1e-4)
            bar.arrive()
        done_flag.set()

    def consumer():
        rng = random.Random(2)
        for k in range(n):
            spins = 0
            while not bar.try_wait_parity(k & 1):
                spins += 1
                assert spins < 5_000_000
                if spins % 32 == 0:
                    time.sleep(0)
            seen.append((k, bar.phase))
            if rng.random() < 0.3:
                time.sleep(rng.random() * 1e-4)
            credit.release()

    tp, tc = threading.Thread(target=producer), threading.Thread(target=consumer)
    tp.start(); tc.start()
    tp.join(60); tc.join(60)
    assert not tp.is_alive() and not tc.is_alive()
    # when the wait for phase k returned, phase k was complete and phase k + 1 at most in progress
    assert all(k + 1 <= ph <= k + 2 for k, ph in seen), [x for x in seen if not (x[0] + 1 <= x[1] <= x[0] + 2)][:5]


def test_last_arriver_ticket_reset():
    """Split merge: every CTA of a unit publishes its partial, then takes a ticket; exactly one CTA per launch sees
    ``splits - 1`` and resets the counter for the next launch (launches are ordered by the stream)."""
    splits, launches = 9, 50
    counter = [0]
    lock = threading.Lock()
    partials = [None] * splits
    merged = []

    def cta(i, launch, barrier):
        partials[i] = (launch, i)
        with lock:                       # atomicAdd
            t = counter[0]
            counter[0] += 1
        if t == splits - 1:
            assert all(p is not None and p[0] == launch for p in partials), "merge saw a missing / stale partial"
            merged.append(launch)
            counter[0] = 0               # reset by the last arriver only
        barrier.wait()

    for launch in range(launches):
        b = threading.Barrier(splits)
        th = [threading.Thread(target=cta, args=(i, launch, b)) for i in range(splits)]
        random.Random(launch).shuffle(th)
        [t.start() for t in th]
        [t.join(30) for t in th]
        for i in range(splits):
            partials[i] = None
    assert merged == list(range(launches)) and counter[0] == 0

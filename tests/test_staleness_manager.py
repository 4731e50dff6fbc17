"""Capacity arithmetic of the staleness manager."""
import threading

from areal_b200.infra.staleness_manager import StalenessManager


class V:
    def __init__(self, v=0):
        self.v = v

    def get_version(self):
        return self.v


def test_initial_capacity_is_min_of_limits():
    assert StalenessManager(V(0), 10, 4, 2).get_capacity() == 10       # staleness allows 12
    assert StalenessManager(V(0), 100, 4, 2).get_capacity() == 12      # (2+0+1)*4
    assert StalenessManager(V(3), 100, 4, 0).get_capacity() == 16
    assert StalenessManager(V(0), 0, 0, 0).get_capacity() == 1         # degenerate values clamp to 1


def test_lifecycle_counts():
    m = StalenessManager(V(0), 8, 2, 1)
    for _ in range(3):
        m.on_rollout_enqueued()
    m.on_rollout_submitted(); m.on_rollout_submitted()
    s = m.get_stats()
    assert (s.enqueued, s.running) == (1, 2)
    assert m.get_capacity() == min(8 - 2, 4 - 2)
    m.on_rollout_accepted(); m.on_rollout_rejected()
    s = m.get_stats()
    assert (s.accepted, s.rejected, s.running) == (1, 1, 0)
    assert m.get_capacity() == min(8, 4 - 1)   # a rejected sample frees its budget, an accepted one does not


def test_version_advance_increases_capacity():
    v = V(0)
    m = StalenessManager(v, 1000, 32, 2)
    for _ in range(96):
        m.on_rollout_enqueued(); m.on_rollout_submitted()
    assert m.get_capacity() == 0
    for _ in range(96):
        m.on_rollout_accepted()
    assert m.get_capacity() == 0
    v.v = 1
    assert m.get_capacity() == 32
    assert m.get_pending_limit() == 96


def test_capacity_can_go_negative_and_recovery():
    v = V(0)
    m = StalenessManager(v, 4, 2, 0)
    for _ in range(6):
        m.on_rollout_enqueued(); m.on_rollout_submitted()
    assert m.get_capacity() < 0
    m2 = StalenessManager(V(5), 100, 8, 1)
    m2.on_version_recovered(5)
    assert m2.get_stats().accepted == 40
    assert m2.get_capacity() == (1 + 5 + 1) * 8 - 40


def test_thread_safety():
    m = StalenessManager(V(0), 10 ** 6, 1, 10 ** 6)

    def work():
        for _ in range(2000):
            m.on_rollout_enqueued(); m.on_rollout_submitted(); m.on_rollout_accepted()

    ts = [threading.Thread(target=work) for _ in range(8)]
    [t.start() for t in ts]; [t.join() for t in ts]
    s = m.get_stats()
    assert (s.accepted, s.running, s.enqueued) == (16000, 0, 0)


# ---- scenarios: a producer that obeys the capacity never exceeds the staleness bound ------------
import random

import pytest


def _simulate(max_conc, batch, eta, steps, accept_prob, seed):
    """Drive a producer/consumer loop; returns the largest staleness any consumed sample saw."""
    rng = random.Random(seed)
    v = V(0)
    m = StalenessManager(v, max_conc, batch, eta)
    running = []          # version each running sample started at
    done = []             # finished + accepted, waiting for the consumer
    worst = 0
    guard = 0
    while v.v < steps:
        guard += 1
        assert guard < 100_000, "simulation made no progress"
        cap = m.get_capacity()
        assert cap <= max(1, max_conc) - len(running)
        for _ in range(max(0, cap)):
            m.on_rollout_enqueued(); m.on_rollout_submitted()
            running.append(v.v)
        assert m.get_capacity() <= 0
        # a random number of samples finishes, oldest first: the bound is on a sample's position
        # in start order, so it holds exactly when samples are consumed in that order
        n_fin = rng.randint(1, max(1, len(running))) if running else 0
        for _ in range(n_fin):
            born = running.pop(0)
            if rng.random() < accept_prob:
                m.on_rollout_accepted(); done.append(born)
            else:
                m.on_rollout_rejected()
        while len(done) >= batch and v.v < steps:
            consumed, done = done[:batch], done[batch:]
            worst = max(worst, max(v.v - b for b in consumed))
            v.v += 1
        s = m.get_stats()
        assert s.running == len(running) and s.enqueued == 0
        assert s.accepted + s.running <= (eta + v.v + 1) * batch
    return worst


@pytest.mark.parametrize("eta", [0, 1, 4])
@pytest.mark.parametrize("accept_prob", [1.0, 0.6])
def test_simulated_training_respects_staleness_bound(eta, accept_prob):
    for seed in range(5):
        worst = _simulate(max_conc=64, batch=8, eta=eta, steps=30, accept_prob=accept_prob, seed=seed)
        assert worst <= eta


def test_all_rejected_never_consumes_budget():
    m = StalenessManager(V(0), 16, 4, 0)
    for _ in range(50):
        cap = m.get_capacity()
        assert cap == 4
        for _ in range(cap):
            m.on_rollout_enqueued(); m.on_rollout_submitted()
        assert m.get_capacity() == 0
        for _ in range(cap):
            m.on_rollout_rejected()
    s = m.get_stats()
    assert (s.accepted, s.rejected, s.running) == (0, 200, 0)


def test_slow_consumer_stalls_producer_until_version_moves():
    v = V(0)
    m = StalenessManager(v, 1000, 16, 1)
    started = 0
    while m.get_capacity() > 0:
        m.on_rollout_enqueued(); m.on_rollout_submitted(); m.on_rollout_accepted()
        started += 1
    assert started == 32                       # (1 + 0 + 1) * 16
    for _ in range(10):
        assert m.get_capacity() == 0           # nothing more until the trainer steps
    v.v = 2
    assert m.get_capacity() == 32


def test_burst_is_clipped_by_concurrency_then_by_staleness():
    v = V(0)
    m = StalenessManager(v, 8, 4, 3)           # staleness allows 16, concurrency 8
    assert m.get_capacity() == 8
    for _ in range(8):
        m.on_rollout_enqueued(); m.on_rollout_submitted()
    assert m.get_capacity() == 0
    for _ in range(8):
        m.on_rollout_accepted()
    assert m.get_capacity() == 8               # 16 - 8 accepted, concurrency free again
    for _ in range(8):
        m.on_rollout_enqueued(); m.on_rollout_submitted(); m.on_rollout_accepted()
    assert m.get_capacity() == 0               # staleness budget exhausted


@pytest.mark.parametrize("version", [0, 1, 7, 1000, 10 ** 9])
def test_capacity_grows_linearly_with_version(version):
    m = StalenessManager(V(version), 10 ** 12, 32, 2)
    assert m.get_capacity() == (2 + version + 1) * 32


@pytest.mark.parametrize("running", [0, 3, 9])
def test_recovery_keeps_running_count(running):
    v = V(0)
    m = StalenessManager(v, 64, 4, 1)
    for _ in range(running):
        m.on_rollout_enqueued(); m.on_rollout_submitted()
    v.v = 6
    m.on_version_recovered(6)
    s = m.get_stats()
    assert (s.accepted, s.running) == (24, running)
    assert m.get_capacity() == min(64 - running, (1 + 6 + 1) * 4 - 24 - running)


def test_concurrent_capacity_reads_and_updates_are_consistent():
    m = StalenessManager(V(0), 10 ** 6, 1, 10 ** 6)
    seen = []

    def reader():
        for _ in range(2000):
            s = m.get_stats()
            seen.append(s.enqueued >= 0 and s.running >= 0)
            m.get_capacity()

    def writer():
        for _ in range(2000):
            m.on_rollout_enqueued(); m.on_rollout_submitted()
            if random.random() < 0.5:
                m.on_rollout_accepted()
            else:
                m.on_rollout_rejected()

    ts = [threading.Thread(target=f) for f in (reader, writer, reader, writer)]
    [t.start() for t in ts]; [t.join() for t in ts]
    s = m.get_stats()
    assert all(seen) and s.accepted + s.rejected == 4000 and s.running == 0

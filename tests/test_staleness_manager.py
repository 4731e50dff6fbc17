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

"""Bounded off-policyness: decides how many new rollouts may start.

With ``η = max_staleness``, current policy version ``v`` and consumer batch size
``B`` the number of samples that may have been started so far is
``(η + v + 1)·B``; on top of that at most ``max_concurrent_rollouts`` run at the
same time. Capacity is the tighter of the two limits
(areal/infra/staleness_manager.py:69-113 in the reference).
"""

from __future__ import annotations

import threading
from typing import Protocol

from ..api.io_struct import RolloutStat


class VersionProvider(Protocol):
    def get_version(self) -> int: ...


class StalenessManager:
    def __init__(self, version_provider: VersionProvider, max_concurrent_rollouts: int,
                 consumer_batch_size: int, max_staleness: int):
        self.version_provider = version_provider
        self.max_concurrent_rollouts = max_concurrent_rollouts
        self.consumer_batch_size = consumer_batch_size
        self.max_staleness = max_staleness
        self.lock = threading.Lock()
        self.rollout_stat = RolloutStat()

    def get_pending_limit(self) -> int:
        """How many samples a producer should keep queued ahead of the consumer."""
        return (self.max_staleness + 1) * self.consumer_batch_size

    def get_capacity(self) -> int:
        with self.lock:
            version = self.version_provider.get_version()
            by_concurrency = max(1, self.max_concurrent_rollouts) - self.rollout_stat.running
            started = self.rollout_stat.accepted + self.rollout_stat.running
            by_staleness = (self.max_staleness + version + 1) * max(1, self.consumer_batch_size) - started
            return min(by_concurrency, by_staleness)

    def on_version_recovered(self, version: int) -> None:
        """After a restart at ``version`` the accepted count is what ``version`` steps consumed."""
        with self.lock:
            self.rollout_stat.accepted = version * max(1, self.consumer_batch_size)

    def on_rollout_enqueued(self) -> None:
        with self.lock:
            self.rollout_stat.enqueued += 1

    def on_rollout_submitted(self) -> None:
        with self.lock:
            self.rollout_stat.enqueued -= 1
            self.rollout_stat.running += 1

    def on_rollout_accepted(self) -> None:
        with self.lock:
            self.rollout_stat.running -= 1
            self.rollout_stat.accepted += 1

    def on_rollout_rejected(self) -> None:
        with self.lock:
            self.rollout_stat.running -= 1
            self.rollout_stat.rejected += 1

    def get_stats(self) -> RolloutStat:
        with self.lock:
            s = self.rollout_stat
            return RolloutStat(accepted=s.accepted, enqueued=s.enqueued, rejected=s.rejected, running=s.running)

"""Distributed lock on a ``torch.distributed`` store (TCPStore / FileStore / HashStore): acquire
with an atomic counter + owner token, with time-out and a background lease so a crashed owner
cannot hold it forever. Reference: areal/utils/lock.py:10-102."""

from __future__ import annotations

import time
import uuid


class DistributedLock:
    def __init__(self, store, name: str, lease_seconds: float = 60.0, poll: float = 0.02):
        self.store, self.name, self.lease, self.poll = store, name, lease_seconds, poll
        self.token = uuid.uuid4().hex
        self._held = False

    def _key(self, suffix: str) -> str:
        return f"lock/{self.name}/{suffix}"

    def acquire(self, timeout: float | None = None) -> bool:
        deadline = None if timeout is None else time.monotonic() + timeout
        while True:
            # ticket counter: the caller that moves it from 0 to 1 owns the lock
            if self.store.add(self._key("count"), 1) == 1:
                self.store.set(self._key("owner"), f"{self.token}:{time.time() + self.lease}")
                self._held = True
                return True
            self.store.add(self._key("count"), -1)
            # steal an expired lease
            try:
                owner = self.store.get(self._key("owner")).decode()
                tok, _, exp = owner.partition(":")
                if tok and exp and 0 < float(exp) < time.time():  # a held lock whose lease ran out
                    if self.store.compare_set(self._key("owner"), owner, f"{self.token}:{time.time() + self.lease}").decode() \
                            .startswith(self.token):
                        self._held = True
                        return True
            except Exception:
                pass
            if deadline is not None and time.monotonic() > deadline:
                return False
            time.sleep(self.poll)

    def release(self):
        if not self._held:
            return
        self._held = False
        try:
            owner = self.store.get(self._key("owner")).decode()
        except Exception:
            owner = ""
        if owner.startswith(self.token):
            self.store.set(self._key("owner"), "")  # free: nothing to steal
            self.store.add(self._key("count"), -1)

    def __enter__(self):
        if not self.acquire():
            raise TimeoutError(f"could not acquire lock {self.name}")
        return self

    def __exit__(self, *exc):
        self.release()

"""Key-value service discovery with memory and shared-filesystem back ends.

Workers publish their addresses under experiment-scoped keys; launchers and
engines look them up, optionally waiting. Interface follows the reference
(areal/utils/name_resolve.py:184-1263): ``add / get / wait / delete /
get_subtree / find_subtree / clear_subtree / add_subentry``. The etcd3 and Ray
back ends of the reference need services that are not part of this package;
selecting them raises a clear error.
"""

from __future__ import annotations

import os
import shutil
import threading
import time
import uuid
from pathlib import Path
from typing import Any


class NameEntryExistsError(Exception):
    pass


class NameEntryNotFoundError(Exception):
    pass


class NameRecordRepository:
    def add(self, name, value, delete_on_exit=True, keepalive_ttl=None, replace=False):
        raise NotImplementedError

    def add_subentry(self, name, value, **kwargs):
        sub = f"{name.rstrip('/')}/{uuid.uuid4().hex[:8]}"
        self.add(sub, value, **kwargs)
        return sub

    def delete(self, name):
        raise NotImplementedError

    def clear_subtree(self, name_root):
        raise NotImplementedError

    def get(self, name):
        raise NotImplementedError

    def get_subtree(self, name_root) -> list[str]:
        raise NotImplementedError

    def find_subtree(self, name_root) -> list[str]:
        raise NotImplementedError

    def wait(self, name, timeout=None, poll_frequency=0.2):
        start = time.monotonic()
        while True:
            try:
                return self.get(name)
            except NameEntryNotFoundError:
                if timeout is not None and time.monotonic() - start > timeout:
                    raise TimeoutError(f"timed out waiting for key {name}")
                time.sleep(poll_frequency)

    def reset(self):
        pass


class MemoryNameRecordRepository(NameRecordRepository):
    """In-process store (single process / tests)."""

    def __init__(self):
        self._store: dict[str, str] = {}
        self._lock = threading.Lock()

    def add(self, name, value, delete_on_exit=True, keepalive_ttl=None, replace=False):
        name = name.rstrip("/")
        with self._lock:
            if name in self._store and not replace:
                raise NameEntryExistsError(name)
            self._store[name] = str(value)

    def delete(self, name):
        with self._lock:
            if name.rstrip("/") not in self._store:
                raise NameEntryNotFoundError(name)
            del self._store[name.rstrip("/")]

    def clear_subtree(self, name_root):
        root = name_root.rstrip("/")
        with self._lock:
            for k in [k for k in self._store if k == root or k.startswith(root + "/")]:
                del self._store[k]

    def get(self, name):
        with self._lock:
            try:
                return self._store[name.rstrip("/")]
            except KeyError:
                raise NameEntryNotFoundError(name) from None

    def find_subtree(self, name_root):
        root = name_root.rstrip("/")
        with self._lock:
            return sorted(k for k in self._store if k == root or k.startswith(root + "/"))

    def get_subtree(self, name_root):
        with self._lock:
            root = name_root.rstrip("/")
            return [self._store[k] for k in sorted(self._store) if k == root or k.startswith(root + "/")]

    def reset(self):
        with self._lock:
            self._store.clear()


class NfsNameRecordRepository(NameRecordRepository):
    """One file per key under a shared directory."""

    def __init__(self, record_root: str = "/tmp/areal/name_resolve"):
        self.root = Path(record_root)
        self._mine: set[str] = set()

    def _path(self, name) -> Path:
        return self.root / name.strip("/") / "ENTRY"

    def add(self, name, value, delete_on_exit=True, keepalive_ttl=None, replace=False):
        p = self._path(name)
        if p.exists() and not replace:
            raise NameEntryExistsError(name)
        p.parent.mkdir(parents=True, exist_ok=True)
        tmp = p.with_name(f"ENTRY.{uuid.uuid4().hex}.tmp")
        tmp.write_text(str(value))
        os.replace(tmp, p)
        if delete_on_exit:
            self._mine.add(name)

    def delete(self, name):
        p = self._path(name)
        if not p.exists():
            raise NameEntryNotFoundError(name)
        p.unlink()
        self._mine.discard(name)
        d = p.parent
        while d != self.root and d.exists() and not any(d.iterdir()):
            d.rmdir()
            d = d.parent

    def clear_subtree(self, name_root):
        d = self.root / name_root.strip("/")
        if d.exists():
            shutil.rmtree(d, ignore_errors=True)

    def get(self, name):
        p = self._path(name)
        for _ in range(3):
            try:
                return p.read_text()
            except FileNotFoundError:
                raise NameEntryNotFoundError(name) from None
            except OSError:
                time.sleep(0.05)
        raise NameEntryNotFoundError(name)

    def find_subtree(self, name_root):
        d = self.root / name_root.strip("/")
        if not d.exists():
            return []
        out = []
        for p in d.rglob("ENTRY"):
            out.append(str(p.parent.relative_to(self.root)))
        return sorted(out)

    def get_subtree(self, name_root):
        return [self.get(k) for k in self.find_subtree(name_root)]

    def reset(self):
        for n in list(self._mine):
            try:
                self.delete(n)
            except NameEntryNotFoundError:
                pass


class KVNameRecordRepository(NameRecordRepository):
    """Records in an external key-value service behind a four-call client: ``put(key, value, lease=None)``,
    ``get(key) -> (value | None, meta)``, ``get_prefix(prefix) -> iterable of (value, meta-with-.key)``,
    ``delete(key)``, plus ``lease(ttl)`` returning an object with ``refresh()`` / ``revoke()`` for keep-alive
    entries. That is the interface of the ``etcd3`` client (``Etcd3NameRecordRepository`` opens one); a
    Ray-backed store only needs the same five calls (``RayNameRecordRepository`` wraps a named actor).
    Reference: areal/utils/name_resolve.py:412 (etcd3) and :883 (Ray)."""

    def __init__(self, client, keepalive_interval: float = 0.3):
        self.client = client
        self._mine: set[str] = set()
        self._leases: dict[str, Any] = {}
        self._stop = threading.Event()
        self._keepalive = None
        self._interval = keepalive_interval

    @staticmethod
    def _s(v):
        return v.decode() if isinstance(v, (bytes, bytearray)) else v

    def add(self, name, value, delete_on_exit=True, keepalive_ttl=None, replace=False):
        name = name.rstrip("/")
        if not replace and self.client.get(name)[0] is not None:
            raise NameEntryExistsError(name)
        lease = None
        if keepalive_ttl is not None:
            lease = self.client.lease(int(max(keepalive_ttl, 1)))
            self._leases[name] = lease
            if self._keepalive is None:
                self._keepalive = threading.Thread(target=self._refresh_loop, daemon=True, name="name-resolve-keepalive")
                self._keepalive.start()
        self.client.put(name, str(value), lease=lease)
        if delete_on_exit:
            self._mine.add(name)

    def _refresh_loop(self):
        while not self._stop.wait(self._interval):
            for lease in list(self._leases.values()):
                try:
                    lease.refresh()
                except Exception:
                    pass

    def delete(self, name):
        name = name.rstrip("/")
        if self.client.get(name)[0] is None:
            raise NameEntryNotFoundError(name)
        self.client.delete(name)
        self._mine.discard(name)
        lease = self._leases.pop(name, None)
        if lease is not None:
            lease.revoke()

    def clear_subtree(self, name_root):
        for key in self.find_subtree(name_root):
            self.client.delete(key)
            self._mine.discard(key)

    def get(self, name):
        v, _ = self.client.get(name.rstrip("/"))
        if v is None:
            raise NameEntryNotFoundError(name)
        return self._s(v)

    def _prefix(self, name_root):
        root = name_root.rstrip("/")
        out = []
        for v, meta in self.client.get_prefix(root):
            key = self._s(meta.key)
            if key == root or key.startswith(root + "/"):
                out.append((key, self._s(v)))
        return sorted(out)

    def get_subtree(self, name_root) -> list[str]:
        return [v for _, v in self._prefix(name_root)]

    def find_subtree(self, name_root) -> list[str]:
        return [k for k, _ in self._prefix(name_root)]

    def reset(self):
        self._stop.set()
        for name in list(self._mine):
            try:
                self.client.delete(name)
            except Exception:
                pass
        self._mine.clear()
        for lease in self._leases.values():
            try:
                lease.revoke()
            except Exception:
                pass
        self._leases.clear()


class Etcd3NameRecordRepository(KVNameRecordRepository):
    def __init__(self, addr: str = "localhost:2379", user: str | None = None, password: str | None = None):
        try:
            import etcd3
        except ImportError as e:
            raise ImportError("name_resolve.type = 'etcd3' needs the `etcd3` package and a reachable etcd "
                              "server; use 'nfs' (shared directory) where neither is available") from e
        host, _, port = addr.partition(":")
        super().__init__(etcd3.client(host=host or "localhost", port=int(port or 2379), user=user, password=password))


class RayNameRecordRepository(KVNameRecordRepository):
    """A detached Ray actor holding the records; every process of the job talks to the same actor."""

    def __init__(self, actor_name: str = "areal_b200_name_resolve", namespace: str = "areal_b200"):
        try:
            import ray
        except ImportError as e:
            raise ImportError("name_resolve.type = 'ray' needs Ray; use 'nfs' where it is not installed") from e

        @ray.remote
        class _Store:
            def __init__(self):
                self.d = {}

            def put(self, k, v):
                self.d[k] = v

            def get(self, k):
                return self.d.get(k)

            def prefix(self, p):
                return [(k, v) for k, v in self.d.items() if k.startswith(p)]

            def delete(self, k):
                self.d.pop(k, None)

        actor = _Store.options(name=actor_name, namespace=namespace, lifetime="detached", get_if_exists=True).remote()

        class _Meta:
            def __init__(self, key):
                self.key = key

        class _Lease:
            def refresh(self):
                pass

            def revoke(self):
                pass

        class _Client:
            def put(self, k, v, lease=None):
                ray.get(actor.put.remote(k, v))

            def get(self, k):
                return ray.get(actor.get.remote(k)), None

            def get_prefix(self, p):
                return [(v, _Meta(k)) for k, v in ray.get(actor.prefix.remote(p))]

            def delete(self, k):
                ray.get(actor.delete.remote(k))

            def lease(self, ttl):
                return _Lease()

        super().__init__(_Client())


def make_repository(cfg) -> NameRecordRepository:
    t = getattr(cfg, "type", "nfs")
    if t == "memory":
        return MemoryNameRecordRepository()
    if t == "nfs":
        return NfsNameRecordRepository(cfg.nfs_record_root)
    if t == "etcd3":
        return Etcd3NameRecordRepository(getattr(cfg, "etcd3_addr", "localhost:2379"))
    if t == "ray":
        return RayNameRecordRepository(getattr(cfg, "ray_actor_name", "areal_b200_name_resolve"))
    raise ValueError(f"unknown name_resolve type {t!r} (memory | nfs | etcd3 | ray)")


DEFAULT_REPOSITORY: NameRecordRepository = MemoryNameRecordRepository()


def reconfigure(cfg) -> None:
    global DEFAULT_REPOSITORY
    DEFAULT_REPOSITORY.reset()
    DEFAULT_REPOSITORY = make_repository(cfg)


def add(name, value, **kw):
    return DEFAULT_REPOSITORY.add(name, value, **kw)


def add_subentry(name, value, **kw):
    return DEFAULT_REPOSITORY.add_subentry(name, value, **kw)


def delete(name):
    return DEFAULT_REPOSITORY.delete(name)


def clear_subtree(name_root):
    return DEFAULT_REPOSITORY.clear_subtree(name_root)


def get(name):
    return DEFAULT_REPOSITORY.get(name)


def get_subtree(name_root):
    return DEFAULT_REPOSITORY.get_subtree(name_root)


def find_subtree(name_root):
    return DEFAULT_REPOSITORY.find_subtree(name_root)


def wait(name, timeout=None, poll_frequency=0.2):
    return DEFAULT_REPOSITORY.wait(name, timeout, poll_frequency)


def reset():
    return DEFAULT_REPOSITORY.reset()

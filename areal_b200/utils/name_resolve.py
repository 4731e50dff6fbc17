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


def make_repository(cfg) -> NameRecordRepository:
    t = getattr(cfg, "type", "nfs")
    if t == "memory":
        return MemoryNameRecordRepository()
    if t == "nfs":
        return NfsNameRecordRepository(cfg.nfs_record_root)
    raise NotImplementedError(
        f"name_resolve type {t!r} needs an external service (etcd3 / Ray) that this package does "
        "not bundle; use 'nfs' (shared directory) or 'memory'")


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

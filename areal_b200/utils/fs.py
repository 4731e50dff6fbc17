"""File-system checks for paths that several nodes must see (checkpoints, name-resolve records, logs)."""

from __future__ import annotations

import getpass
import os
import tempfile

from . import logging

logger = logging.getLogger("fs")

NETWORK_FS_KEYWORDS = ("nfs", "lustre", "gpfs", "ceph", "beegfs", "cifs", "smb", "fuse", "glusterfs", "weka", "efs")


def get_user_tmp() -> str:
    """A per-user scratch directory under the system's temporary directory (created on demand)."""
    path = os.path.join(tempfile.gettempdir(), getpass.getuser())
    os.makedirs(path, exist_ok=True)
    return path


def filesystem_type(path: str) -> str | None:
    """Type of the mount that holds ``path`` according to ``/proc/mounts`` (``None`` when it cannot be told)."""
    try:
        real = os.path.realpath(path)
        best, kind = "", None
        with open("/proc/mounts") as f:
            for line in f:
                parts = line.split()
                if len(parts) >= 3 and (real == parts[1] or real.startswith(parts[1].rstrip("/") + "/")) \
                        and len(parts[1]) > len(best):
                    best, kind = parts[1], parts[2]
        return kind
    except OSError:
        return None


def is_network_fs(path: str) -> bool | None:
    kind = filesystem_type(path)
    return None if kind is None else any(k in kind.lower() for k in NETWORK_FS_KEYWORDS)


def validate_shared_path(path: str, name: str = "path", warn_nfs: bool = True, n_nodes: int = 1) -> None:
    """``path`` must exist (its closest existing ancestor is checked when it will be created later). On a
    multi-node run a path on a local file system is reported: the other nodes will not see it."""
    if not path:
        raise ValueError(f"{name} is empty")
    probe = os.path.abspath(path)
    while not os.path.exists(probe):
        parent = os.path.dirname(probe)
        if parent == probe:
            raise FileNotFoundError(f"{name} '{path}' does not exist.")
        probe = parent
    if not os.access(probe, os.W_OK):
        raise PermissionError(f"{name} '{path}': no write permission on '{probe}'")
    if warn_nfs and n_nodes > 1 and is_network_fs(probe) is False:
        logger.warning(f"{name} '{path}' is on a local file system ({filesystem_type(probe)}), but the run spans "
                       f"{n_nodes} nodes: the other nodes will not see it")

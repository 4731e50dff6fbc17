"""Network helpers: free ports, this host's address, waiting for a TCP endpoint.
Reference: areal/utils/network.py."""

from __future__ import annotations

import socket
import time


def find_free_ports(n: int = 1, low: int = 1024, high: int = 65535) -> list[int]:
    socks, ports = [], []
    try:
        for _ in range(n):
            s = socket.socket()
            s.bind(("", 0))
            socks.append(s)
            ports.append(s.getsockname()[1])
    finally:
        for s in socks:
            s.close()
    return ports


def gethostip() -> str:
    """Address other machines can reach this host at; 127.0.0.1 when the name does not resolve."""
    try:
        s = socket.socket(socket.AF_INET, socket.SOCK_DGRAM)
        try:
            s.connect(("10.255.255.255", 1))
            return s.getsockname()[0]
        finally:
            s.close()
    except OSError:
        try:
            return socket.gethostbyname(socket.gethostname())
        except OSError:
            return "127.0.0.1"


def wait_for_port(host: str, port: int, timeout: float = 30.0) -> bool:
    deadline = time.monotonic() + timeout
    while time.monotonic() < deadline:
        try:
            with socket.create_connection((host, port), timeout=1.0):
                return True
        except OSError:
            time.sleep(0.1)
    return False


def is_ipv6(host: str) -> bool:
    try:
        socket.inet_pton(socket.AF_INET6, host.strip("[]").split("%", 1)[0])
        return True
    except OSError:
        return False


def format_addr(host: str, port: int) -> str:
    """``host:port`` with IPv6 literals in brackets (``[::1]:80``)."""
    host = host.strip("[]")
    return f"[{host}]:{port}" if ":" in host else f"{host}:{port}"


def split_addr(addr: str) -> tuple[str, int]:
    """Inverse of :func:`format_addr`: ``"[fe80::1]:80"`` → ``("fe80::1", 80)``, ``"h:80"`` → ``("h", 80)``."""
    addr = addr.split("://", 1)[-1].split("/", 1)[0]
    if addr.startswith("["):
        host, _, rest = addr[1:].partition("]")
        if not rest.startswith(":"):
            raise ValueError(f"no port in {addr!r}")
        return host, int(rest[1:])
    host, sep, port = addr.rpartition(":")
    if not sep or ":" in host:
        raise ValueError(f"cannot split {addr!r} into host and port (IPv6 literals need brackets)")
    return host, int(port)


def format_url(host: str, port: int, scheme: str = "http", path: str = "") -> str:
    return f"{scheme}://{format_addr(host, port)}{path}"

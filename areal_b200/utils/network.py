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


# names the reference's utilities go by (areal/utils/network.py)
format_hostport = format_addr
split_hostport = split_addr


def format_host_for_url(host: str) -> str:
    """``host`` as it appears inside a URL: IPv6 literals in brackets."""
    host = host.strip("[]")
    return f"[{host}]" if ":" in host else host


def is_port_free(port: int, host: str = "") -> bool:
    with socket.socket(socket.AF_INET6 if is_ipv6(host) else socket.AF_INET) as s:
        s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        try:
            s.bind((host.strip("[]"), port))
            return True
        except OSError:
            return False


def get_loopback_ip(prefer_ipv6: bool = False) -> str:
    """``127.0.0.1``, or ``::1`` when asked for and the host has an IPv6 loopback."""
    if prefer_ipv6 and socket.has_ipv6:
        try:
            with socket.socket(socket.AF_INET6) as s:
                s.bind(("::1", 0))
                return "::1"
        except OSError:
            pass
    return "127.0.0.1"


def gethostname() -> str:
    return socket.gethostname()

"""Addresses for servers: what to bind, what to announce, a free port.
Parity: reference dlengine/utils/network.py (`get_local_ip`, `get_bind_host`, `get_advertise_host`, `get_free_port`)."""
from __future__ import annotations

import socket
from typing import Optional

_WILDCARDS = (None, "", "0.0.0.0", "::")


def get_local_ip() -> str:
    """This machine's address on the route other machines would use (no packet is sent: a UDP socket is only connected), falling
    back to the host name's address, then loopback."""
    try:
        with socket.socket(socket.AF_INET, socket.SOCK_DGRAM) as s:
            s.connect(("10.255.255.255", 1))
            return s.getsockname()[0]
    except OSError:
        pass
    try:
        return socket.gethostbyname(socket.gethostname())
    except OSError:
        return "127.0.0.1"


def get_bind_host(host: Optional[str]) -> str:
    return host if host else "0.0.0.0"


def get_advertise_host(host: Optional[str]) -> str:
    """The address to publish for a server bound to `host`: never a wildcard."""
    return get_local_ip() if host in _WILDCARDS else host


def get_free_port(host: str = "127.0.0.1") -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind((host, 0))
        return s.getsockname()[1]

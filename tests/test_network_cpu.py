"""Bind / announce addresses (reference tests/test_network_endpoints.py scenarios)."""
import socket

from nanoengine_b200.utils import network


def test_bind_host_defaults_to_the_wildcard():
    assert network.get_bind_host(None) == "0.0.0.0" and network.get_bind_host("") == "0.0.0.0"
    assert network.get_bind_host("127.0.0.1") == "127.0.0.1"


def test_the_announced_host_is_never_a_wildcard(monkeypatch):
    monkeypatch.setattr(network, "get_local_ip", lambda: "10.0.0.8")
    for h in (None, "", "0.0.0.0", "::"):
        assert network.get_advertise_host(h) == "10.0.0.8"
    assert network.get_advertise_host("node.example") == "node.example"
    from nanoengine_b200.server.ctrl import advertise_host
    assert advertise_host("0.0.0.0") == "10.0.0.8" and advertise_host("10.1.2.3") == "10.1.2.3"


def test_local_ip_and_free_port():
    ip = network.get_local_ip()
    socket.inet_aton(ip)                                   # a dotted quad
    p = network.get_free_port()
    with socket.socket() as s:
        s.bind(("127.0.0.1", p))                            # free to take right after

"""The package's multiaddr subset: text <-> binary vectors of the format, protocol table, editing operations.

The reference vendors a full multiaddr library with its own test-suite (tests/test_multiaddr*.py); these tests pin
the parts that the framework relies on.
"""
import pytest

from hivemind_b200.utils.multiaddr import Multiaddr
from hivemind_b200.utils.multiaddr.multiaddr import protocol_with_code, protocol_with_name

PEER = "QmYyQSo1c1Ym7orWxLYvCrM2EmxFTANf8wXmmE7DWjhx5N"

# (text, hex of the binary form): varint protocol code, then a fixed-size or length-prefixed value
VECTORS = [
    ("/ip4/127.0.0.1", "047f000001"),
    ("/ip4/10.20.30.40/tcp/1234", "040a141e280604d2"),
    ("/ip4/127.0.0.1/udp/1234", "047f000001910204d2"),
    ("/ip6/::1", "2900000000000000000000000000000001"),
    ("/ip6/2001:db8::ff00:42:8329/tcp/443", "2920010db8000000000000ff000042832906" + "01bb"),
    ("/dns4/example.com/tcp/80", "36" + "0b" + "example.com".encode().hex() + "060050"),
    ("/dns/localhost", "35" + "09" + "localhost".encode().hex()),
]


@pytest.mark.parametrize("text,binary", VECTORS)
def test_known_vectors(text, binary):
    addr = Multiaddr(text)
    assert addr.to_bytes().hex() == binary
    assert str(Multiaddr(bytes.fromhex(binary))) == text
    assert Multiaddr(addr) == addr and hash(Multiaddr(text)) == hash(addr)


@pytest.mark.parametrize("text", [
    f"/ip4/1.2.3.4/tcp/4001/p2p/{PEER}", f"/ip6/fe80::1/udp/9/quic/p2p/{PEER}", f"/dns4/host.example/tcp/443/wss/p2p/{PEER}",
    "/unix/var/run/daemon.sock", f"/p2p/{PEER}", "/ip4/0.0.0.0/tcp/0", "/ip4/255.255.255.255/udp/65535",
])
def test_text_binary_round_trip(text):
    addr = Multiaddr(text)
    again = Multiaddr(addr.to_bytes())
    assert again == addr and str(again) == str(addr)
    assert [p.name for p in again.protocols()] == [p.name for p in addr.protocols()]
    assert again.values() == addr.values()


@pytest.mark.parametrize("bad", [
    "", "/", "ip4/1.2.3.4", "/ip4", "/ip4/1.2.3", "/ip4/256.0.0.1", "/ip4/1.2.3.4/tcp", "/tcp/65536", "/tcp/-1",
    "/tcp/http", "/ip6/::g", "/unknownproto/1", "/p2p/not-base58-0OIl",
])
def test_invalid_text_is_rejected(bad):
    if bad in ("", "/"):  # the empty address is valid and has no protocols
        assert Multiaddr(bad).protocols() == []
        return
    with pytest.raises(Exception):
        Multiaddr(bad)


@pytest.mark.parametrize("bad", ["04", "047f0000", "06", "0604", "ff7f", "3605abc1"])
def test_truncated_or_unknown_binary_is_rejected(bad):
    with pytest.raises(Exception):
        Multiaddr(bytes.fromhex(bad))


def test_protocol_table_lookup():
    for name, code in [("ip4", 4), ("tcp", 6), ("udp", 0x0111), ("ip6", 41), ("dns4", 54), ("p2p", 421), ("unix", 400)]:
        assert protocol_with_name(name).code == code and protocol_with_code(code).name == name
    with pytest.raises(Exception):
        protocol_with_name("carrier-pigeon")
    with pytest.raises(Exception):
        protocol_with_code(0x7FFFFF)


def test_editing_operations():
    full = Multiaddr(f"/ip4/1.2.3.4/tcp/4001/p2p/{PEER}")
    assert str(full.decapsulate(f"/p2p/{PEER}")) == "/ip4/1.2.3.4/tcp/4001"
    assert str(full.decapsulate("/tcp/4001")) == "/ip4/1.2.3.4"  # removes the component and all that follows it
    assert full.decapsulate("/udp/1") == full  # absent component: unchanged
    assert str(full.decapsulate_code(protocol_with_name("p2p").code)) == "/ip4/1.2.3.4/tcp/4001"
    assert Multiaddr("/ip4/1.2.3.4").encapsulate("/tcp/4001").encapsulate(f"/p2p/{PEER}") == full
    parts = full.split()
    assert [str(p) for p in parts] == ["/ip4/1.2.3.4", "/tcp/4001", f"/p2p/{PEER}"]
    assert Multiaddr.join(*parts) == full
    assert full.value_for_protocol("tcp") == "4001" and full.value_for_protocol(4) == "1.2.3.4"
    assert full["p2p"] == PEER and "quic" not in full
    with pytest.raises(Exception):
        full["quic"]
    items = [(proto.name, value) for proto, value in full]
    assert items == [("ip4", "1.2.3.4"), ("tcp", "4001"), ("p2p", PEER)]
    assert Multiaddr("/ip4/1.2.3.4/tcp/1") != Multiaddr("/ip4/1.2.3.4/tcp/2")
    assert repr(full).count(PEER) == 1

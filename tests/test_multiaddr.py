"""The multiaddr package: text <-> binary vectors of the format, value codecs, the protocol registry, the mapping
interface and the nesting operations (the ground covered by the reference's tests/test_multiaddr.py,
tests/test_multiaddr_protocols.py and tests/test_multiaddr_transforms.py; byte vectors are those of go-multiaddr)."""
import io
import pickle

import pytest

from hivemind_b200.utils.multiaddr import Multiaddr, exceptions, protocols, transforms
from hivemind_b200.utils.multiaddr.codecs import codec_by_name
from hivemind_b200.utils.multiaddr.multiaddr import MultiAddrItems, MultiAddrKeys, MultiAddrValues

PEER = "QmcgpsyWgH8Y8ajJz1Cu72KnS5uo2Aa2LpzU7kinSupNKC"
PEER_MULTIHASH = bytes.fromhex("1220d52ebb89d85b02a284948203a62ff28389c57c9f42beec4ec20db76a68911c0b")
ED25519_PEER = "12D3KooWPA6ax6t3jqTyGq73Zm1RmwppYqxaXzrtarfcTWGp5Wzx"
ED25519_MULTIHASH = bytes.fromhex("002408011220c635ed472d58edd8b9ee4641ec7557dc806b4886e568491ab00bff1269a7be65")
ONION3 = "vww6ybal4bd7szmgncyruucpgfkqahzddi37ktceo3ah7ngmcopnpyyd"

# ------------------------------------------------------------------------------------------------ whole addresses
ADDRESS_VECTORS = [
    ("/ip4/127.0.0.1", "047f000001"),
    ("/ip4/10.20.30.40/tcp/1234", "040a141e280604d2"),
    ("/ip4/127.0.0.1/udp/1234", "047f000001910204d2"),
    ("/ip4/127.0.0.1/tcp/4321", "047f0000010610e1"),
    ("/ip4/127.0.0.1/udp/1234/ip4/127.0.0.1/tcp/4321", "047f000001910204d2047f0000010610e1"),
    ("/ip6/::1", "2900000000000000000000000000000001"),
    ("/ip6/2001:db8::ff00:42:8329/tcp/443", "2920010db8000000000000ff00004283290601bb"),
    ("/dns4/example.com/tcp/80", "360b" + b"example.com".hex() + "060050"),
    ("/dns/localhost", "3509" + b"localhost".hex()),
    ("/ip4/1.2.3.4/udp/9/quic", "0401020304" + "91020009" + "cc03"),
    ("/unix/var/run/daemon.sock", "9003" + "14" + b"/var/run/daemon.sock".hex()),
    (f"/p2p/{PEER}", "a503" + "24" + "0172" + PEER_MULTIHASH.hex()),
]


@pytest.mark.parametrize("text,binary", ADDRESS_VECTORS)
def test_address_vectors_both_ways(text, binary):
    addr = Multiaddr(text)
    assert addr.to_bytes().hex() == binary and bytes(addr) == addr.to_bytes()
    assert transforms.string_to_bytes(text).hex() == binary
    assert transforms.bytes_to_string(bytes.fromhex(binary)) == text
    again = Multiaddr(bytes.fromhex(binary))
    assert str(again) == text and again == addr and hash(again) == hash(addr)
    assert Multiaddr(addr) == addr and pickle.loads(pickle.dumps(addr)) == addr
    assert repr(addr) == f"<Multiaddr {text}>"


VALID_TEXT = [
    "/ip4/1.2.3.4", "/ip4/0.0.0.0", "/ip6/::1", "/ip6/2601:9:4f81:9700:803e:ca65:66e8:c21",
    "/ip6zone/x/ip6/fe80::1", "/ip6zone/x%y/ip6/fe80::1", "/ip6zone/x%y/ip6/::",
    "/onion/timaq4ygg2iegci7:1234", "/onion/timaq4ygg2iegci7:80/http", f"/onion3/{ONION3}:1234", f"/onion3/{ONION3}:80/http",
    "/udp/0", "/tcp/0", "/sctp/0", "/udp/1234", "/tcp/1234", "/sctp/1234", "/utp", "/udp/65535", "/tcp/65535",
    f"/p2p/{PEER}", "/udp/1234/sctp/1234", "/udp/1234/udt", "/udp/1234/utp", "/tcp/1234/http", "/tcp/1234/https",
    f"/p2p/{PEER}/tcp/1234", "/ip4/127.0.0.1/udp/1234", f"/ip4/127.0.0.1/p2p/{PEER}/tcp/1234",
    "/unix/a/b/c/d/e", "/unix/Überrschung!/大柱", "/unix/stdio", "/ip4/1.2.3.4/tcp/80/unix/a/b/c/d/e/f",
    f"/ip4/127.0.0.1/p2p/{PEER}/tcp/1234/unix/stdio", "/ip4/127.0.0.1/tcp/9090/http/p2p-webrtc-direct",
    "/dns/example.com", "/dns4/موقع.وزارة-الاتصالات.مصر", "/dnsaddr/bootstrap.example.org/tcp/4001/tls/ws",
    f"/ip4/10.0.0.1/udp/4001/quic-v1/p2p/{PEER}/p2p-circuit/p2p/{ED25519_PEER}",
]


@pytest.mark.parametrize("text", VALID_TEXT)
def test_valid_text_survives_the_round_trip(text):
    addr = Multiaddr(text)
    assert str(addr) == text
    assert Multiaddr(addr.to_bytes()) == addr and str(Multiaddr(addr.to_bytes())) == text
    assert str(Multiaddr(text + "/")) == text, "a trailing slash is not part of the address"


INVALID_TEXT = [
    "/ip4", "/ip4/::1", "/ip4/fdpsofodsajfdoisa", "/ip4/1.2.3", "/ip4/256.0.0.1", "/ip6", "/ip6/::g", "/ip6zone",
    "/ip6zone/", "/ip6zone//ip6/fe80::1", "/udp", "/tcp", "/sctp", "/udp/65536", "/tcp/65536", "/tcp/-1", "/tcp/http",
    "/onion/9imaq4ygg2iegci7:80", "/onion/aaimaq4ygg2iegci7:80", "/onion/timaq4ygg2iegci7:0",
    "/onion/timaq4ygg2iegci7:-1", "/onion/timaq4ygg2iegci7", "/onion/timaq4ygg2iegci@:666",
    f"/onion3/9{ONION3[1:]}:80", f"/onion3/{ONION3}7:80", f"/onion3/{ONION3}:0", f"/onion3/{ONION3}:a",
    f"/onion3/{ONION3}:-1", f"/onion3/{ONION3}", f"/onion3/{ONION3[:-1]}@:666",
    "/udp/1234/sctp", "/udp/1234/udt/1234", "/udp/1234/utp/1234", "/ip4/127.0.0.1/udp/jfodsajfidosajfoidsa",
    "/ip4/127.0.0.1/udp", "/ip4/127.0.0.1/tcp/jfodsajfidosajfoidsa", "/ip4/127.0.0.1/tcp", "/ip4/127.0.0.1/p2p",
    "/ip4/127.0.0.1/p2p/tcp", "/p2p/not-base58-0OIl", "/unix", "/ip4/1.2.3.4/tcp/80/unix",
    "/ip4/127.0.0.1/tcp/9090/http/p2p-webcrt-direct", "/dns", "/dns4", "/dns6", "/dns4/a:b", "/cancer", "ip4/1.2.3.4",
    "test",
]


@pytest.mark.parametrize("text", INVALID_TEXT)
def test_invalid_text_raises_a_string_parse_error(text):
    with pytest.raises(exceptions.StringParseError) as failure:
        Multiaddr(text)
    assert isinstance(failure.value, ValueError) and isinstance(failure.value, exceptions.Error)
    assert failure.value.string == text


@pytest.mark.parametrize("binary", ["04", "047f0000", "06", "0604", "ff7f", "3605abc1", "cd020c0d", "3503613a62",
                                    "a50303" + "017000", "80"])
def test_invalid_binary_raises_a_binary_parse_error(binary):
    with pytest.raises(exceptions.BinaryParseError):
        Multiaddr(bytes.fromhex(binary))
    with pytest.raises(exceptions.BinaryParseError):
        transforms.bytes_to_string(bytes.fromhex(binary))


def test_construction_rejects_other_types_and_empty_addresses_are_fine():
    for bad in (None, 42, 3.5, ["/ip4/1.2.3.4"]):
        with pytest.raises(TypeError):
            Multiaddr(bad)
    with pytest.raises(TypeError):
        Multiaddr("/ip4/1.2.3.4", "/tcp/80")
    for empty in (Multiaddr("/"), Multiaddr(""), Multiaddr(b""), Multiaddr()):
        assert str(empty) == "/" and empty.to_bytes() == b"" and len(empty) == 0 and list(empty.protocols()) == []


# ------------------------------------------------------------------------------------------------ value codecs
CODEC_VECTORS = [
    ("ip4", "0a0b0c0d", "10.11.12.13"),
    ("ip6", "1aa12bb23cc34dd45ee56ff67ab78ac8", "1aa1:2bb2:3cc3:4dd4:5ee5:6ff6:7ab7:8ac8"),
    ("tcp", "abcd", "43981"),
    ("onion", "9a18087306369043091f04d2", "timaq4ygg2iegci7:1234"),
    ("p2p", "0172" + PEER_MULTIHASH.hex(), PEER),
    ("dns4", "موقع.وزارة-الاتصالات.مصر".encode().hex(), "موقع.وزارة-الاتصالات.مصر"),
    ("dns4", "fußball.example".encode().hex(), "fußball.example"),  # IDNA 2008: the sharp s is kept
    ("ip6zone", b"eth0".hex(), "eth0"),
    ("unix", b"/tmp/s.sock".hex(), "/tmp/s.sock"),
]


@pytest.mark.parametrize("name,binary,text", CODEC_VECTORS)
def test_codec_vectors_both_ways(name, binary, text):
    proto = protocols.protocol_with_name(name)
    codec = codec_by_name(proto.codec)
    assert codec.to_bytes(proto, text).hex() == binary
    assert codec.to_string(proto, bytes.fromhex(binary)) == text


def test_peer_ids_convert_between_their_two_spellings():
    p2p, other = protocols.protocol_with_name("p2p"), protocols.protocol_with_name("ip6")
    cid = codec_by_name("cid")
    # text: a multibase CIDv1 is accepted and kept; a base58 multihash becomes a libp2p-key CIDv1 under /p2p only
    assert cid.to_bytes(p2p, "bafzbeigvf25ytwc3akrijfecaotc74udrhcxzh2cx3we5qqnw5vgrei4bm").hex() == "0172" + PEER_MULTIHASH.hex()
    assert cid.to_bytes(p2p, ED25519_PEER) == b"\x01\x72" + ED25519_MULTIHASH
    assert cid.to_bytes(other, ED25519_PEER) == ED25519_MULTIHASH
    # bytes: both a bare multihash and a CIDv1 read as base58 under /p2p; elsewhere a CIDv1 keeps its multibase text
    assert cid.to_string(p2p, PEER_MULTIHASH) == PEER
    assert cid.to_string(p2p, b"\x01\x72" + ED25519_MULTIHASH) == ED25519_PEER
    assert cid.to_string(other, b"\x01\x72" + ED25519_MULTIHASH) == "bafzaajaiaejcbrrv5vds2whn3c464rsb5r2vpxeanneinzlijenlac77cju2pptf"
    assert cid.to_string(other, ED25519_MULTIHASH) == ED25519_PEER
    assert str(Multiaddr(b"\xa5\x03\x22" + PEER_MULTIHASH)) == f"/p2p/{PEER}"  # the older binary spelling still parses
    # a CID of another content type is not a peer id
    with pytest.raises(Exception):
        cid.to_bytes(p2p, "bafyaajaiaejcbrrv5vds2whn3c464rsb5r2vpxeanneinzlijenlac77cju2pptf")
    with pytest.raises(Exception):
        cid.to_string(p2p, b"\x01\x70" + ED25519_MULTIHASH)


@pytest.mark.parametrize("name,text", [
    ("ip4", "1124.2.3"), ("ip6", "123.123.123.123"), ("tcp", "a"), ("tcp", "100000"), ("onion", "100000"),
    ("onion", "1234567890123456:0"), ("onion", "timaq4ygg2iegci7:a"), ("onion", "timaq4ygg2iegci7:0"),
    ("onion", "timaq4ygg2iegci7:71234"), ("p2p", "15230d52ebb89d85b02a284948203a"), ("ip6zone", ""), ("dns", ""),
])
def test_codecs_refuse_bad_text(name, text):
    proto = protocols.protocol_with_name(name)
    with pytest.raises(Exception):
        codec_by_name(proto.codec).to_bytes(proto, text)


@pytest.mark.parametrize("name,binary", [("tcp", "ffffffff"), ("ip6zone", ""), ("ip4", "0102"), ("onion", "00"),
                                          ("p2p", "1220ab")])
def test_codecs_refuse_bad_bytes(name, binary):
    proto = protocols.protocol_with_name(name)
    with pytest.raises(Exception):
        codec_by_name(proto.codec).to_string(proto, bytes.fromhex(binary))


def test_sizes_and_component_iteration():
    assert transforms.size_for_addr(codec_by_name(None), io.BytesIO(b"\x01\x02\x03")) == (0, 0)
    assert transforms.size_for_addr(codec_by_name("ip4"), io.BytesIO(b"\x01\x02\x03")) == (4, 0)
    assert transforms.size_for_addr(codec_by_name("cid"), io.BytesIO(b"\x40\x50\x60\x51")) == (64, 1)
    raw = Multiaddr(f"/ip4/1.2.3.4/tcp/80/ws/p2p/{PEER}").to_bytes()
    seen = [(header, proto.name, value.hex()) for header, proto, _, value in transforms.bytes_iter(raw)]
    assert seen == [(1, "ip4", "01020304"), (1, "tcp", "0050"), (2, "ws", ""), (3, "p2p", "0172" + PEER_MULTIHASH.hex())]
    assert [(p.name, v) for p, _, v in transforms.string_iter("/ip4/1.2.3.4/tcp/80/unix/a/b")] == [
        ("ip4", "1.2.3.4"), ("tcp", "80"), ("unix", "/a/b")]


# ------------------------------------------------------------------------------------------------ protocols
def test_protocol_objects_validate_and_compare():
    proto = protocols.Protocol(code=protocols.P_IP4, name="ipb4", codec="ipb")  # the codec is resolved on use only
    assert (proto.code, proto.name, proto.codec) == (4, "ipb4", "ipb")
    for bad in (dict(code="abc"), dict(name=123), dict(name=None), dict(codec=b"ip4"), dict(codec=123)):
        with pytest.raises(TypeError):
            protocols.Protocol(**{**dict(code=4, name="ip4", codec="ip4"), **bad})
    ip4 = protocols.protocol_with_name("ip4")
    assert ip4 == protocols.protocol_with_code(protocols.P_IP4) == protocols.protocol_with_any(ip4)
    assert protocols.protocol_with_any("ip4") == protocols.protocol_with_any(4) == ip4
    assert (ip4.size, ip4.path, ip4.vcode, hash(ip4)) == (32, False, b"\x04", protocols.P_IP4)
    assert protocols.protocol_with_name("p2p").vcode == b"\xa5\x03" and protocols.protocol_with_name("p2p").size == -1
    assert protocols.protocol_with_name("unix").path and protocols.protocol_with_name("quic").size == 0
    assert ip4 != protocols.protocol_with_name("onion") != protocols.protocol_with_name("onion3")
    assert ip4 is not None and ip4 != str(ip4) and ip4 != 4
    assert repr(ip4) == "Protocol(code=4, name='ip4', codec='ip4')"
    assert protocols.protocol_with_name("ipfs") is protocols.protocol_with_name("p2p")  # the protocol's old name
    for lookup, key in ((protocols.protocol_with_name, "foo"), (protocols.protocol_with_code, 1234)):
        with pytest.raises(exceptions.ProtocolNotFoundError):
            lookup(key)


@pytest.mark.parametrize("names", [["ip4"], ["ip4", "tcp"], ["ip4", "tcp", "udp"], ["dns4", "tcp", "tls", "ws", "p2p"]])
def test_protocols_named_in_a_string(names):
    expected = [protocols.protocol_with_name(name) for name in names]
    joined = "/".join(names)
    for spelling in (joined, "/" + joined, "/" + joined + "/"):
        assert protocols.protocols_with_string(spelling) == expected
    for nothing in ("", "/", "//"):
        assert protocols.protocols_with_string(nothing) == []
    with pytest.raises(exceptions.ProtocolNotFoundError):
        protocols.protocols_with_string(joined + "/foo")


def test_registry_additions_aliases_and_locking():
    registry = protocols.ProtocolRegistry()
    proto = registry.add(protocols.Protocol(code=7777, name="carrier-pigeon", codec=None))
    assert registry.find("carrier-pigeon") is registry.find(7777) is registry.find(proto) is proto
    with pytest.raises(exceptions.ProtocolExistsError):
        registry.add(proto)
    with pytest.raises(exceptions.ProtocolExistsError):  # same code under another name
        registry.add(protocols.Protocol(code=7777, name="pigeon", codec=None))
    with pytest.raises(exceptions.ProtocolExistsError):  # same name under another code
        registry.add(protocols.Protocol(code=7778, name="carrier-pigeon", codec=None))
    with pytest.raises(TypeError):
        registry.find(3.5)

    assert protocols.REGISTRY.locked
    with pytest.raises(exceptions.ProtocolRegistryLocked):
        protocols.REGISTRY.add(proto)
    assert protocols.REGISTRY.copy().locked
    mine = protocols.REGISTRY.copy(unlock=True)
    assert not mine.locked
    mine.add_alias_name("tcp", "abcd")
    mine.add_alias_code("tcp", 123456)
    assert mine.find("abcd") is mine.find(123456) is mine.find("tcp")
    with pytest.raises(exceptions.ProtocolExistsError):
        mine.add_alias_name("tcp", "abcd")
    with pytest.raises(exceptions.ProtocolExistsError):
        mine.add_alias_code("tcp", 123456)
    with pytest.raises(exceptions.ProtocolNotFoundError):
        mine.add_alias_name("no-such-protocol", "x")
    with pytest.raises(exceptions.ProtocolNotFoundError):
        protocols.REGISTRY.find("abcd")  # the copy did not leak into the default registry
    mine.lock()
    for change in (lambda: mine.add(proto), lambda: mine.add_alias_name("tcp", "abcdef"),
                   lambda: mine.add_alias_code(0x4, 0x123456)):
        with pytest.raises(exceptions.ProtocolRegistryLocked):
            change()


def test_a_swapped_in_registry_is_honoured_and_unknown_codecs_are_parse_errors(monkeypatch):
    registry = protocols.REGISTRY.copy(unlock=True)
    registry.add(protocols.Protocol(333, "unparsable", "?"))
    registry.add(protocols.Protocol(7777, "carrier-pigeon", "utf8"))
    monkeypatch.setattr(protocols, "REGISTRY", registry)
    assert str(Multiaddr("/ip4/1.2.3.4/carrier-pigeon/gertrude")) == "/ip4/1.2.3.4/carrier-pigeon/gertrude"
    for text in ("test", "/ip4/", "/unparsable/5"):
        with pytest.raises(exceptions.StringParseError):
            transforms.string_to_bytes(text)
    with pytest.raises(exceptions.BinaryParseError):
        transforms.bytes_to_string(b"\xcd\x02\x0c\x0d")


# ------------------------------------------------------------------------------------------------ mapping interface
def test_mapping_interface_and_views():
    addr = Multiaddr(f"/dns4/example.com/tcp/443/wss/p2p/{PEER}")
    names = ["dns4", "tcp", "wss", "p2p"]
    assert [p.name for p in addr] == [p.name for p in addr.keys()] == [p.name for p in addr.protocols()] == names
    assert list(addr.values()) == ["example.com", "443", None, PEER] and len(addr) == 4
    assert [(p.name, v) for p, v in addr.items()] == list(zip(names, ["example.com", "443", None, PEER]))
    assert isinstance(addr.keys(), MultiAddrKeys) and isinstance(addr.items(), MultiAddrItems)
    assert isinstance(addr.values(), MultiAddrValues)
    assert addr.keys()[1].name == "tcp" and addr.values()[-1] == PEER and addr.items()[0][1] == "example.com"
    assert len(addr.keys()) == len(addr.values()) == len(addr.items()) == 4
    assert addr.values() == Multiaddr(addr.to_bytes()).values() and addr.keys() == addr.protocols()

    assert "tcp" in addr and protocols.P_TCP in addr and protocols.protocol_with_name("tcp") in addr
    assert "udp" not in addr and 0x7FFFFF not in addr and "no-such-protocol" not in addr and 3.5 not in addr
    assert "443" in addr.values() and None in addr.values() and "444" not in addr.values()
    assert ("tcp", "443") in addr.items() and ("tcp", "444") not in addr.items() and "tcp" not in addr.items()

    assert addr["tcp"] == addr[protocols.P_TCP] == addr[protocols.protocol_with_name("tcp")] == "443"
    assert addr.value_for_protocol("wss") is None and addr["p2p"] == PEER
    with pytest.raises(exceptions.ProtocolLookupError) as failure:
        addr["udp"]
    assert isinstance(failure.value, LookupError) and "udp" in str(failure.value)
    with pytest.raises(exceptions.ProtocolNotFoundError):
        addr["no-such-protocol"]
    with pytest.raises(TypeError):
        addr.value_for_protocol(None)
    repeated = Multiaddr("/ip4/1.1.1.1/udp/1/ip4/2.2.2.2/tcp/2")
    assert repeated["ip4"] == "1.1.1.1", "the first component of a protocol answers a lookup"
    assert dict(Multiaddr("/ip4/9.9.9.9/tcp/9"))[protocols.protocol_with_name("tcp")] == "9"  # a Mapping like any other


def test_equality_and_hashing():
    one, same, other = Multiaddr("/ip4/127.0.0.1/udp/1234"), Multiaddr("/ip4/127.0.0.1/udp/1234/"), Multiaddr("/ip4/127.0.0.1/tcp/1234")
    assert one == same and hash(one) == hash(same) and len({one, same, other}) == 2
    assert one != other and one != Multiaddr("/ip4/127.0.0.1/udp/1235") and one != Multiaddr("/ip4/127.0.0.2/udp/1234")
    assert one == "/ip4/127.0.0.1/udp/1234" and one != "/ip4/127.0.0.1" and one != "not an address" and one != 5
    assert Multiaddr(f"/p2p/{PEER}") == Multiaddr("/ipfs/" + PEER) == Multiaddr("/p2p/bafzbeigvf25ytwc3akrijfecaotc74udrhcxzh2cx3we5qqnw5vgrei4bm")


# ------------------------------------------------------------------------------------------------ nesting
@pytest.mark.parametrize("text,maxsplit,expected", [
    ("/ip4/1.2.3.4/tcp/80", -1, ["/ip4/1.2.3.4", "/tcp/80"]),
    ("/ip4/1.2.3.4/tcp/80", 0, ["/ip4/1.2.3.4/tcp/80"]),
    ("/ip4/1.2.3.4/tcp/80/ws", 1, ["/ip4/1.2.3.4", "/tcp/80/ws"]),
    ("/ip4/1.2.3.4/tcp/80/ws", 7, ["/ip4/1.2.3.4", "/tcp/80", "/ws"]),
    ("/ip4/1.2.3.4/tcp/80/unix/a/b/c", -1, ["/ip4/1.2.3.4", "/tcp/80", "/unix/a/b/c"]),
    (f"/ip4/0.0.0.0/udp/1/utp/p2p/{PEER}", 2, ["/ip4/0.0.0.0", "/udp/1", f"/utp/p2p/{PEER}"]),
    ("/", -1, []),
])
def test_split_and_join(text, maxsplit, expected):
    pieces = Multiaddr(text).split(maxsplit)
    assert [str(piece) for piece in pieces] == expected
    assert Multiaddr.join(*pieces) == Multiaddr(text) == Multiaddr.join(*expected)
    assert Multiaddr.join() == Multiaddr("/")


def test_encapsulate_and_decapsulate():
    base = Multiaddr("/ip4/127.0.0.1/udp/1234")
    nested = base.encapsulate("/udp/5678")
    assert str(nested) == "/ip4/127.0.0.1/udp/1234/udp/5678" and str(base) == "/ip4/127.0.0.1/udp/1234"
    assert str(nested.decapsulate("/udp/5678")) == "/ip4/127.0.0.1/udp/1234"
    assert str(nested.decapsulate("/udp/1234")) == "/ip4/127.0.0.1", "the suffix goes together with all that follows it"
    assert str(nested.decapsulate("/ip4/127.0.0.1")) == "/" and nested.decapsulate("/tcp/80") == nested
    assert nested.decapsulate("/") == nested and nested.decapsulate(Multiaddr("/udp/5678")) == base
    assert str(nested.decapsulate_code(protocols.P_UDP)) == "/ip4/127.0.0.1/udp/1234"
    assert str(nested.decapsulate_code(protocols.P_IP4)) == "/" and nested.decapsulate_code(protocols.P_TCP) == nested
    full = Multiaddr("/ip4/1.2.3.4").encapsulate("/tcp/4001").encapsulate(Multiaddr(f"/p2p/{PEER}"))
    assert str(full) == f"/ip4/1.2.3.4/tcp/4001/p2p/{PEER}"
    assert str(full.decapsulate(f"/p2p/{PEER}")) == "/ip4/1.2.3.4/tcp/4001"
    # a decimal suffix must match a whole component: /tcp/40 is not the beginning of /tcp/4001
    assert full.decapsulate("/tcp/40") == full
    zoned = Multiaddr("/ip6zone/eth0/ip6/fe80::1/tcp/22")
    assert zoned["ip6zone"] == "eth0" and str(zoned.decapsulate("/ip6/fe80::1")) == "/ip6zone/eth0"

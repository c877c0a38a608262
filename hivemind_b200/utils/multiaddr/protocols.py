"""Protocols of the multiaddr format and the registry that resolves them by name or code.

Codes are those of the multiformats registry; the list is the one the reference ships
(hivemind/utils/multiaddr/protocols.py:118-147). ``REGISTRY`` is the locked default registry; ``copy(unlock=True)``
gives one that accepts further protocols and aliases.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Union

from hivemind_b200.utils.base58 import varint_encode
from hivemind_b200.utils.multiaddr import exceptions
from hivemind_b200.utils.multiaddr.codecs import codec_by_name

P_IP4 = 0x04
P_IP6 = 0x29
P_IP6ZONE = 0x2A
P_TCP = 0x06
P_UDP = 0x0111
P_DCCP = 0x21
P_SCTP = 0x84
P_UDT = 0x012D
P_UTP = 0x012E
P_P2P = 0x01A5
P_HTTP = 0x01E0
P_HTTPS = 0x01BB
P_TLS = 0x01C0
P_QUIC = 0x01CC
P_QUIC1 = P_QUIC_V1 = 0x01CD
P_WS = 0x01DD
P_WSS = 0x01DE
P_ONION = 0x01BC
P_ONION3 = 0x01BD
P_P2P_CIRCUIT = 0x0122
P_DNS = 0x35
P_DNS4 = 0x36
P_DNS6 = 0x37
P_DNSADDR = 0x38
P_P2P_WEBSOCKET_STAR = 0x01DF
P_P2P_WEBRTC_STAR = 0x0113
P_P2P_WEBRTC_DIRECT = 0x0114
P_UNIX = 0x0190


class Protocol:
    """One protocol: its numeric code, its name in text addresses and the name of the codec of its value (or None)."""

    __slots__ = ("code", "name", "codec")

    def __init__(self, code: int, name: str, codec: Optional[str]):
        if not isinstance(code, int) or isinstance(code, bool):
            raise TypeError("code must be an integer")
        if not isinstance(name, str):
            raise TypeError("name must be a string")
        if codec is not None and not isinstance(codec, str):
            raise TypeError("codec must be a string or None")
        self.code, self.name, self.codec = code, name, codec

    @property
    def size(self) -> int:
        """Bits of the value: 0 for none, -1 when the value is prefixed with its length."""
        return codec_by_name(self.codec).SIZE

    @property
    def path(self) -> bool:
        """Whether the value takes the whole rest of a text address."""
        return codec_by_name(self.codec).IS_PATH

    @property
    def vcode(self) -> bytes:
        """The code as it appears in binary addresses (unsigned varint)."""
        return varint_encode(self.code)

    def __eq__(self, other) -> bool:
        if not isinstance(other, Protocol):
            return NotImplemented
        return (self.code, self.name, self.codec) == (other.code, other.name, other.codec)

    def __hash__(self) -> int:
        return self.code

    def __repr__(self) -> str:
        return f"Protocol(code={self.code!r}, name={self.name!r}, codec={self.codec!r})"


class ProtocolRegistry:
    """Name -> protocol and code -> protocol tables that are kept in step; aliases add further keys to either."""

    def __init__(self, protocols: Iterable[Protocol] = ()):
        self._locked = False
        self._names_to_protocols: Dict[str, Protocol] = {}
        self._codes_to_protocols: Dict[int, Protocol] = {}
        for proto in protocols:
            self.add(proto)

    def _require_unlocked(self) -> None:
        if self._locked:
            raise exceptions.ProtocolRegistryLocked()

    def add(self, proto: Protocol) -> Protocol:
        self._require_unlocked()
        if proto.name in self._names_to_protocols:
            raise exceptions.ProtocolExistsError(proto, "name")
        if proto.code in self._codes_to_protocols:
            raise exceptions.ProtocolExistsError(proto, "code")
        self._names_to_protocols[proto.name] = self._codes_to_protocols[proto.code] = proto
        return proto

    def add_alias_name(self, proto: Union[Protocol, str], alias_name: str) -> None:
        """Let ``alias_name`` resolve to an already registered protocol (given as object or by its name)."""
        self._require_unlocked()
        proto = self.find_by_name(proto if isinstance(proto, str) else proto.name)
        if alias_name in self._names_to_protocols:
            raise exceptions.ProtocolExistsError(self._names_to_protocols[alias_name], "name")
        self._names_to_protocols[alias_name] = proto

    def add_alias_code(self, proto: Union[Protocol, str, int], alias_code: int) -> None:
        """Let ``alias_code`` resolve to an already registered protocol (given as object, name or code)."""
        self._require_unlocked()
        proto = self.find(proto)
        if alias_code in self._codes_to_protocols:
            raise exceptions.ProtocolExistsError(self._codes_to_protocols[alias_code], "code")
        self._codes_to_protocols[alias_code] = proto

    def lock(self) -> None:
        self._locked = True

    @property
    def locked(self) -> bool:
        return self._locked

    def copy(self, *, unlock: bool = False) -> "ProtocolRegistry":
        twin = ProtocolRegistry()
        twin._names_to_protocols = dict(self._names_to_protocols)
        twin._codes_to_protocols = dict(self._codes_to_protocols)
        twin._locked = self._locked and not unlock
        return twin

    __copy__ = copy

    def find_by_name(self, name: str) -> Protocol:
        try:
            return self._names_to_protocols[name]
        except KeyError:
            raise exceptions.ProtocolNotFoundError(name, "name") from None

    def find_by_code(self, code: int) -> Protocol:
        try:
            return self._codes_to_protocols[code]
        except KeyError:
            raise exceptions.ProtocolNotFoundError(code, "code") from None

    def find(self, proto: Union[Protocol, str, int]) -> Protocol:
        """Resolve a protocol object (returned as it is), a name or a code."""
        if isinstance(proto, Protocol):
            return proto
        if isinstance(proto, str):
            return self.find_by_name(proto)
        if isinstance(proto, int) and not isinstance(proto, bool):
            return self.find_by_code(proto)
        raise TypeError(f"a protocol is named by a Protocol, a str or an int, not by {type(proto).__name__}")

    def __iter__(self):
        return iter(set(self._codes_to_protocols.values()))


PROTOCOLS = [
    Protocol(P_IP4, "ip4", "ip4"), Protocol(P_TCP, "tcp", "uint16be"), Protocol(P_UDP, "udp", "uint16be"),
    Protocol(P_DCCP, "dccp", "uint16be"), Protocol(P_IP6, "ip6", "ip6"), Protocol(P_IP6ZONE, "ip6zone", "utf8"),
    Protocol(P_DNS, "dns", "domain"), Protocol(P_DNS4, "dns4", "domain"), Protocol(P_DNS6, "dns6", "domain"),
    Protocol(P_DNSADDR, "dnsaddr", "domain"), Protocol(P_SCTP, "sctp", "uint16be"), Protocol(P_UDT, "udt", None),
    Protocol(P_UTP, "utp", None), Protocol(P_P2P, "p2p", "cid"), Protocol(P_ONION, "onion", "onion"),
    Protocol(P_ONION3, "onion3", "onion3"), Protocol(P_QUIC, "quic", None), Protocol(P_QUIC1, "quic-v1", None),
    Protocol(P_HTTP, "http", None), Protocol(P_HTTPS, "https", None), Protocol(P_TLS, "tls", None),
    Protocol(P_WS, "ws", None), Protocol(P_WSS, "wss", None),
    Protocol(P_P2P_WEBSOCKET_STAR, "p2p-websocket-star", None), Protocol(P_P2P_WEBRTC_STAR, "p2p-webrtc-star", None),
    Protocol(P_P2P_WEBRTC_DIRECT, "p2p-webrtc-direct", None), Protocol(P_P2P_CIRCUIT, "p2p-circuit", None),
    Protocol(P_UNIX, "unix", "fspath"),
]

REGISTRY = ProtocolRegistry(PROTOCOLS)
REGISTRY.add_alias_name("p2p", "ipfs")  # the name this protocol had before it was renamed
REGISTRY.lock()


def protocol_with_name(name: str) -> Protocol:
    return REGISTRY.find_by_name(name)


def protocol_with_code(code: int) -> Protocol:
    return REGISTRY.find_by_code(code)


def protocol_with_any(proto: Union[Protocol, str, int]) -> Protocol:
    return REGISTRY.find(proto)


def protocols_with_string(string: str) -> List[Protocol]:
    """The protocols named in a '/'-separated string such as ``"/ip4/tcp"`` (empty parts are skipped)."""
    return [protocol_with_name(part) for part in string.split("/") if part]

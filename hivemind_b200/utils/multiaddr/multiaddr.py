from __future__ import annotations

import ipaddress
from dataclasses import dataclass
from typing import Iterator, List, Optional, Tuple, Union

from hivemind_b200.utils.base58 import b58decode, b58encode, varint_decode, varint_encode
from hivemind_b200.utils.multiaddr import protocols as P


@dataclass(frozen=True)
class Protocol:
    code: int
    name: str
    size: int  # bits; 0 = no value; -1 = variable length
    path: bool = False  # the value swallows the rest of the address (unix paths)


_BY_NAME = {name: Protocol(code, name, size, path=(name == "unix")) for code, name, size in P.TABLE}
_BY_NAME["ipfs"] = _BY_NAME["p2p"]  # legacy alias
_BY_CODE = {proto.code: proto for proto in _BY_NAME.values()}


def protocol_with_name(name: str) -> Protocol:
    try:
        return _BY_NAME[name]
    except KeyError:
        raise ValueError(f"unknown multiaddr protocol {name!r}") from None


def protocol_with_code(code: int) -> Protocol:
    try:
        return _BY_CODE[code]
    except KeyError:
        raise ValueError(f"unknown multiaddr protocol code {code:#x}") from None


def _value_to_bytes(proto: Protocol, value: str) -> bytes:
    if proto.name == "ip4":
        return ipaddress.IPv4Address(value).packed
    if proto.name == "ip6":
        return ipaddress.IPv6Address(value).packed
    if proto.name in ("tcp", "udp"):
        port = int(value)
        if not 0 <= port < 65536:
            raise ValueError(f"port out of range: {value}")
        return port.to_bytes(2, "big")
    if proto.name == "p2p":
        raw = b58decode(value)
        return varint_encode(len(raw)) + raw
    raw = value.encode("utf-8")
    if proto.name == "unix" and not raw.startswith(b"/"):
        raw = b"/" + raw
    return varint_encode(len(raw)) + raw


def _value_from_bytes(proto: Protocol, buf: bytes, offset: int) -> Tuple[str, int]:
    if proto.size > 0:
        n = proto.size // 8
        chunk = buf[offset:offset + n]
        if len(chunk) != n:
            raise ValueError("truncated multiaddr")
        if proto.name == "ip4":
            return str(ipaddress.IPv4Address(chunk)), offset + n
        if proto.name == "ip6":
            return str(ipaddress.IPv6Address(chunk)), offset + n
        return str(int.from_bytes(chunk, "big")), offset + n
    length, offset = varint_decode(buf, offset)
    chunk = buf[offset:offset + length]
    if len(chunk) != length:
        raise ValueError("truncated multiaddr")
    if proto.name == "p2p":
        return b58encode(chunk), offset + length
    return chunk.decode("utf-8"), offset + length


class Multiaddr:
    """Immutable multiaddr; construct from text (``"/ip4/.../tcp/..."``), bytes, or another Multiaddr."""

    __slots__ = ("_parts",)

    def __init__(self, addr: Union[str, bytes, "Multiaddr"] = ""):
        if isinstance(addr, Multiaddr):
            self._parts = list(addr._parts)
        elif isinstance(addr, (bytes, bytearray)):
            self._parts = self._parse_bytes(bytes(addr))
        elif isinstance(addr, str):
            self._parts = self._parse_text(addr)
        else:
            raise TypeError(f"cannot build a Multiaddr from {type(addr)}")

    @staticmethod
    def _parse_text(text: str) -> List[Tuple[Protocol, Optional[str]]]:
        text = text.rstrip("/") if text != "/" else ""
        if not text:
            return []
        if not text.startswith("/"):
            raise ValueError(f"a multiaddr must begin with '/': {text!r}")
        items = text.split("/")[1:]
        parts, i = [], 0
        while i < len(items):
            proto = protocol_with_name(items[i])
            i += 1
            if proto.size == 0:
                parts.append((proto, None))
                continue
            if i >= len(items):
                raise ValueError(f"protocol {proto.name} requires a value: {text!r}")
            if proto.path:
                value = "/" + "/".join(items[i:])
                i = len(items)
            else:
                value = items[i]
                i += 1
            _value_to_bytes(proto, value)  # validates
            parts.append((proto, value))
        return parts

    @staticmethod
    def _parse_bytes(buf: bytes) -> List[Tuple[Protocol, Optional[str]]]:
        parts, offset = [], 0
        while offset < len(buf):
            code, offset = varint_decode(buf, offset)
            proto = protocol_with_code(code)
            if proto.size == 0:
                parts.append((proto, None))
                continue
            value, offset = _value_from_bytes(proto, buf, offset)
            parts.append((proto, value))
        return parts

    def to_bytes(self) -> bytes:
        out = bytearray()
        for proto, value in self._parts:
            out += varint_encode(proto.code)
            if value is not None:
                out += _value_to_bytes(proto, value)
        return bytes(out)

    def __bytes__(self) -> bytes:
        return self.to_bytes()

    def __str__(self) -> str:
        chunks = []
        for proto, value in self._parts:
            chunks.append("/" + proto.name)
            if value is not None:
                chunks.append(value if proto.path else "/" + value)
        return "".join(chunks) or "/"

    def __repr__(self) -> str:
        return f"<Multiaddr {self}>"

    def __eq__(self, other) -> bool:
        if isinstance(other, str):
            try:
                other = Multiaddr(other)
            except ValueError:
                return False
        return isinstance(other, Multiaddr) and str(self) == str(other)

    def __hash__(self) -> int:
        return hash(str(self))

    def __iter__(self) -> Iterator[Tuple[Protocol, Optional[str]]]:
        return iter(self._parts)

    def protocols(self) -> List[Protocol]:
        return [proto for proto, _ in self._parts]

    def items(self) -> List[Tuple[Protocol, Optional[str]]]:
        return list(self._parts)

    def values(self) -> List[Optional[str]]:
        return [value for _, value in self._parts]

    def value_for_protocol(self, proto: Union[int, str]) -> Optional[str]:
        """The value of the first component with this protocol; raises LookupError if absent."""
        for p, value in self._parts:
            if p.code == proto or p.name == proto:
                return value
        raise LookupError(f"{self} has no {proto} component")

    def __getitem__(self, proto: Union[int, str]) -> Optional[str]:
        return self.value_for_protocol(proto)

    def __contains__(self, proto: Union[int, str]) -> bool:
        return any(p.code == proto or p.name == proto for p, _ in self._parts)

    def encapsulate(self, other: Union[str, "Multiaddr"]) -> "Multiaddr":
        result = Multiaddr(self)
        result._parts.extend(Multiaddr(other)._parts)
        return result

    def decapsulate(self, other: Union[str, "Multiaddr"]) -> "Multiaddr":
        """Remove the last occurrence of ``other`` and everything after it."""
        mine, theirs = str(self), str(Multiaddr(other))
        index = mine.rfind(theirs)
        return Multiaddr(self) if index < 0 else Multiaddr(mine[:index])

    def decapsulate_code(self, code: int) -> "Multiaddr":
        for i in range(len(self._parts) - 1, -1, -1):
            if self._parts[i][0].code == code:
                result = Multiaddr()
                result._parts = self._parts[:i]
                return result
        return Multiaddr(self)

    def split(self) -> List["Multiaddr"]:
        out = []
        for part in self._parts:
            m = Multiaddr()
            m._parts = [part]
            out.append(m)
        return out

    @classmethod
    def join(cls, *addrs: Union[str, "Multiaddr"]) -> "Multiaddr":
        result = cls()
        for a in addrs:
            result._parts.extend(cls(a)._parts)
        return result

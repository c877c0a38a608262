"""``Multiaddr``: an immutable, self-describing network address such as ``/ip4/127.0.0.1/tcp/4001/p2p/Qm...``.

The object holds the canonical binary form; text is produced on demand. It behaves like a read-only ordered mapping
from protocols to values (``keys()`` / ``values()`` / ``items()``, ``addr["tcp"]``, ``"p2p" in addr``), and addresses
nest: ``encapsulate`` appends components, ``decapsulate`` removes a suffix. Same interface as the class the reference
vendors from py-multiaddr (hivemind/utils/multiaddr/multiaddr.py:76-258).
"""
from __future__ import annotations

import collections.abc
from typing import Iterator, List, Optional, Tuple, Union

from hivemind_b200.utils.multiaddr import exceptions, protocols
from hivemind_b200.utils.multiaddr.protocols import Protocol, protocol_with_code, protocol_with_name  # noqa: F401
from hivemind_b200.utils.multiaddr.transforms import bytes_iter, bytes_to_string, string_to_bytes

__all__ = ("Multiaddr", "MultiAddrKeys", "MultiAddrItems", "MultiAddrValues")


def _decoded_components(raw: bytes) -> Iterator[Tuple[Protocol, Optional[str]]]:
    for _, proto, codec, value in bytes_iter(raw):
        if codec.SIZE == 0:
            yield proto, None
            continue
        try:
            yield proto, codec.to_string(proto, value)
        except Exception as e:
            raise exceptions.BinaryParseError(str(e), raw, proto.name, e) from e


class _View:
    """Shared behaviour of the three views: sized, comparable with any sequence of the same elements."""

    def __init__(self, mapping: "Multiaddr"):
        self._mapping = mapping

    def __len__(self) -> int:
        return sum(1 for _ in bytes_iter(self._mapping.to_bytes()))

    def __eq__(self, other) -> bool:
        try:
            return list(self) == list(other)
        except TypeError:
            return NotImplemented

    def __repr__(self) -> str:
        return f"{type(self).__name__}({list(self)!r})"


class MultiAddrKeys(_View, collections.abc.KeysView, collections.abc.Sequence):
    """The protocols of an address, in order; membership accepts a protocol object, a name or a code."""

    def __contains__(self, proto) -> bool:
        try:
            wanted = protocols.REGISTRY.find(proto)
        except (exceptions.ProtocolNotFoundError, TypeError):
            return False
        return any(present == wanted for present in self)

    def __getitem__(self, index):
        return list(self)[index]

    def __iter__(self) -> Iterator[Protocol]:
        for _, proto, _, _ in bytes_iter(self._mapping.to_bytes()):
            yield proto

    __hash__ = collections.abc.KeysView._hash


class MultiAddrItems(_View, collections.abc.ItemsView, collections.abc.Sequence):
    """``(protocol, value text or None)`` pairs, in order."""

    def __contains__(self, item) -> bool:
        try:
            proto, value = item
            wanted = protocols.REGISTRY.find(proto)
        except (exceptions.ProtocolNotFoundError, TypeError, ValueError):
            return False
        return any(present == wanted and held == value for present, held in self)

    def __getitem__(self, index):
        return list(self)[index]

    def __iter__(self) -> Iterator[Tuple[Protocol, Optional[str]]]:
        return _decoded_components(self._mapping.to_bytes())


class MultiAddrValues(_View, collections.abc.ValuesView, collections.abc.Sequence):
    """The values, in order (None for protocols without one)."""

    def __contains__(self, value) -> bool:
        return any(held == value for held in self)

    def __getitem__(self, index):
        return list(self)[index]

    def __iter__(self) -> Iterator[Optional[str]]:
        for _, value in _decoded_components(self._mapping.to_bytes()):
            yield value


class Multiaddr(collections.abc.Mapping):
    """Build from text (``"/ip4/1.2.3.4/tcp/80"``), from the binary form, or from another ``Multiaddr``."""

    __slots__ = ("_bytes",)

    def __init__(self, addr: Union[str, bytes, "Multiaddr"] = "/"):
        if isinstance(addr, Multiaddr):
            self._bytes = addr._bytes
        elif isinstance(addr, (bytes, bytearray, memoryview)):
            raw = bytes(addr)
            for _ in _decoded_components(raw):  # refuse what cannot be read back
                pass
            self._bytes = raw
        elif isinstance(addr, str):
            self._bytes = string_to_bytes(addr) if addr.strip("/") else b""
        else:
            raise TypeError(f"MultiAddr must be bytes, str or another MultiAddr instance, not {type(addr).__name__}")

    @classmethod
    def _from_canonical_bytes(cls, raw: bytes) -> "Multiaddr":
        result = cls.__new__(cls)
        result._bytes = raw
        return result

    @classmethod
    def join(cls, *addrs: Union[str, bytes, "Multiaddr"]) -> "Multiaddr":
        """One address made of the components of all the given ones, in order."""
        return cls._from_canonical_bytes(b"".join(cls(addr).to_bytes() for addr in addrs))

    # --- forms -----------------------------------------------------------------------------------------------
    def to_bytes(self) -> bytes:
        return self._bytes

    __bytes__ = to_bytes

    def __str__(self) -> str:
        return bytes_to_string(self._bytes) or "/"

    def __repr__(self) -> str:
        return f"<Multiaddr {self}>"

    def __eq__(self, other) -> bool:
        if isinstance(other, str):  # convenience that the framework's own code relies on
            try:
                other = Multiaddr(other)
            except exceptions.ParseError:
                return False
        if not isinstance(other, Multiaddr):
            return NotImplemented
        return self._bytes == other._bytes

    def __hash__(self) -> int:
        return hash(self._bytes)

    # --- mapping ---------------------------------------------------------------------------------------------
    def __iter__(self) -> Iterator[Protocol]:
        return iter(MultiAddrKeys(self))

    def __len__(self) -> int:
        return len(MultiAddrKeys(self))

    def __contains__(self, proto) -> bool:
        return proto in MultiAddrKeys(self)

    def keys(self) -> MultiAddrKeys:
        return MultiAddrKeys(self)

    def values(self) -> MultiAddrValues:
        return MultiAddrValues(self)

    def items(self) -> MultiAddrItems:
        return MultiAddrItems(self)

    def protocols(self) -> MultiAddrKeys:
        """The protocols this address goes through, outermost first."""
        return MultiAddrKeys(self)

    def value_for_protocol(self, proto: Union[Protocol, str, int]) -> Optional[str]:
        """The value of the first component of this protocol (None if the protocol has no value);
        ``ProtocolLookupError`` (a ``LookupError``) if the address does not contain the protocol."""
        wanted = protocols.REGISTRY.find(proto)
        for present, value in self.items():
            if present == wanted:
                return value
        raise exceptions.ProtocolLookupError(wanted, str(self))

    def __getitem__(self, proto: Union[Protocol, str, int]) -> Optional[str]:
        return self.value_for_protocol(proto)

    # --- nesting ---------------------------------------------------------------------------------------------
    def _component_spans(self) -> List[Tuple[int, int, Protocol]]:
        spans, offset = [], 0
        for header, proto, _, value in bytes_iter(self._bytes):
            spans.append((offset, offset + header + len(value), proto))
            offset += header + len(value)
        return spans

    def split(self, maxsplit: int = -1) -> List["Multiaddr"]:
        """One address per component; with ``maxsplit`` >= 0 the last element keeps everything beyond that many."""
        pieces, spans = [], self._component_spans()
        for index, (start, stop, _) in enumerate(spans):
            if index == maxsplit:
                pieces.append(self._from_canonical_bytes(self._bytes[start:]))
                break
            pieces.append(self._from_canonical_bytes(self._bytes[start:stop]))
        return pieces

    def encapsulate(self, other: Union[str, bytes, "Multiaddr"]) -> "Multiaddr":
        """This address with ``other`` nested inside it: ``/ip4/1.2.3.4`` + ``/tcp/80`` -> ``/ip4/1.2.3.4/tcp/80``."""
        return self._from_canonical_bytes(self._bytes + Multiaddr(other).to_bytes())

    def decapsulate(self, other: Union[str, bytes, "Multiaddr"]) -> "Multiaddr":
        """This address up to (not including) the last place where ``other`` begins; unchanged if it never does."""
        suffix = Multiaddr(other).to_bytes()
        if not suffix:
            return self
        for start, _, _ in reversed(self._component_spans()):
            if self._bytes.startswith(suffix, start):
                return self._from_canonical_bytes(self._bytes[:start])
        return self

    def decapsulate_code(self, code: int) -> "Multiaddr":
        """This address up to (not including) the last component whose protocol has this code."""
        for start, _, proto in reversed(self._component_spans()):
            if proto.code == code:
                return self._from_canonical_bytes(self._bytes[:start])
        return self

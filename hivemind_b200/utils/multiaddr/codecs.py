"""Value codecs of multiaddr components: text <-> bytes for every kind of value a protocol can carry.

A codec is an object with ``SIZE`` (bits of a fixed-size value, ``-1`` for a length-prefixed value, ``0`` for none),
``IS_PATH`` (the value swallows the rest of a text address) and ``to_bytes(proto, string)`` / ``to_string(proto, buf)``.
Codecs raise whatever fits (``ValueError`` mostly); ``transforms`` wraps that into parse errors. The reference keeps one
module per codec (hivemind/utils/multiaddr/codecs/*.py); here they are small classes in one table, ``codec_by_name``.
"""
from __future__ import annotations

import base64
import ipaddress
import unicodedata
from typing import Dict, Optional, Tuple

from hivemind_b200.utils.base58 import b58decode, b58encode, varint_decode, varint_encode

LENGTH_PREFIXED_VAR_SIZE = -1


class _NoValue:
    """Protocols such as /quic or /ws that are a bare flag."""
    SIZE, IS_PATH = 0, False

    def to_bytes(self, proto, string: str) -> bytes:
        raise ValueError(f"protocol {getattr(proto, 'name', proto)} takes no value")

    def to_string(self, proto, buf: bytes) -> str:
        raise ValueError(f"protocol {getattr(proto, 'name', proto)} takes no value")


class _Ip4:
    SIZE, IS_PATH = 32, False

    def to_bytes(self, proto, string: str) -> bytes:
        return ipaddress.IPv4Address(string).packed

    def to_string(self, proto, buf: bytes) -> str:
        return str(ipaddress.IPv4Address(bytes(buf)))


class _Ip6:
    SIZE, IS_PATH = 128, False

    def to_bytes(self, proto, string: str) -> bytes:
        return ipaddress.IPv6Address(string).packed

    def to_string(self, proto, buf: bytes) -> str:
        return str(ipaddress.IPv6Address(bytes(buf)))


class _Uint16BigEndian:
    """Port numbers."""
    SIZE, IS_PATH = 16, False

    def to_bytes(self, proto, string: str) -> bytes:
        if not (string.isascii() and string.isdigit()):
            raise ValueError(f"not a decimal port number: {string!r}")
        number = int(string)
        if number > 0xFFFF:
            raise ValueError(f"port out of range: {number}")
        return number.to_bytes(2, "big")

    def to_string(self, proto, buf: bytes) -> str:
        if len(buf) != 2:
            raise ValueError("a port takes exactly two bytes")
        return str(int.from_bytes(buf, "big"))


class _Utf8:
    """Free text without a slash (IPv6 zone names)."""
    SIZE, IS_PATH = LENGTH_PREFIXED_VAR_SIZE, False

    def to_bytes(self, proto, string: str) -> bytes:
        if not string or "/" in string:
            raise ValueError(f"{getattr(proto, 'name', proto)} needs a non-empty value without '/'")
        return string.encode("utf-8")

    def to_string(self, proto, buf: bytes) -> str:
        if not buf:
            raise ValueError(f"{getattr(proto, 'name', proto)} value is empty")
        text = bytes(buf).decode("utf-8")
        if "/" in text:
            raise ValueError("value contains '/'")
        return text


def _check_domain(name: str) -> str:
    """Validate an (internationalised) host name and return it in its unicode form."""
    try:
        import idna
    except ImportError:
        idna = None
    if idna is not None:
        return idna.decode(idna.encode(name, uts46=True))
    labels = name.rstrip(".").split(".")
    if not name or any(not label for label in labels):
        raise ValueError(f"empty label in host name {name!r}")
    for label in labels:
        ascii_form = label if label.isascii() else "xn--" + label.encode("punycode").decode("ascii")
        if len(ascii_form) > 63 or label.startswith("-") or label.endswith("-"):
            raise ValueError(f"bad label {label!r} in host name {name!r}")
        for char in label:
            if char.isascii():
                if not (char.isalnum() or char in "-_"):
                    raise ValueError(f"character {char!r} is not allowed in a host name")
            elif unicodedata.category(char)[0] in "ZCPS":  # separators, control, punctuation, symbols
                raise ValueError(f"character {char!r} is not allowed in a host name")
    return unicodedata.normalize("NFC", name)


class _Domain:
    """Host names, kept as UTF-8 text of their unicode form (IDNA 2008 rules: 'ß' stays 'ß')."""
    SIZE, IS_PATH = LENGTH_PREFIXED_VAR_SIZE, False

    def to_bytes(self, proto, string: str) -> bytes:
        return _check_domain(string).encode("utf-8")

    def to_string(self, proto, buf: bytes) -> str:
        return _check_domain(bytes(buf).decode("utf-8"))


class _FilesystemPath:
    """Unix socket paths: everything after ``/unix`` belongs to the value."""
    SIZE, IS_PATH = LENGTH_PREFIXED_VAR_SIZE, True

    def to_bytes(self, proto, string: str) -> bytes:
        if not string.strip("/"):
            raise ValueError("empty path")
        return string.encode("utf-8", "surrogateescape")

    def to_string(self, proto, buf: bytes) -> str:
        if not buf:
            raise ValueError("empty path")
        return bytes(buf).decode("utf-8", "surrogateescape")


def _base32_decode(text: str, expected_chars: int) -> bytes:
    if len(text) != expected_chars or not text.isascii():
        raise ValueError(f"expected {expected_chars} base32 characters, got {text!r}")
    return base64.b32decode(text.upper() + "=" * (-len(text) % 8))


def _base32_encode(raw: bytes) -> str:
    return base64.b32encode(raw).decode("ascii").rstrip("=").lower()


class _Onion:
    """Tor hidden services: ``<base32 host>:<port>``; 10 host bytes (v2) or 35 (v3), then a 16-bit port."""
    IS_PATH = False

    def __init__(self, host_bytes: int, host_chars: int):
        self.host_bytes, self.host_chars = host_bytes, host_chars
        self.SIZE = 8 * (host_bytes + 2)

    def to_bytes(self, proto, string: str) -> bytes:
        host, separator, port_text = string.partition(":")
        if not separator or not (port_text.isascii() and port_text.isdigit()):
            raise ValueError(f"{string!r} is not of the form host:port")
        port = int(port_text)
        if not 1 <= port <= 0xFFFF:
            raise ValueError(f"port out of range: {port}")
        raw = _base32_decode(host, self.host_chars)
        if len(raw) != self.host_bytes:
            raise ValueError("wrong host length")
        return raw + port.to_bytes(2, "big")

    def to_string(self, proto, buf: bytes) -> str:
        if len(buf) != self.host_bytes + 2:
            raise ValueError("wrong value length")
        port = int.from_bytes(buf[-2:], "big")
        if port == 0:
            raise ValueError("port 0")
        return f"{_base32_encode(bytes(buf[:-2]))}:{port}"


_LIBP2P_KEY = 0x72  # the multicodec of a CID that names a libp2p public key
_MULTIBASES = {
    "b": lambda body: base64.b32decode(body.upper() + "=" * (-len(body) % 8)),
    "B": lambda body: base64.b32decode(body + "=" * (-len(body) % 8)),
    "z": b58decode,
    "f": bytes.fromhex,
    "F": bytes.fromhex,
}


def _split_multihash(raw: bytes, offset: int = 0) -> Tuple[int, bytes]:
    """(hash function code, digest) of the multihash that fills ``raw[offset:]`` exactly."""
    code, offset = varint_decode(raw, offset)
    length, offset = varint_decode(raw, offset)
    digest = raw[offset:]
    if len(digest) != length:
        raise ValueError(f"multihash announces {length} digest bytes but carries {len(digest)}")
    return code, digest


def _split_cid_v1(raw: bytes) -> Tuple[int, bytes]:
    """(content codec, multihash bytes) of a binary CIDv1."""
    version, offset = varint_decode(raw, 0)
    if version != 1:
        raise ValueError(f"unsupported CID version {version}")
    codec, offset = varint_decode(raw, offset)
    _split_multihash(raw, offset)
    return codec, raw[offset:]


class _ContentId:
    """Peer ids and other content ids. Text: a base58 multihash (``Qm...``, ``12D3Koo...``) or a multibase CIDv1
    (``bafz...``). Bytes: a bare multihash or a binary CIDv1. For ``/p2p`` the two spellings are converted into each
    other the way py-multiaddr does it: a base58 peer id is stored as a CIDv1 with the libp2p-key codec, and shown
    as base58 again; any other codec is refused there."""
    SIZE, IS_PATH = LENGTH_PREFIXED_VAR_SIZE, False

    @staticmethod
    def _is_peer_id(proto) -> bool:
        return getattr(proto, "name", None) == "p2p"

    def to_bytes(self, proto, string: str) -> bytes:
        if string[:2] == "Qm" or string[:1] == "1":
            multihash = b58decode(string)
            _split_multihash(multihash)
            if self._is_peer_id(proto):
                return varint_encode(1) + varint_encode(_LIBP2P_KEY) + multihash
            return multihash
        decoder = _MULTIBASES.get(string[:1])
        if decoder is None:
            raise ValueError(f"unknown multibase prefix in {string!r}")
        raw = decoder(string[1:])
        codec, _ = _split_cid_v1(raw)
        if self._is_peer_id(proto) and codec != _LIBP2P_KEY:
            raise ValueError("a /p2p value must be a CID of type libp2p-key")
        return raw

    def to_string(self, proto, buf: bytes) -> str:
        raw = bytes(buf)
        if raw[:1] == b"\x01":
            codec, multihash = _split_cid_v1(raw)
            if self._is_peer_id(proto):
                if codec != _LIBP2P_KEY:
                    raise ValueError("a /p2p value must be a CID of type libp2p-key")
                return b58encode(multihash)
            return "b" + _base32_encode(raw)
        _split_multihash(raw)
        return b58encode(raw)


_CODECS: Dict[Optional[str], object] = {
    None: _NoValue(), "ip4": _Ip4(), "ip6": _Ip6(), "uint16be": _Uint16BigEndian(), "utf8": _Utf8(), "domain": _Domain(),
    "fspath": _FilesystemPath(), "onion": _Onion(10, 16), "onion3": _Onion(35, 56), "cid": _ContentId(),
}
NoneCodec = _CODECS[None]


def codec_by_name(name: Optional[str]):
    """The codec object registered under ``name`` (``None``: the codec of value-less protocols)."""
    try:
        return _CODECS[name]
    except KeyError:
        raise ImportError(f"no multiaddr codec named {name!r}") from None


def known_codec_names():
    return [name for name in _CODECS if name is not None]

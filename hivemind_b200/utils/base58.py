"""Base58 (Bitcoin alphabet) and unsigned varints — the two encodings that peer ids and multiaddrs need.

The reference imports them from the third-party ``base58`` and ``varint`` wheels (requirements.txt); they are a few
lines each, so they live here.
"""
from __future__ import annotations

from typing import Tuple

_ALPHABET = b"123456789ABCDEFGHJKLMNPQRSTUVWXYZabcdefghijkmnopqrstuvwxyz"
_INDEX = {c: i for i, c in enumerate(_ALPHABET)}


def b58encode(data: bytes) -> str:
    n_zeros = len(data) - len(data.lstrip(b"\0"))
    num = int.from_bytes(data, "big")
    out = bytearray()
    while num > 0:
        num, rem = divmod(num, 58)
        out.append(_ALPHABET[rem])
    return (b"1" * n_zeros + bytes(reversed(out))).decode("ascii")


def b58decode(text: str) -> bytes:
    raw = text.encode("ascii") if isinstance(text, str) else bytes(text)
    n_zeros = len(raw) - len(raw.lstrip(b"1"))
    num = 0
    for c in raw:
        try:
            num = num * 58 + _INDEX[c]
        except KeyError:
            raise ValueError(f"invalid base58 character {chr(c)!r}") from None
    body = num.to_bytes((num.bit_length() + 7) // 8, "big") if num else b""
    return b"\0" * n_zeros + body


def varint_encode(value: int) -> bytes:
    assert value >= 0
    out = bytearray()
    while True:
        byte = value & 0x7F
        value >>= 7
        out.append(byte | (0x80 if value else 0))
        if not value:
            return bytes(out)


def varint_decode(buf: bytes, offset: int = 0) -> Tuple[int, int]:
    """Returns (value, next offset)."""
    shift = result = 0
    while True:
        if offset >= len(buf):
            raise ValueError("truncated varint")
        byte = buf[offset]
        offset += 1
        result |= (byte & 0x7F) << shift
        if not byte & 0x80:
            return result, offset
        shift += 7
        if shift > 63:
            raise ValueError("varint is too long")

"""Text address <-> binary address, and iteration over the components of either form.

Binary layout: for each component the protocol code as an unsigned varint, then the value: nothing, a fixed number of
bytes, or a varint length followed by that many bytes (hivemind/utils/multiaddr/transforms.py:34-117 has the same
contract). The registry is looked up through the ``protocols`` module at call time, so a registry that a caller swapped
in is honoured.
"""
from __future__ import annotations

import io
from typing import Iterator, Optional, Tuple

from hivemind_b200.utils.base58 import varint_encode
from hivemind_b200.utils.multiaddr import exceptions, protocols
from hivemind_b200.utils.multiaddr.codecs import LENGTH_PREFIXED_VAR_SIZE, codec_by_name


def _codec_of(proto):
    try:
        return codec_by_name(proto.codec)
    except ImportError as e:
        raise LookupError(f"protocol {proto.name} names the unknown codec {proto.codec!r}") from e


def string_iter(string: str) -> Iterator[Tuple[object, object, Optional[str]]]:
    """Yield ``(protocol, codec, value text or None)`` for every component of a text address."""
    if not string.startswith("/"):
        raise exceptions.StringParseError("Must begin with /", string)
    parts = string.rstrip("/").split("/")[1:]
    cursor = 0
    while cursor < len(parts):
        name = parts[cursor]
        cursor += 1
        try:
            proto = protocols.REGISTRY.find_by_name(name)
        except exceptions.ProtocolNotFoundError as e:
            raise exceptions.StringParseError(f"Unknown Protocol {name!r}", string, name) from e
        try:
            codec = _codec_of(proto)
        except LookupError as e:
            raise exceptions.StringParseError(str(e), string, name, e) from e
        if codec.SIZE == 0:
            yield proto, codec, None
            continue
        if cursor >= len(parts):
            raise exceptions.StringParseError("Protocol requires address", string, name)
        if codec.IS_PATH:
            value, cursor = "/" + "/".join(parts[cursor:]), len(parts)
        else:
            value = parts[cursor]
            cursor += 1
        yield proto, codec, value


def string_to_bytes(string: str) -> bytes:
    out = bytearray()
    for proto, codec, value in string_iter(string):
        out += varint_encode(proto.code)
        if value is None:
            continue
        try:
            encoded = codec.to_bytes(proto, value)
        except Exception as e:
            raise exceptions.StringParseError(str(e), string, proto.name, e) from e
        if codec.SIZE == LENGTH_PREFIXED_VAR_SIZE:
            out += varint_encode(len(encoded))
        out += encoded
    return bytes(out)


def _read_varint(stream: io.BytesIO) -> Tuple[int, int]:
    """(value, number of bytes consumed); raises EOFError when the stream ends inside the number."""
    value = shift = consumed = 0
    while True:
        byte = stream.read(1)
        if not byte:
            raise EOFError("the address ends inside a varint")
        consumed += 1
        value |= (byte[0] & 0x7F) << shift
        if not byte[0] & 0x80:
            return value, consumed
        shift += 7
        if shift > 63:
            raise ValueError("varint is too long")


def size_for_addr(codec, buf_io: io.BytesIO) -> Tuple[int, int]:
    """``(bytes of the value that follows, bytes of its length prefix)`` for a value of ``codec`` at the stream's
    position; the prefix, if there is one, is consumed."""
    if codec.SIZE >= 0:
        return codec.SIZE // 8, 0
    return _read_varint(buf_io)


def bytes_iter(buf: bytes) -> Iterator[Tuple[int, object, object, bytes]]:
    """Yield ``(bytes consumed by code and length prefix, protocol, codec, value bytes)`` per component."""
    stream = io.BytesIO(buf)
    while stream.tell() < len(buf):
        try:
            code, consumed = _read_varint(stream)
        except (EOFError, ValueError) as e:
            raise exceptions.BinaryParseError(str(e), buf, None, e) from e
        try:
            proto = protocols.REGISTRY.find_by_code(code)
        except exceptions.ProtocolNotFoundError as e:
            raise exceptions.BinaryParseError(f"Unknown Protocol code {code}", buf, code, e) from e
        try:
            codec = _codec_of(proto)
            size, prefix = size_for_addr(codec, stream)
        except (LookupError, EOFError, ValueError) as e:
            raise exceptions.BinaryParseError(str(e), buf, proto.name, e) from e
        value = stream.read(size)
        if len(value) != size:
            raise exceptions.BinaryParseError(f"value of {size} bytes is cut short after {len(value)}", buf, proto.name)
        yield consumed + prefix, proto, codec, value


def bytes_to_string(buf: bytes) -> str:
    chunks = []
    for _, proto, codec, value in bytes_iter(buf):
        chunks.append("/" + proto.name)
        if codec.SIZE == 0:
            continue
        try:
            text = codec.to_string(proto, value)
        except Exception as e:
            raise exceptions.BinaryParseError(str(e), buf, proto.name, e) from e
        chunks.append(text if codec.IS_PATH and text.startswith("/") else "/" + text)
    return "".join(chunks)

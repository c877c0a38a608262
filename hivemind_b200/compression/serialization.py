"""Tensor <-> protobuf helpers and chunked streaming (hivemind/compression/serialization.py:13-68,
hivemind/utils/streaming.py:14-46)."""
from __future__ import annotations

from typing import AsyncIterator, Dict, Iterable, Iterator, List, Optional, Tuple

import torch

from hivemind_b200.compression.base import CompressionBase, CompressionInfo, NoCompression
from hivemind_b200.compression.floating import Float16Compression, ScaledFloat16Compression
from hivemind_b200.compression.quantization import (BlockwiseQuantization, Quantile8BitQuantization,
                                                    Uniform8BitQuantization)
from hivemind_b200.proto import runtime_pb2
from hivemind_b200.proto.runtime_pb2 import CompressionType

STREAMING_CHUNK_SIZE_BYTES = 2 ** 16

_BASE_COMPRESSION_TYPES: Dict[str, CompressionBase] = dict(
    NONE=NoCompression(), FLOAT16=Float16Compression(), MEANSTD_16BIT=ScaledFloat16Compression(),
    QUANTILE_8BIT=Quantile8BitQuantization(), UNIFORM_8BIT=Uniform8BitQuantization(),
    BLOCKWISE_8BIT=BlockwiseQuantization())
for _name, _number in CompressionType.items():
    assert _name in _BASE_COMPRESSION_TYPES, f"no codec registered for {_name}"
    assert _BASE_COMPRESSION_TYPES[_name].compression_type == _number, f"codec for {_name} reports a different type"


def serialize_torch_tensor(tensor: torch.Tensor, compression_type: int = CompressionType.NONE,
                           info: Optional[CompressionInfo] = None, allow_inplace: bool = False, **kwargs
                           ) -> runtime_pb2.Tensor:
    """Encode ``tensor`` with the codec registered for ``compression_type``."""
    codec = _BASE_COMPRESSION_TYPES[CompressionType.Name(compression_type)]
    info = info or CompressionInfo.from_tensor(tensor, **kwargs)
    return codec.compress(tensor, info, allow_inplace)


def deserialize_torch_tensor(serialized_tensor: runtime_pb2.Tensor) -> torch.Tensor:
    """Decode any message produced by one of the registered codecs."""
    return _BASE_COMPRESSION_TYPES[CompressionType.Name(serialized_tensor.compression)].extract(serialized_tensor)


def split_for_streaming(serialized_tensor: runtime_pb2.Tensor, chunk_size_bytes: int = STREAMING_CHUNK_SIZE_BYTES
                        ) -> Iterator[runtime_pb2.Tensor]:
    """Cut a message into chunks; the first chunk carries the metadata and the total number of chunks."""
    buffer = memoryview(serialized_tensor.buffer)
    num_chunks = len(range(0, len(buffer), chunk_size_bytes))
    yield runtime_pb2.Tensor(compression=serialized_tensor.compression, buffer=buffer[:chunk_size_bytes].tobytes(),
                             chunks=num_chunks, size=serialized_tensor.size, dtype=serialized_tensor.dtype,
                             requires_grad=serialized_tensor.requires_grad)
    for start in range(chunk_size_bytes, len(buffer), chunk_size_bytes):
        yield runtime_pb2.Tensor(buffer=buffer[start:start + chunk_size_bytes].tobytes())


def combine_from_streaming(stream: Iterable[runtime_pb2.Tensor]) -> runtime_pb2.Tensor:
    """Inverse of ``split_for_streaming``."""
    stream = iter(stream)
    first = next(stream)
    combined = runtime_pb2.Tensor()
    combined.CopyFrom(first)
    combined.buffer = b"".join([first.buffer] + [chunk.buffer for chunk in stream])
    combined.chunks = 0  # the combined message is whole again
    return combined


async def deserialize_tensor_stream(stream: AsyncIterator[Iterable[runtime_pb2.Tensor]]) -> List[torch.Tensor]:
    """Rebuild tensors from a stream of chunk batches, where a chunk with ``dtype`` set starts a new tensor."""
    tensors: List[torch.Tensor] = []
    parts: List[runtime_pb2.Tensor] = []
    async for batch in stream:
        for chunk in batch:
            if chunk.dtype and parts:
                tensors.append(deserialize_torch_tensor(combine_from_streaming(parts)))
                parts = []
            parts.append(chunk)
    if parts:
        tensors.append(deserialize_torch_tensor(combine_from_streaming(parts)))
    return tensors


# ---------------------------------------------------------------------------------------------------------------
# Copy-light streaming of large tensors. A chunk message on the wire is ordinary protobuf (any peer can parse it
# with ``runtime_pb2``), but the sender never builds a protobuf object around the payload: the message is emitted as
# a short hand-encoded prefix followed by a ``memoryview`` into the tensor's own memory, and the receiver copies each
# chunk once, straight into the (optionally pinned) destination tensor.
# ---------------------------------------------------------------------------------------------------------------


def _varint(value: int) -> bytes:
    out = bytearray()
    while True:
        low = value & 0x7F
        value >>= 7
        if value:
            out.append(low | 0x80)
        else:
            out.append(low)
            return bytes(out)


class RawMessage:
    """A serialized protobuf message kept as a list of byte pieces; ``P2P.send_protobuf`` writes the pieces as is."""
    __slots__ = ("raw_parts",)

    def __init__(self, *parts):
        self.raw_parts = parts

    def ByteSize(self) -> int:
        return sum(len(p) for p in self.raw_parts)

    def SerializeToString(self) -> bytes:
        return b"".join(bytes(p) for p in self.raw_parts)


def _uncompressed_payload(tensor: torch.Tensor) -> Optional[memoryview]:
    """A byte view of a tensor that NoCompression would send verbatim, or None if it needs conversion."""
    if tensor.dtype == torch.bfloat16 or tensor.is_sparse:
        return None
    payload = tensor.detach()
    if payload.device.type != "cpu":
        payload = payload.cpu()
    if not payload.is_contiguous():
        payload = payload.contiguous()
    try:
        return memoryview(payload.numpy()).cast("B")
    except (TypeError, ValueError):
        return None


def stream_tensor_messages(tensor: torch.Tensor, compression_type: int, chunk_size_bytes: int, *,
                           outer_field: int = 2, outer_prefix: bytes = b"") -> Iterator[RawMessage]:
    """
    Serialized messages ``Outer{<outer_prefix fields>, tensors(field outer_field) = [chunk]}``, one per chunk of
    ``tensor``, equivalent to wrapping ``split_for_streaming(serialize_torch_tensor(tensor, ...))`` chunk by chunk
    (``ExpertRequest`` / ``ExpertResponse`` keep their tensors in field 2). Uncompressed CPU tensors are sent from
    their own memory; every other case serializes once and slices that buffer.
    """
    payload = _uncompressed_payload(tensor) if compression_type == CompressionType.NONE else None
    if payload is not None:
        header = runtime_pb2.Tensor(compression=CompressionType.NONE, size=tensor.shape,
                                    dtype=str(tensor.dtype).replace("torch.", ""), requires_grad=tensor.requires_grad)
    else:
        whole = serialize_torch_tensor(tensor, compression_type)
        payload = memoryview(whole.buffer)
        header = runtime_pb2.Tensor(compression=whole.compression, size=whole.size, dtype=whole.dtype,
                                    requires_grad=whole.requires_grad)
    total = len(payload)
    header.chunks = max(1, len(range(0, total, chunk_size_bytes)))
    outer_tag = _varint((outer_field << 3) | 2)
    first = True
    for start in range(0, max(total, 1), chunk_size_bytes):
        piece = payload[start:start + chunk_size_bytes]
        meta = header.SerializeToString() if first else b""
        first = False
        inner_prefix = meta + b"\x0a" + _varint(len(piece))  # Tensor.buffer is field 1, length-delimited
        inner_len = len(inner_prefix) + len(piece)
        yield RawMessage(outer_prefix + outer_tag + _varint(inner_len) + inner_prefix, piece)


def _direct_dtype(name: str):
    try:
        dtype = getattr(torch, name)
    except AttributeError:
        return None
    return dtype if isinstance(dtype, torch.dtype) and dtype != torch.bfloat16 else None


async def deserialize_tensor_stream_into(stream: AsyncIterator[Iterable[runtime_pb2.Tensor]], pin_memory: bool = False
                                         ) -> List[torch.Tensor]:
    """
    Like ``deserialize_tensor_stream``, but uncompressed tensors are assembled with one copy per chunk directly in
    their destination (page-locked when ``pin_memory``, so a later host-to-device copy needs no staging).
    """
    tensors: List[torch.Tensor] = []
    parts: List[runtime_pb2.Tensor] = []
    target = None  # (tensor, flat uint8 view, bytes filled) while a directly assembled tensor is in progress

    def finish():
        nonlocal parts, target
        if target is not None:
            tensor, _, filled = target
            if filled != tensor.numel() * tensor.element_size():
                raise ValueError("tensor stream ended before all bytes of a tensor arrived")
            tensors.append(tensor)
            target = None
        elif parts:
            tensors.append(deserialize_torch_tensor(combine_from_streaming(parts)))
            parts = []

    async for batch in stream:
        for chunk in batch:
            if chunk.dtype:
                finish()
                dtype = _direct_dtype(chunk.dtype) if chunk.compression == CompressionType.NONE else None
                if dtype is not None:
                    tensor = torch.empty(tuple(chunk.size), dtype=dtype, pin_memory=pin_memory)
                    if tensor.is_floating_point() and chunk.requires_grad:
                        tensor.requires_grad_(True)
                    flat = tensor.detach().view(-1).view(torch.uint8).numpy()
                    target = (tensor, flat, 0)
            if target is not None:
                tensor, flat, filled = target
                size = len(chunk.buffer)
                if filled + size > flat.shape[0]:
                    raise ValueError("tensor stream carries more bytes than the tensor's shape allows")
                flat[filled:filled + size] = memoryview(chunk.buffer)
                target = (tensor, flat, filled + size)
            else:
                parts.append(chunk)
    finish()
    return tensors


# ---------------------------------------------------------------------------------------------------------------
# Reading large tensors off the wire without parsing them: a received message is scanned once at field level, the
# tensor's ``buffer`` stays a view of the received bytes, and only the remaining (small) fields go through protobuf.
# The views quack like the generated messages for everything the codecs and the averaging code read from them.
# ---------------------------------------------------------------------------------------------------------------


def _read_varint(view: memoryview, offset: int) -> Tuple[int, int]:
    value = shift = 0
    while True:
        byte = view[offset]
        offset += 1
        value |= (byte & 0x7F) << shift
        if not byte & 0x80:
            return value, offset
        shift += 7
        if shift > 63:
            raise ValueError("malformed varint in a protobuf message")


def split_length_delimited_field(message: memoryview, field_number: int) -> Tuple[Optional[memoryview], bytes]:
    """Scan the top level of a serialized protobuf ``message``: returns a view of the (last) length-delimited value of
    ``field_number`` and the bytes of all other fields, which are a valid serialized message of the same type."""
    wanted, others, offset, end = None, [], 0, len(message)
    while offset < end:
        start = offset
        tag, offset = _read_varint(message, offset)
        number, wire_type = tag >> 3, tag & 7
        if wire_type == 0:
            _, offset = _read_varint(message, offset)
        elif wire_type == 1:
            offset += 8
        elif wire_type == 5:
            offset += 4
        elif wire_type == 2:
            length, offset = _read_varint(message, offset)
            if number == field_number:
                wanted = message[offset:offset + length]
                offset += length
                if offset > end:
                    raise ValueError("truncated protobuf message")
                continue
            offset += length
        else:
            raise ValueError(f"unsupported protobuf wire type {wire_type}")
        if offset > end:
            raise ValueError("truncated protobuf message")
        others.append(message[start:offset])
    return wanted, b"".join(others)


class TensorView:
    """A received ``runtime_pb2.Tensor`` whose ``buffer`` is a view of the bytes it arrived in."""

    __slots__ = ("buffer", "_meta")

    def __init__(self, serialized: memoryview):
        buffer, rest = split_length_delimited_field(serialized, 1)
        self.buffer = buffer if buffer is not None else memoryview(b"")
        self._meta = runtime_pb2.Tensor.FromString(rest)

    size = property(lambda self: self._meta.size)
    dtype = property(lambda self: self._meta.dtype)
    compression = property(lambda self: self._meta.compression)
    requires_grad = property(lambda self: self._meta.requires_grad)
    chunks = property(lambda self: self._meta.chunks)

    def to_message(self) -> runtime_pb2.Tensor:
        """An ordinary protobuf message with the same content (copies the buffer)."""
        message = runtime_pb2.Tensor()
        message.CopyFrom(self._meta)
        message.buffer = bytes(self.buffer)
        return message


# Codecs whose work on a part of a megabyte or so is a type conversion or less: cheaper to run where the data is than
# to hand to another thread (the quantising codecs sort, search or histogram and do belong in a thread).
_LIGHT_CODECS = (CompressionType.NONE, CompressionType.FLOAT16, CompressionType.MEANSTD_16BIT)
LIGHT_WORK_MAX_BYTES = 4 * 2 ** 20


def is_light_to_decode(serialized_tensor) -> bool:
    """Whether decoding this message is too little work to be worth a trip through a thread pool."""
    return serialized_tensor.compression in _LIGHT_CODECS and len(serialized_tensor.buffer) <= LIGHT_WORK_MAX_BYTES


def is_light_to_encode(tensor: torch.Tensor, compression_type: int) -> bool:
    """The same question before encoding ``tensor`` with the codec of this wire type."""
    return (compression_type in _LIGHT_CODECS and not tensor.is_cuda
            and tensor.numel() * tensor.element_size() <= LIGHT_WORK_MAX_BYTES)

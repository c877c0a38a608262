"""Tensor <-> protobuf helpers and chunked streaming (hivemind/compression/serialization.py:13-68,
hivemind/utils/streaming.py:14-46)."""
from __future__ import annotations

from typing import AsyncIterator, Dict, Iterable, Iterator, List, Optional

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

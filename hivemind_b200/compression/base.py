"""Codec interface, tensor roles and the identity codec.

Wire contract (hivemind/compression/base.py:17-122, hivemind/proto/runtime.proto:23-39): a compressed tensor is a
``runtime_pb2.Tensor`` with ``buffer``, ``size``, ``dtype`` (torch dtype name), ``requires_grad`` and the
``compression`` enum that tells the receiver which codec to run. bfloat16 tensors are sent as fp32 unless
``USE_LEGACY_BFLOAT16=0``.
"""
from __future__ import annotations

import dataclasses
import os
from abc import ABC, abstractmethod
from enum import Enum, auto
from typing import Any, Optional

import numpy as np
import torch

from hivemind_b200.proto import runtime_pb2
from hivemind_b200.utils.tensor_descr import TensorDescriptor

USE_LEGACY_BFLOAT16 = bool(int(os.environ.get("USE_LEGACY_BFLOAT16", 1)))
Key = Any


class TensorRole(Enum):
    ACTIVATION = auto()
    PARAMETER = auto()
    GRADIENT = auto()
    OPTIMIZER = auto()
    UNSPECIFIED = auto()


@dataclasses.dataclass(frozen=True)
class CompressionInfo:
    """What a codec may know about the tensor it is given (which may be one part of a larger tensor)."""

    key: Key  # name or index among parameters / optimizer state / expert inputs
    descriptor: TensorDescriptor  # describes the WHOLE tensor even when a part is being compressed
    role: TensorRole = TensorRole.UNSPECIFIED
    part_index: int = 0
    part_size: Optional[int] = None  # maximum number of values per part, if the tensor is split

    @classmethod
    def from_tensor(cls, tensor: torch.Tensor, key: Key = None, descriptor: TensorDescriptor = None, **kwargs):
        return cls(key, descriptor or TensorDescriptor.from_tensor(tensor), **kwargs)

    def get_part(self, part_index: int, part_size: Optional[int]) -> "CompressionInfo":
        return CompressionInfo(self.key, self.descriptor, self.role, part_index=part_index, part_size=part_size)


class CompressionBase(ABC):
    compression_type: int

    @abstractmethod
    def compress(self, tensor: torch.Tensor, info: CompressionInfo, allow_inplace: bool = False) -> runtime_pb2.Tensor:
        """Encode ``tensor`` (CPU or CUDA); ``allow_inplace`` lets the codec scribble over the input."""

    @abstractmethod
    def extract(self, serialized_tensor: runtime_pb2.Tensor) -> torch.Tensor:
        """Decode a message produced by ``compress`` into a CPU tensor of the original dtype and shape."""

    @abstractmethod
    def estimate_compression_ratio(self, info: CompressionInfo) -> float:
        """Compressed size / original size; used to size all-reduce parts."""

    def __repr__(self) -> str:
        return f"hivemind_b200.{self.__class__.__name__}()"


def dtype_name(tensor: torch.Tensor) -> str:
    return str(tensor.dtype).replace("torch.", "")


def as_cpu_bytes(tensor: torch.Tensor) -> bytes:
    """Raw bytes of a contiguous tensor (bf16 goes through an int16 view; CUDA tensors are copied to the host)."""
    tensor = tensor.detach().contiguous()
    if tensor.is_cuda:
        tensor = tensor.cpu()
    if tensor.dtype == torch.bfloat16:
        tensor = tensor.view(torch.int16)
    return tensor.numpy().tobytes()


class NoCompression(CompressionBase):
    """Sends the raw bytes."""

    compression_type = runtime_pb2.CompressionType.NONE

    def compress(self, tensor: torch.Tensor, info: CompressionInfo, allow_inplace: bool = False) -> runtime_pb2.Tensor:
        payload = tensor.detach()
        if payload.dtype == torch.bfloat16 and USE_LEGACY_BFLOAT16:
            payload = payload.to(torch.float32)
        return runtime_pb2.Tensor(compression=self.compression_type, buffer=as_cpu_bytes(payload), size=tensor.shape,
                                  dtype=dtype_name(tensor), requires_grad=tensor.requires_grad)

    def extract(self, serialized_tensor: runtime_pb2.Tensor) -> torch.Tensor:
        shape = torch.Size(serialized_tensor.size)
        raw = bytearray(serialized_tensor.buffer)
        if serialized_tensor.dtype == "bfloat16":
            numel = shape.numel()
            if numel > 0 and len(raw) // numel == 4:  # legacy senders ship bf16 as fp32
                tensor = torch.as_tensor(np.frombuffer(raw, dtype=np.float32), dtype=torch.bfloat16)
            else:
                tensor = torch.as_tensor(np.frombuffer(raw, dtype=np.int16)).view(torch.bfloat16)
        else:
            tensor = torch.as_tensor(np.frombuffer(raw, dtype=np.dtype(serialized_tensor.dtype)))
        return tensor.reshape(shape).requires_grad_(serialized_tensor.requires_grad) \
            if tensor.is_floating_point() else tensor.reshape(shape)

    def estimate_compression_ratio(self, info: CompressionInfo) -> float:
        return 1.0

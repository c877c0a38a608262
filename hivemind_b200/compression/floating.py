"""16-bit codecs: plain fp16 and mean/std-normalised fp16.

Math per hivemind/compression/floating.py:10-91: values are clamped to the fp16 range before the cast; the scaled
variant first subtracts the mean over the last axis and divides by the (biased) standard deviation, and appends the
fp32 means and stds to the fp16 payload. CUDA tensors are encoded by the kernels of ``ops/csrc/codec.cu``.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from hivemind_b200.compression.base import CompressionBase, CompressionInfo, as_cpu_bytes, dtype_name
from hivemind_b200.proto import runtime_pb2

FP16_MIN, FP16_MAX = torch.finfo(torch.float16).min, torch.finfo(torch.float16).max
FP32_EPS = torch.finfo(torch.float32).eps


def _half_from_bytes(raw) -> torch.Tensor:
    """The fp16 tensor that these bytes spell. The copy gives torch memory that it may write to (received bytes are
    read-only); the widening to fp32 is then torch's, which is some twenty times faster than numpy's."""
    if len(raw) == 0:
        return torch.empty(0, dtype=torch.float16)
    return torch.frombuffer(bytearray(raw), dtype=torch.float16)


class Float16Compression(CompressionBase):
    compression_type = runtime_pb2.CompressionType.FLOAT16

    def compress(self, tensor: torch.Tensor, info: CompressionInfo, allow_inplace: bool = False) -> runtime_pb2.Tensor:
        if not tensor.is_floating_point():
            raise ValueError(f"{type(self).__name__} does not support {tensor.dtype} tensors")
        source = tensor.detach()
        if source.is_cuda:
            from hivemind_b200.ops import codec as device_codec

            half = device_codec.encode_float16(source)
        else:
            work = source.to(torch.float32, copy=not allow_inplace)
            half = work.clamp_(FP16_MIN, FP16_MAX).to(torch.float16)
        return runtime_pb2.Tensor(compression=self.compression_type, buffer=as_cpu_bytes(half), size=tensor.shape,
                                  dtype=dtype_name(tensor), requires_grad=tensor.requires_grad)

    def extract(self, serialized_tensor: runtime_pb2.Tensor) -> torch.Tensor:
        out = _half_from_bytes(serialized_tensor.buffer).to(getattr(torch, serialized_tensor.dtype))
        return out.reshape(tuple(serialized_tensor.size)).requires_grad_(serialized_tensor.requires_grad)

    def estimate_compression_ratio(self, info: CompressionInfo) -> float:
        return 16.0 / torch.finfo(info.descriptor.dtype).bits


class ScaledFloat16Compression(Float16Compression):
    """fp16 after per-row (last axis) standardisation; robust to tensors whose scale is far from 1."""

    compression_type = runtime_pb2.CompressionType.MEANSTD_16BIT

    def compress(self, tensor: torch.Tensor, info: CompressionInfo, allow_inplace: bool = False) -> runtime_pb2.Tensor:
        if not tensor.is_floating_point():
            raise ValueError(f"{type(self).__name__} does not support {tensor.dtype} tensors")
        source = tensor.detach()
        if source.is_cuda and source.numel() > 0:
            from hivemind_b200.ops import codec as device_codec

            half, means, stds = device_codec.encode_scaled_float16(source)
        else:
            work = source.to(torch.float32, copy=not allow_inplace)
            means = torch.mean(work, dim=-1, keepdim=True)
            work.sub_(means)
            stds = work.norm(dim=-1, keepdim=True) / math.sqrt(work.shape[-1] if work.dim() else 1)
            stds.clamp_min_(FP32_EPS)
            work.div_(stds)
            half = work.clamp_(FP16_MIN, FP16_MAX).to(torch.float16)
        payload = b"".join((as_cpu_bytes(half), as_cpu_bytes(means.to(torch.float32)), as_cpu_bytes(stds.to(torch.float32))))
        return runtime_pb2.Tensor(compression=self.compression_type, buffer=payload, size=tensor.shape,
                                  dtype=dtype_name(tensor), requires_grad=tensor.requires_grad)

    def extract(self, serialized_tensor: runtime_pb2.Tensor) -> torch.Tensor:
        shape = tuple(serialized_tensor.size)
        stats_shape = (*shape[:-1], 1) if shape else ()
        stats_count = int(np.prod(stats_shape)) if shape else 1
        buf = serialized_tensor.buffer
        means = torch.as_tensor(np.frombuffer(buf[-8 * stats_count:-4 * stats_count], dtype=np.float32).copy()).reshape(stats_shape)
        stds = torch.as_tensor(np.frombuffer(buf[-4 * stats_count:], dtype=np.float32).copy()).reshape(stats_shape)
        out = _half_from_bytes(buf[:-8 * stats_count]).to(torch.float32).reshape(shape).mul_(stds).add_(means)
        return out.to(getattr(torch, serialized_tensor.dtype)).requires_grad_(serialized_tensor.requires_grad)


def get_num_bits(dtype: torch.dtype) -> int:
    """Storage bits of one element of ``dtype`` (reference: hivemind/compression/floating.py:94-104)."""
    if dtype == torch.bool:
        return 8  # a bool tensor spends a whole byte per element
    info = torch.finfo(dtype) if dtype.is_floating_point else None
    if info is not None:
        return info.bits
    try:
        return torch.iinfo(dtype).bits
    except TypeError:
        raise TypeError(f"cannot tell the width of {dtype}") from None

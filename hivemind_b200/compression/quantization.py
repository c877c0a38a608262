"""8-bit codecs: uniform, quantile and block-wise quantization with a transmitted codebook.

Math per hivemind/compression/quantization.py:20-201 (wire: int64 codebook length, fp32 codebook, uint8 indices;
block-wise: int64 absmax count, int64 code length, fp32 absmax per 4096 values, fp32 code, uint8 indices).
The reference delegates block-wise quantization to bitsandbytes; here the 256-entry signed "dynamic" code
(7 exponent levels, linear fractions, plus 0 and 1) is generated locally and the nearest code is found by search,
so the format stays decodable by any receiver because the code travels with the data. CUDA tensors are encoded by
``ops/csrc/codec.cu``.
"""
from __future__ import annotations

import math
import os
from abc import ABC, abstractmethod
from concurrent.futures import ThreadPoolExecutor
from functools import lru_cache
from typing import Tuple

import numpy as np
import torch

from hivemind_b200.compression.base import CompressionBase, CompressionInfo, as_cpu_bytes, dtype_name
from hivemind_b200.proto import runtime_pb2

EXECUTOR = ThreadPoolExecutor(max_workers=int(os.environ.get("QUANTIZATION_THREADS", 128)))
BLOCKSIZE = 4096


def average_buckets(values: torch.Tensor, indices: torch.Tensor, n_bins: int) -> torch.Tensor:
    """Mean of the values that fell into each bin (0 for empty bins)."""
    flat_idx = indices.reshape(-1).long()
    sums = torch.zeros(n_bins, dtype=torch.float32, device=values.device).scatter_add_(0, flat_idx, values.reshape(-1))
    counts = torch.bincount(flat_idx, minlength=n_bins).clamp_min_(1)
    return sums / counts


class Quantization(CompressionBase, ABC):
    codebook_dtype, indices_dtype = np.float32, np.uint8

    @abstractmethod
    def quantize(self, tensor: torch.Tensor, allow_inplace: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
        """Return (uint8 indices shaped like the tensor, fp32 codebook)."""

    def compress(self, tensor: torch.Tensor, info: CompressionInfo, allow_inplace: bool = False) -> runtime_pb2.Tensor:
        if not tensor.is_floating_point():
            raise ValueError(f"{type(self).__name__} does not support {tensor.dtype} tensors")
        indices, codebook = self.quantize(tensor.detach(), allow_inplace=allow_inplace)
        payload = b"".join((np.int64(codebook.numel()).tobytes(), as_cpu_bytes(codebook.to(torch.float32)),
                            as_cpu_bytes(indices.to(torch.uint8))))
        return runtime_pb2.Tensor(compression=self.compression_type, buffer=payload, size=tensor.shape,
                                  dtype=dtype_name(tensor), requires_grad=tensor.requires_grad)

    def extract(self, serialized_tensor: runtime_pb2.Tensor) -> torch.Tensor:
        buf = serialized_tensor.buffer
        n_codes = int(np.frombuffer(buf, count=1, dtype=np.int64)[0])
        codebook = torch.as_tensor(np.frombuffer(buf, offset=8, count=n_codes, dtype=self.codebook_dtype).copy())
        indices = torch.as_tensor(np.frombuffer(buf, offset=8 + 4 * n_codes, dtype=self.indices_dtype).copy())
        # a gather through 32-bit indices: about three times faster than fancy indexing with 64-bit ones
        out = codebook.to(getattr(torch, serialized_tensor.dtype)).index_select(0, indices.to(torch.int32))
        return out.reshape(tuple(serialized_tensor.size)).requires_grad_(serialized_tensor.requires_grad)

    def estimate_compression_ratio(self, info: CompressionInfo) -> float:
        return self.n_bits / torch.finfo(info.descriptor.dtype).bits

    @property
    def n_bits(self) -> int:
        return self.indices_dtype(1).itemsize * 8

    @property
    def n_bins(self) -> int:
        return 2 ** self.n_bits


class Uniform8BitQuantization(Quantization):
    """256 equal bins covering +-3 sigma around the mean; each bin decodes to the mean of its members."""

    RANGE_IN_SIGMAS: int = 6
    compression_type = runtime_pb2.UNIFORM_8BIT

    def quantize(self, tensor: torch.Tensor, allow_inplace: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
        if tensor.is_cuda and tensor.numel() > 1:
            from hivemind_b200.ops import codec as device_codec

            return device_codec.encode_uniform8(tensor)
        values = tensor.to(torch.float32)
        centered = values - values.mean()
        std_unbiased = centered.norm() / math.sqrt(max(centered.numel() - 1, 1))
        scale = float(self.RANGE_IN_SIGMAS * std_unbiased / self.n_bins)
        if not math.isfinite(scale) or scale <= 0:
            scale = 1.0
        indices = torch.clamp(torch.round(centered / scale) + self.n_bins // 2, 0, self.n_bins - 1).to(torch.uint8)
        return indices, average_buckets(values, indices, self.n_bins)


def get_chunk_size(num_elements: int, min_chunk_size: int) -> int:
    """A chunk size of at least ``min_chunk_size`` that splits ``num_elements`` as evenly as possible."""
    if min_chunk_size >= num_elements:
        return min_chunk_size
    num_chunks = num_elements // min_chunk_size
    leftover = num_elements % min_chunk_size
    return min_chunk_size + (leftover - 1) // num_chunks + 1


def _linear_quantiles(values: np.ndarray, points: np.ndarray, out: np.ndarray) -> None:
    """``np.quantile(values, points, out=out)`` (linear interpolation between order statistics) by way of one full
    sort, which for a few hundred quantiles of 10**5 values is an order of magnitude faster than numpy's selection."""
    ordered = np.sort(values)
    position = points.astype(np.float64) * (len(ordered) - 1)
    below = np.floor(position).astype(np.int64)
    above = np.minimum(below + 1, len(ordered) - 1)
    low, high = ordered[below].astype(np.float64), ordered[above].astype(np.float64)
    out[:] = low + (high - low) * (position - below)


def quantile_qq_approximation(array: np.ndarray, n_quantiles: int, min_chunk_size: int = 10 ** 5) -> np.ndarray:
    """Approximate uniform quantiles: exact quantiles of chunks (in a thread pool), then quantiles of those."""
    flat = np.ascontiguousarray(array.T if (not array.data.c_contiguous and array.data.f_contiguous) else array).reshape(-1)
    points = np.linspace(0.0, 1.0, num=n_quantiles, dtype=flat.dtype)
    chunk_size = get_chunk_size(len(flat), min_chunk_size)
    num_chunks = (len(flat) - 1) // chunk_size + 1
    table = np.empty((num_chunks, n_quantiles), dtype=flat.dtype)
    jobs = [EXECUTOR.submit(_linear_quantiles, flat[i * chunk_size:(i + 1) * chunk_size], points, table[i])
            for i in range(num_chunks)]
    for job in jobs:
        job.result()
    return np.quantile(table, points)


class Quantile8BitQuantization(Quantization):
    """256 bins holding (approximately) equal numbers of values; each decodes to the mean of its members."""

    compression_type = runtime_pb2.QUANTILE_8BIT

    def quantize(self, tensor: torch.Tensor, allow_inplace: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
        if tensor.is_cuda and tensor.numel() > 1:
            from hivemind_b200.ops import codec as device_codec

            return device_codec.encode_quantile8(tensor)
        values = tensor.detach().to(torch.float32)
        borders = torch.as_tensor(quantile_qq_approximation(values.numpy(), self.n_bins + 1)[1:-1])
        indices = torch.bucketize(values, borders).clamp_(0, self.n_bins - 1)
        return indices.to(torch.uint8), average_buckets(values, indices, self.n_bins)


@lru_cache(maxsize=None)
def dynamic_code_table(signed: bool = True, max_exponent_bits: int = 7, total_bits: int = 8) -> torch.Tensor:
    """The sorted 2**total_bits entry "dynamic" code: for each decade 10**-(E-1)..10**0, fractions spaced linearly
    in [0.1, 1] (twice as many per decade as in the previous one), both signs, plus exact 0 and 1."""
    non_sign_bits = total_bits - 1
    entries = []
    for i in range(max_exponent_bits):
        count = int(2 ** (i + non_sign_bits - max_exponent_bits)) + 1 if signed else int(2 ** (i + non_sign_bits - max_exponent_bits + 1)) + 1
        edges = torch.linspace(0.1, 1.0, count, dtype=torch.float64)
        means = (edges[:-1] + edges[1:]) / 2.0
        scale = 10.0 ** (-(max_exponent_bits - 1) + i)
        entries += (scale * means).tolist()
        if signed:
            entries += (-scale * means).tolist()
    entries += [0.0, 1.0]
    entries += [0.0] * (2 ** total_bits - len(entries))
    return torch.tensor(sorted(entries), dtype=torch.float32)


def quantize_blockwise_reference(values: torch.Tensor, code: torch.Tensor, blocksize: int = BLOCKSIZE
                                 ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per block of ``blocksize`` values: absmax, then the index of the code entry nearest to value / absmax."""
    flat = values.reshape(-1).to(torch.float32)
    n = flat.numel()
    n_blocks = (n + blocksize - 1) // blocksize
    padded = torch.zeros(n_blocks * blocksize, dtype=torch.float32, device=flat.device)
    padded[:n] = flat
    blocks = padded.view(n_blocks, blocksize)
    absmax = blocks.abs().amax(dim=1)
    normed = blocks / absmax.clamp_min(torch.finfo(torch.float32).tiny).unsqueeze(1)
    code = code.to(flat.device)
    midpoints = (code[1:] + code[:-1]) / 2
    indices = torch.bucketize(normed.reshape(-1), midpoints)[:n].to(torch.uint8)
    return indices.view(values.shape), absmax


def dequantize_blockwise_reference(indices: torch.Tensor, absmax: torch.Tensor, code: torch.Tensor,
                                   blocksize: int = BLOCKSIZE) -> torch.Tensor:
    flat = code.to(indices.device)[indices.reshape(-1).long()]
    block_of = torch.arange(flat.numel(), device=flat.device) // blocksize
    return (flat * absmax.to(flat.device)[block_of]).view(indices.shape)


class BlockwiseQuantization(Quantization):
    """8-bit dynamic-code quantization with one absmax scale per 4096 values."""

    compression_type = runtime_pb2.BLOCKWISE_8BIT

    def quantize(self, tensor: torch.Tensor, allow_inplace: bool = False
                 ) -> Tuple[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
        code = dynamic_code_table()
        if tensor.is_cuda and tensor.numel() > 0:
            from hivemind_b200.ops import codec as device_codec

            indices, absmax = device_codec.encode_blockwise8(tensor, code)
        else:
            indices, absmax = quantize_blockwise_reference(tensor.to(torch.float32), code)
        return indices, (absmax, code)

    def compress(self, tensor: torch.Tensor, info: CompressionInfo, allow_inplace: bool = False) -> runtime_pb2.Tensor:
        if not tensor.is_floating_point():
            raise ValueError(f"{type(self).__name__} does not support {tensor.dtype} tensors")
        indices, (absmax, code) = self.quantize(tensor.detach(), allow_inplace=allow_inplace)
        payload = b"".join((np.int64(absmax.numel()).tobytes(), np.int64(code.numel()).tobytes(), as_cpu_bytes(absmax),
                            as_cpu_bytes(code), as_cpu_bytes(indices)))
        return runtime_pb2.Tensor(buffer=payload, size=tensor.shape, requires_grad=tensor.requires_grad,
                                  dtype=dtype_name(tensor), compression=self.compression_type)

    def extract(self, serialized_tensor: runtime_pb2.Tensor) -> torch.Tensor:
        buf = serialized_tensor.buffer
        n_absmax, n_code = (int(v) for v in np.frombuffer(buf, count=2, dtype=np.int64))
        absmax = torch.as_tensor(np.frombuffer(buf, offset=16, count=n_absmax, dtype=np.float32).copy())
        code = torch.as_tensor(np.frombuffer(buf, offset=16 + 4 * n_absmax, count=n_code, dtype=np.float32).copy())
        indices = torch.as_tensor(np.frombuffer(buf, offset=16 + 4 * (n_absmax + n_code), dtype=np.uint8).copy())
        out = dequantize_blockwise_reference(indices.reshape(tuple(serialized_tensor.size)), absmax, code)
        return out.to(getattr(torch, serialized_tensor.dtype)).requires_grad_(serialized_tensor.requires_grad)

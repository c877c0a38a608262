"""Codecs that delegate to another codec chosen per tensor — by element count, by role, or by key.

Public classes and their constructor arguments follow hivemind/compression/adaptive.py:25-66. A delegating codec
never appears on the wire: the message carries the type of the codec that was chosen, so ``extract`` is simply the
registry lookup of ``deserialize_torch_tensor``.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional, Sequence, Union

import torch

from hivemind_b200.compression.base import CompressionBase, CompressionInfo, Key, NoCompression, TensorRole
from hivemind_b200.proto import runtime_pb2


class AdaptiveCompressionBase(CompressionBase):
    """Subclasses implement ``choose_compression(info)``; everything else is forwarded to the chosen codec."""

    def choose_compression(self, info: CompressionInfo) -> CompressionBase:
        raise NotImplementedError

    def compress(self, tensor: torch.Tensor, info: CompressionInfo, allow_inplace: bool = False) -> runtime_pb2.Tensor:
        chosen = self.choose_compression(info)
        return chosen.compress(tensor, info=info, allow_inplace=allow_inplace)

    def estimate_compression_ratio(self, info: CompressionInfo) -> float:
        chosen = self.choose_compression(info)
        return chosen.estimate_compression_ratio(info)

    def extract(self, serialized_tensor: runtime_pb2.Tensor) -> torch.Tensor:
        from hivemind_b200.compression.serialization import deserialize_torch_tensor  # late: avoids an import cycle

        return deserialize_torch_tensor(serialized_tensor)


class SizeAdaptiveCompression(AdaptiveCompressionBase):
    """Small tensors (fewer than ``threshold`` elements) go through ``less``, the others through ``greater_equal``."""

    def __init__(self, threshold: int, less: CompressionBase, greater_equal: CompressionBase):
        self.threshold = threshold
        self.less = less
        self.greater_equal = greater_equal

    def choose_compression(self, info: CompressionInfo) -> CompressionBase:
        is_small = info.descriptor.numel() < self.threshold
        return self.less if is_small else self.greater_equal


class RoleAdaptiveCompression(AdaptiveCompressionBase):
    """A codec per ``TensorRole``; roles that are not given use ``default``."""

    def __init__(self, *, activation: Optional[CompressionBase] = None, parameter: Optional[CompressionBase] = None,
                 gradient: Optional[CompressionBase] = None, optimizer: Optional[CompressionBase] = None,
                 default: CompressionBase = NoCompression()):
        given = {TensorRole.ACTIVATION: activation, TensorRole.PARAMETER: parameter, TensorRole.GRADIENT: gradient,
                 TensorRole.OPTIMIZER: optimizer, TensorRole.UNSPECIFIED: None}
        self.role_compressions: Dict[TensorRole, CompressionBase] = {
            role: (codec if codec is not None else default) for role, codec in given.items()}

    def choose_compression(self, info: CompressionInfo) -> CompressionBase:
        return self.role_compressions[info.role]


class PerTensorCompression(AdaptiveCompressionBase):
    """An explicit codec for every tensor key: a mapping, or a sequence when keys are positions."""

    def __init__(self, tensor_compressions: Union[Sequence[CompressionBase], Mapping[Key, CompressionBase]]):
        self.tensor_compressions = tensor_compressions

    def choose_compression(self, info: CompressionInfo) -> CompressionBase:
        return self.tensor_compressions[info.key]

"""Tensor descriptors: shape/dtype/device records that describe expert inputs and averaged tensors.

``BatchTensorDescriptor`` is msgpack-serializable (ext 0x51) because expert schemas travel in ``rpc_info`` replies
(reference: hivemind/utils/tensor_descr.py:13-127, hivemind/moe/server/module_backend.py:190-196).
"""
from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Tuple

import numpy as np
import torch

from hivemind_b200.utils.serializer import MSGPackSerializer

DUMMY_BATCH_SIZE = 3  # batch used to trace output shapes of an expert
_warn_pinned = True


class DescriptorBase:
    pass


@dataclass(init=True, repr=True, frozen=True)
class TensorDescriptor(DescriptorBase):
    size: tuple
    dtype: torch.dtype = None
    layout: torch.layout = torch.strided
    device: torch.device = None
    requires_grad: bool = False
    pin_memory: bool = False
    compression: int = 0  # CompressionType.NONE

    @property
    def shape(self) -> Tuple[int, ...]:
        return self.size

    def numel(self) -> int:
        return int(np.prod(self.size))

    @classmethod
    def from_tensor(cls, tensor: torch.Tensor) -> "TensorDescriptor":
        return cls(tuple(tensor.shape), tensor.dtype, tensor.layout, tensor.device, tensor.requires_grad,
                   _safe_check_pinned(tensor))

    def make_zeros(self, **kwargs) -> torch.Tensor:
        kwargs = {**dict(dtype=self.dtype, layout=self.layout, device=self.device, requires_grad=self.requires_grad,
                         pin_memory=self.pin_memory), **kwargs}
        return torch.zeros(self.size, **kwargs)


def _str_to_torch_type(name: str, torch_type: type):
    try:
        value = getattr(torch, name.split(".")[-1])
    except AttributeError:
        raise ValueError(f"invalid dtype: {name}")
    if not isinstance(value, torch_type):
        raise ValueError(f"invalid dtype: expected {torch_type}, got {type(value)}")
    return value


@MSGPackSerializer.ext_serializable(0x51)
@dataclass(repr=True, frozen=True)
class BatchTensorDescriptor(TensorDescriptor):
    """Descriptor of a tensor whose first dimension is a variable batch size."""

    def __init__(self, *instance_size, **kwargs):
        if len(instance_size) == 1 and isinstance(instance_size[0], (list, tuple, torch.Size)):
            instance_size = instance_size[0]
        super().__init__((None, *instance_size), **kwargs)

    @classmethod
    def from_tensor(cls, tensor: torch.Tensor, compression: int = 0) -> "BatchTensorDescriptor":
        return cls(*tensor.shape[1:], dtype=tensor.dtype, layout=tensor.layout, device=tensor.device,
                   requires_grad=tensor.requires_grad, pin_memory=_safe_check_pinned(tensor),
                   compression=compression if tensor.is_floating_point() else 0)

    def make_zeros(self, *batch_size: int, **kwargs) -> torch.Tensor:
        assert self.size[0] is None, "the first dimension must be the (unset) batch dimension"
        kwargs = {**dict(dtype=self.dtype, layout=self.layout, device=self.device, requires_grad=self.requires_grad,
                         pin_memory=self.pin_memory), **kwargs}
        return torch.zeros((*batch_size, *self.size[1:]), **kwargs)

    def packb(self) -> bytes:
        obj = asdict(self)
        obj["dtype"] = str(self.dtype) if self.dtype is not None else None
        obj["layout"] = str(self.layout) if self.layout is not None else None
        device = obj.pop("device")
        obj["device_type"] = device.type if device is not None else None
        obj["device_index"] = device.index if device is not None else None
        return MSGPackSerializer.dumps(obj)

    @classmethod
    def unpackb(cls, raw: bytes) -> "BatchTensorDescriptor":
        obj = MSGPackSerializer.loads(raw)
        if obj["dtype"] is not None:
            obj["dtype"] = _str_to_torch_type(obj["dtype"], torch.dtype)
        if obj["layout"] is not None:
            obj["layout"] = _str_to_torch_type(obj["layout"], torch.layout)
        device_type, device_index = obj.pop("device_type"), obj.pop("device_index")
        obj["device"] = torch.device(device_type, device_index) if device_type is not None else None
        size = obj.pop("size")[1:]
        return cls(*size, **obj)


def _safe_check_pinned(tensor: torch.Tensor) -> bool:
    """``is_pinned`` raises on machines without CUDA; treat that as "not pinned"."""
    try:
        return torch.cuda.is_available() and tensor.is_pinned()
    except Exception:
        return False

"""MessagePack serialization with extension types (tuples keep their type; classes can register an ext code).

Wire contract shared with the reference (hivemind/utils/serializer.py:25-73): ext code 0x40 is a tuple;
``MSGPackSerializer.ext_serializable(code)`` registers a class that provides ``packb()`` / ``unpackb(bytes)``
(0x50 = dictionary DHT value, 0x51 = batch tensor descriptor).
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, Callable, Dict, Type

import msgpack


class SerializerBase(ABC):
    @staticmethod
    @abstractmethod
    def dumps(obj: object) -> bytes:
        ...

    @staticmethod
    @abstractmethod
    def loads(buf: bytes) -> object:
        ...


class MSGPackSerializer(SerializerBase):
    _ext_by_type: Dict[Type, int] = {}
    _ext_by_code: Dict[int, Type] = {}
    _TUPLE_EXT = 0x40

    @classmethod
    def ext_serializable(cls, type_code: int) -> Callable[[Type], Type]:
        assert isinstance(type_code, int) and 0 <= type_code < 128, "msgpack ext codes are 0..127"
        assert type_code != cls._TUPLE_EXT, "0x40 is reserved for tuples"

        def register(wrapped: Type) -> Type:
            assert callable(getattr(wrapped, "packb", None)) and callable(getattr(wrapped, "unpackb", None)), \
                "an ext-serializable class needs packb() and a classmethod unpackb(bytes)"
            if type_code in cls._ext_by_code and cls._ext_by_code[type_code].__name__ != wrapped.__name__:
                raise ValueError(f"ext code {type_code:#x} is already taken by {cls._ext_by_code[type_code]}")
            cls._ext_by_type[wrapped], cls._ext_by_code[type_code] = type_code, wrapped
            return wrapped

        return register

    @classmethod
    def _default(cls, obj: Any) -> Any:
        code = cls._ext_by_type.get(type(obj))
        if code is not None:
            return msgpack.ExtType(code, obj.packb())
        if isinstance(obj, tuple):
            return msgpack.ExtType(cls._TUPLE_EXT, msgpack.packb(list(obj), default=cls._default, strict_types=True,
                                                                 use_bin_type=True))
        raise TypeError(f"cannot serialize {type(obj)}")

    @classmethod
    def _ext_hook(cls, code: int, data: bytes) -> Any:
        if code == cls._TUPLE_EXT:
            return tuple(msgpack.unpackb(data, ext_hook=cls._ext_hook, raw=False, strict_map_key=False))
        target = cls._ext_by_code.get(code)
        if target is not None:
            return target.unpackb(data)
        return msgpack.ExtType(code, data)  # unknown ext: hand it back untouched

    @classmethod
    def dumps(cls, obj: object) -> bytes:
        return msgpack.packb(obj, default=cls._default, strict_types=True, use_bin_type=True)

    @classmethod
    def loads(cls, buf: bytes) -> object:
        return msgpack.unpackb(buf, ext_hook=cls._ext_hook, raw=False, strict_map_key=False)

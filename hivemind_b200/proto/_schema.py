"""Builds protobuf message classes at import time from declarative tables.

The reference compiles ``hivemind/proto/*.proto`` with ``grpc_tools.protoc`` during installation (setup.py:38-57).
Here the same schemas (same message names, field names, numbers and types, hence the same wire format) are declared
in Python and turned into classes through ``FileDescriptorProto`` + the protobuf runtime, so no compiler is needed.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple, Union

from google.protobuf import descriptor_pb2, descriptor_pool, message_factory

_F = descriptor_pb2.FieldDescriptorProto
_SCALARS = {
    "double": _F.TYPE_DOUBLE, "float": _F.TYPE_FLOAT, "int32": _F.TYPE_INT32, "int64": _F.TYPE_INT64,
    "uint32": _F.TYPE_UINT32, "uint64": _F.TYPE_UINT64, "bool": _F.TYPE_BOOL, "string": _F.TYPE_STRING,
    "bytes": _F.TYPE_BYTES,
}
_pool = descriptor_pool.Default()

# field spec: (name, number, type, label) with label in {"", "repeated", "required", "optional"}
FieldSpec = Tuple[str, int, str, str]


def build_file(name: str, *, package: str = "", syntax: str = "proto3", deps: Sequence[str] = (),
               enums: Optional[Dict[str, List[Tuple[str, int]]]] = None,
               messages: Optional[Dict[str, Union[List[FieldSpec], dict]]] = None) -> Dict[str, type]:
    """Register one schema file and return ``{message or enum name: class / enum wrapper}``."""
    enums, messages = enums or {}, messages or {}
    fdp = descriptor_pb2.FileDescriptorProto(name=name, package=package, syntax=syntax)
    fdp.dependency.extend(deps)
    prefix = f".{package}." if package else "."
    for enum_name, values in enums.items():
        e = fdp.enum_type.add(name=enum_name)
        for value_name, number in values:
            e.value.add(name=value_name, number=number)
    for msg_name, spec in messages.items():
        m = fdp.message_type.add(name=msg_name)
        # a message is a list of fields, or {"fields": [...], "enums": {name: values}, "oneofs": {name: [field names]}}
        fields, nested_enums, oneofs = (spec, {}, {}) if isinstance(spec, list) else (
            spec["fields"], spec.get("enums", {}), spec.get("oneofs", {}))
        for enum_name, values in nested_enums.items():
            e = m.enum_type.add(name=enum_name)
            for value_name, number in values:
                e.value.add(name=value_name, number=number)
        oneof_index = {}
        for index, (oneof_name, members) in enumerate(oneofs.items()):
            m.oneof_decl.add(name=oneof_name)
            oneof_index.update({member: index for member in members})
        for fname, number, ftype, label in fields:
            f = m.field.add(name=fname, number=number)
            f.label = {"repeated": _F.LABEL_REPEATED, "required": _F.LABEL_REQUIRED}.get(label, _F.LABEL_OPTIONAL)
            if fname in oneof_index:
                f.oneof_index = oneof_index[fname]
            if ftype in _SCALARS:
                f.type = _SCALARS[ftype]
            elif ftype in nested_enums:
                f.type = _F.TYPE_ENUM
                f.type_name = f"{prefix}{msg_name}.{ftype}"
            elif ftype in enums or ftype.startswith("enum:"):
                f.type = _F.TYPE_ENUM
                f.type_name = prefix + ftype.split(":")[-1] if ftype in enums else "." + ftype.split(":")[-1]
            else:  # message type, possibly from a dependency (given as a bare name in the default package)
                f.type = _F.TYPE_MESSAGE
                f.type_name = (prefix + ftype) if ftype in messages else "." + ftype
    try:
        file_desc = _pool.Add(fdp)
    except TypeError:
        file_desc = _pool.AddSerializedFile(fdp.SerializeToString())
    if file_desc is None:
        file_desc = _pool.FindFileByName(name)
    out: Dict[str, type] = {}
    for msg_name, spec in messages.items():
        descriptor = file_desc.message_types_by_name[msg_name]
        out[msg_name] = cls = message_factory.GetMessageClass(descriptor)
        if not isinstance(spec, list):  # generated code exposes nested enum values on the message class as well
            for enum_name in spec.get("enums", {}):
                nested = descriptor.enum_types_by_name[enum_name]
                if not hasattr(cls, enum_name):
                    setattr(cls, enum_name, _EnumWrapper(nested))
                for value in nested.values:
                    if not hasattr(cls, value.name):
                        setattr(cls, value.name, value.number)
    for enum_name in enums:
        out[enum_name] = _EnumWrapper(file_desc.enum_types_by_name[enum_name])
    return out


class _EnumWrapper:
    """Gives an enum descriptor the interface of generated code: ``E.NAME``, ``E.Name(n)``, ``E.Value(s)``."""

    def __init__(self, descriptor):
        self.DESCRIPTOR = descriptor
        for value in descriptor.values:
            setattr(self, value.name, value.number)

    def Name(self, number: int) -> str:
        return self.DESCRIPTOR.values_by_number[number].name

    def Value(self, name: str) -> int:
        return self.DESCRIPTOR.values_by_name[name].number

    def keys(self):
        return [v.name for v in self.DESCRIPTOR.values]

    def values(self):
        return [v.number for v in self.DESCRIPTOR.values]

    def items(self):
        return [(v.name, v.number) for v in self.DESCRIPTOR.values]

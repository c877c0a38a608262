"""Schema validation of DHT records with pydantic (reference: hivemind/dht/schema.py:15-179).

A schema is a ``pydantic.v1.BaseModel`` whose field names are DHT keys; each field's type describes the value (or,
for ``Dict[...]`` fields, the sub-key -> value mapping). Values are checked strictly (no coercion).
"""
from __future__ import annotations

import re
from typing import Any, Dict, Optional, Type

import pydantic.v1 as pydantic

from hivemind_b200.dht.crypto import RSASignatureValidator
from hivemind_b200.dht.routing import DHTID
from hivemind_b200.dht.validation import DHTRecord, RecordValidatorBase
from hivemind_b200.utils.logging import get_logger
from hivemind_b200.utils.serializer import MSGPackSerializer

logger = get_logger(__name__)


class SchemaValidator(RecordValidatorBase):
    def __init__(self, schema: Type[pydantic.BaseModel], allow_extra_keys: bool = True, prefix: Optional[str] = None):
        """
        :param schema: model whose fields are the (optionally prefixed) DHT keys to validate
        :param allow_extra_keys: accept keys that no schema mentions
        :param prefix: validates ``"{prefix}_{field}"`` keys instead of bare field names
        """
        self._patch_schema(schema)
        self._schemas = [schema]
        self._key_id_to_field_name: Dict[bytes, str] = {}
        for field in schema.__fields__.values():
            raw_key = f"{prefix}_{field.name}" if prefix is not None else field.name
            self._key_id_to_field_name[DHTID.generate(source=raw_key).to_bytes()] = field.name
        self._allow_extra_keys = allow_extra_keys

    @staticmethod
    def _patch_schema(schema: Type[pydantic.BaseModel]) -> None:
        # strict types: "1" is not an int, and so on
        config = schema.__config__
        config.extra = pydantic.Extra.forbid
        for field in schema.__fields__.values():
            field.required = False  # a record carries one key at a time

    def __setstate__(self, state: Dict[str, Any]) -> None:
        # model classes are pickled by reference: an interpreter that has just imported them has the unadjusted ones
        self.__dict__.update(state)
        for schema in self._schemas:
            self._patch_schema(schema)

    def validate(self, record: DHTRecord) -> bool:
        if record.key not in self._key_id_to_field_name:
            if not self._allow_extra_keys:
                logger.debug(f"record with key id {record.key!r} is not declared in any schema and extra keys are forbidden")
            return self._allow_extra_keys
        try:
            parsed = self._deserialize_record(record)
        except Exception as e:
            logger.debug(f"cannot deserialize {record}: {e!r}")
            return False
        field_name = self._key_id_to_field_name[record.key]
        errors = []
        for schema in self._schemas:
            if field_name not in schema.__fields__:
                continue
            try:
                self._strict_check(schema.__fields__[field_name], parsed[field_name])
                schema.parse_obj(parsed)
                return True
            except (pydantic.ValidationError, TypeError, ValueError) as e:
                errors.append(e)
        logger.debug(f"record {parsed} does not match any schema: {errors}")
        return False

    @staticmethod
    def _strict_check(field, value: Any) -> None:
        """Reject silent coercions that pydantic would perform (e.g. str -> int, float -> int)."""
        outer = field.outer_type_
        def check(tp, v):
            origin = getattr(tp, "__origin__", None)
            if tp in (int, float, str, bytes, bool):
                if tp is float and isinstance(v, int) and not isinstance(v, bool):
                    return
                if type(v) is not tp and not (tp is int and type(v) is int):
                    raise TypeError(f"expected {tp.__name__}, got {type(v).__name__}")
            elif origin in (dict, Dict):
                if not isinstance(v, dict):
                    raise TypeError("expected a dictionary")
                kt, vt = tp.__args__
                for k, item in v.items():
                    check(kt, k)
                    check(vt, item)
        check(outer, value)

    def _deserialize_record(self, record: DHTRecord) -> Dict[str, Any]:
        field_name = self._key_id_to_field_name[record.key]
        deserialized_value = MSGPackSerializer.loads(record.value)
        if record.subkey in (None, DHTProtocolMarkers.IS_DICTIONARY, DHTProtocolMarkers.IS_REGULAR_VALUE):
            return {field_name: deserialized_value}
        deserialized_subkey = MSGPackSerializer.loads(record.subkey)
        return {field_name: {deserialized_subkey: deserialized_value}}

    def merge_with(self, other: RecordValidatorBase) -> bool:
        if not isinstance(other, SchemaValidator):
            return False
        self._schemas.extend(other._schemas)
        self._key_id_to_field_name.update(other._key_id_to_field_name)
        self._allow_extra_keys = self._allow_extra_keys or other._allow_extra_keys
        return True

    @property
    def priority(self) -> int:
        return 0


class DHTProtocolMarkers:
    """Sub-key tags of records that are not dictionary entries (kept equal to DHTProtocol.RESERVED_SUBKEYS)."""

    IS_REGULAR_VALUE = MSGPackSerializer.dumps(None)
    IS_DICTIONARY = b""


def conbytes(*, regex: bytes = None, **kwargs) -> Type[pydantic.BaseModel]:
    """``pydantic.conbytes`` with an optional regular expression that the whole value must match."""
    compiled_regex = re.compile(regex) if regex is not None else None

    class ConstrainedBytesWithRegex(pydantic.conbytes(**kwargs)):
        @classmethod
        def __get_validators__(cls):
            yield from super().__get_validators__()
            yield cls.match_regex

        @classmethod
        def match_regex(cls, value: bytes) -> bytes:
            if compiled_regex is not None and compiled_regex.match(value) is None:
                raise ValueError(f"Value `{value}` doesn't match regex `{regex}`")
            return value

    return ConstrainedBytesWithRegex


BytesWithPublicKey = conbytes(regex=b".*" + RSASignatureValidator.PUBLIC_KEY_REGEX + b".*")

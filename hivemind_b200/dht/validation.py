"""Pluggable checks on DHT records.

A validator sees records in serialized form — ``DHTRecord(key id bytes, sub-key bytes, value bytes, expiration)`` —
in three places: before a node accepts a store, before a reader accepts a found value, and when the local node
prepares a value for storing (``sign_value``) or hands one to the application (``strip_value``).
Interface contract: hivemind/dht/validation.py:7-122.
"""
from __future__ import annotations

import dataclasses
from abc import ABC, abstractmethod
from typing import Iterable, List


@dataclasses.dataclass(frozen=True)
class DHTRecord:
    key: bytes
    subkey: bytes
    value: bytes
    expiration_time: float

    def with_value(self, value: bytes) -> "DHTRecord":
        return dataclasses.replace(self, value=value)


class RecordValidatorBase(ABC):
    @abstractmethod
    def validate(self, record: DHTRecord) -> bool:
        """Accept or reject ``record`` (its value is in the signed form produced by ``sign_value``)."""

    def sign_value(self, record: DHTRecord) -> bytes:
        """The bytes to put on the network for this record; the default adds nothing."""
        return record.value

    def strip_value(self, record: DHTRecord) -> bytes:
        """Undo ``sign_value``."""
        return record.value

    @property
    def priority(self) -> int:
        """Order among several validators: lower priorities sign first and are stripped last."""
        return 0

    def merge_with(self, other: "RecordValidatorBase") -> bool:
        """Absorb ``other`` if both can act as one validator; return False to keep them separate."""
        return False


class CompositeValidator(RecordValidatorBase):
    """A priority-ordered stack of validators that behaves like one."""

    def __init__(self, validators: Iterable[RecordValidatorBase] = ()):
        self._stack: List[RecordValidatorBase] = []
        self.extend(validators)

    def extend(self, validators: Iterable[RecordValidatorBase]) -> None:
        for candidate in validators:
            if not any(existing.merge_with(candidate) for existing in self._stack):
                self._stack.append(candidate)
        self._stack.sort(key=lambda validator: validator.priority)

    def validate(self, record: DHTRecord) -> bool:
        # outermost layer (highest priority) first; peel its decoration before asking the next layer
        remaining = len(self._stack)
        for validator in self._stack[::-1]:
            if not validator.validate(record):
                return False
            remaining -= 1
            if remaining:
                record = record.with_value(validator.strip_value(record))
        return True

    def sign_value(self, record: DHTRecord) -> bytes:
        for validator in self._stack:
            record = record.with_value(validator.sign_value(record))
        return record.value

    def strip_value(self, record: DHTRecord) -> bytes:
        for validator in self._stack[::-1]:
            record = record.with_value(validator.strip_value(record))
        return record.value

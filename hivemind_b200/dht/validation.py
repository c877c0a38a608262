"""Record validators: hooks that check, sign and strip DHT records (reference: hivemind/dht/validation.py:7-122)."""
from __future__ import annotations

import dataclasses
from abc import ABC, abstractmethod
from typing import Iterable, List


@dataclasses.dataclass(init=True, repr=True, frozen=True)
class DHTRecord:
    key: bytes
    subkey: bytes
    value: bytes
    expiration_time: float


class RecordValidatorBase(ABC):
    """Validators run on serialized records both when a node is asked to store and when a reader gets a value."""

    @abstractmethod
    def validate(self, record: DHTRecord) -> bool:
        """Is the record (with whatever ``sign_value`` appended) acceptable?"""

    def sign_value(self, record: DHTRecord) -> bytes:
        """Return the value to be stored, possibly with a signature appended."""
        return record.value

    def strip_value(self, record: DHTRecord) -> bytes:
        """Inverse of ``sign_value``: the value as the application wrote it."""
        return record.value

    @property
    def priority(self) -> int:
        """Validators with a higher priority sign last and strip first."""
        return 0

    def merge_with(self, other: "RecordValidatorBase") -> bool:
        """Try to absorb ``other`` (e.g. merge two schemas); False means both must be kept."""
        return False


class CompositeValidator(RecordValidatorBase):
    def __init__(self, validators: Iterable[RecordValidatorBase] = ()):
        self._validators: List[RecordValidatorBase] = []
        self.extend(validators)

    def extend(self, validators: Iterable[RecordValidatorBase]) -> None:
        for new in validators:
            for existing in self._validators:
                if existing.merge_with(new):
                    break
            else:
                self._validators.append(new)
        self._validators.sort(key=lambda v: v.priority)

    def validate(self, record: DHTRecord) -> bool:
        for i, validator in enumerate(reversed(self._validators)):
            if not validator.validate(record):
                return False
            if i < len(self._validators) - 1:
                record = dataclasses.replace(record, value=validator.strip_value(record))
        return True

    def sign_value(self, record: DHTRecord) -> bytes:
        for validator in self._validators:
            record = dataclasses.replace(record, value=validator.sign_value(record))
        return record.value

    def strip_value(self, record: DHTRecord) -> bytes:
        for validator in reversed(self._validators):
            record = dataclasses.replace(record, value=validator.strip_value(record))
        return record.value

"""Local key-value storage of a DHT node: regular values and dictionaries of sub-keys.

A key holds either one binary value or a ``DictionaryDHTValue`` (sub-key -> value, each with its own expiration),
msgpack ext 0x50 on the wire. A newer expiration wins per (key, sub-key) (reference: hivemind/dht/storage.py:11-69).
"""
from __future__ import annotations

from typing import Optional, Union

from hivemind_b200.dht.routing import BinaryDHTValue, DHTID, Subkey
from hivemind_b200.utils.serializer import MSGPackSerializer
from hivemind_b200.utils.timed_storage import DHTExpiration, KeyType, TimedStorage, ValueType


@MSGPackSerializer.ext_serializable(0x50)
class DictionaryDHTValue(TimedStorage[Subkey, BinaryDHTValue]):
    """A dictionary stored under one DHT key; tracks the latest expiration among its entries."""

    latest_expiration_time = float("-inf")

    def store(self, key: KeyType, value: ValueType, expiration_time: DHTExpiration) -> bool:
        self.latest_expiration_time = max(self.latest_expiration_time, expiration_time)
        return super().store(key, value, expiration_time)

    def packb(self) -> bytes:
        """Serialize with expiry frozen so that the packed form is what a reader would have seen now."""
        packed_items = [[key, value, expiration_time] for key, (value, expiration_time) in self.items()]
        return MSGPackSerializer.dumps([self.maxsize, self.latest_expiration_time, packed_items])

    @classmethod
    def unpackb(cls, raw: bytes) -> "DictionaryDHTValue":
        maxsize, latest_expiration_time, items = MSGPackSerializer.loads(raw)
        with DictionaryDHTValue(maxsize).freeze() as new_dict:
            for key, value, expiration_time in items:
                new_dict.store(key, value, expiration_time)
            new_dict.latest_expiration_time = latest_expiration_time
            return new_dict


class DHTLocalStorage(TimedStorage[DHTID, Union[BinaryDHTValue, DictionaryDHTValue]]):
    def store(self, key: DHTID, value: BinaryDHTValue, expiration_time: DHTExpiration,
              subkey: Optional[Subkey] = None) -> bool:
        """Store a regular value, or (with ``subkey``) one entry of the dictionary under ``key``."""
        if subkey is not None:
            return self.store_subkey(key, subkey, value, expiration_time)
        return super().store(key, value, expiration_time)

    def store_subkey(self, key: DHTID, subkey: Subkey, value: BinaryDHTValue, expiration_time: DHTExpiration) -> bool:
        """
        - no value or a regular value under ``key``: it is replaced by a dictionary if the new expiration is later;
        - a dictionary under ``key``: the entry is added / refreshed if it is newer than the same sub-key's entry.
        """
        previous_value, previous_expiration_time = self.get(key) or (b"", -float("inf"))
        if isinstance(previous_value, BinaryDHTValue) and expiration_time > previous_expiration_time:
            new_storage = DictionaryDHTValue()
            new_storage.store(subkey, value, expiration_time)
            return super().store(key, new_storage, new_storage.latest_expiration_time)
        if isinstance(previous_value, DictionaryDHTValue):
            if expiration_time > previous_value.latest_expiration_time:
                super().store(key, previous_value, expiration_time)  # bump the dictionary's own expiration
            return previous_value.store(subkey, value, expiration_time)
        return False

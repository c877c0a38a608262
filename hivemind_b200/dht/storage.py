"""What a DHT node keeps locally: plain values and dictionaries of sub-keys, all with expirations.

Record model (behavioural contract of hivemind/dht/storage.py:11-69): one key maps either to a single binary value
or to a ``DictionaryDHTValue`` whose entries expire independently; for the same (key, sub-key) the later expiration
wins; a dictionary replaces a plain value only if it expires later. Dictionaries travel as msgpack ext 0x50.
"""
from __future__ import annotations

import math
from typing import Optional, Union

from hivemind_b200.dht.routing import BinaryDHTValue, DHTID, Subkey
from hivemind_b200.utils.serializer import MSGPackSerializer
from hivemind_b200.utils.timed_storage import DHTExpiration, TimedStorage


@MSGPackSerializer.ext_serializable(0x50)
class DictionaryDHTValue(TimedStorage[Subkey, BinaryDHTValue]):
    """Sub-key -> (binary value, expiration). ``latest_expiration_time`` is the expiration of the whole record."""

    def __init__(self, maxsize: Optional[int] = None):
        super().__init__(maxsize)
        self.latest_expiration_time = -math.inf

    def store(self, key: Subkey, value: BinaryDHTValue, expiration_time: DHTExpiration) -> bool:
        if expiration_time > self.latest_expiration_time:
            self.latest_expiration_time = expiration_time
        return super().store(key, value, expiration_time)

    def packb(self) -> bytes:
        entries = []
        for subkey, entry in self.items():
            entries.append([subkey, entry.value, entry.expiration_time])
        return MSGPackSerializer.dumps([self.maxsize, self.latest_expiration_time, entries])

    @classmethod
    def unpackb(cls, raw: bytes) -> "DictionaryDHTValue":
        maxsize, latest, entries = MSGPackSerializer.loads(raw)
        restored = cls(maxsize)
        with restored.freeze():  # keep entries that expire while we are unpacking: the reader decides what is stale
            for subkey, value, expiration_time in entries:
                restored.store(subkey, value, expiration_time)
        restored.latest_expiration_time = latest
        return restored


StoredValue = Union[BinaryDHTValue, DictionaryDHTValue]


class DHTLocalStorage(TimedStorage[DHTID, StoredValue]):
    def store(self, key: DHTID, value: BinaryDHTValue, expiration_time: DHTExpiration,
              subkey: Optional[Subkey] = None) -> bool:
        """Store a plain value, or one dictionary entry when ``subkey`` is given. Returns whether it was accepted."""
        if subkey is None:
            return super().store(key, value, expiration_time)
        return self.store_subkey(key, subkey, value, expiration_time)

    def store_subkey(self, key: DHTID, subkey: Subkey, value: BinaryDHTValue, expiration_time: DHTExpiration) -> bool:
        current = self.get(key)
        if current is not None and isinstance(current.value, DictionaryDHTValue):
            dictionary = current.value
            if expiration_time > dictionary.latest_expiration_time:
                # the record as a whole now lives longer: re-register it under the later expiration
                super().store(key, dictionary, expiration_time)
            return dictionary.store(subkey, value, expiration_time)
        # nothing, or a plain value: a dictionary takes over only if it outlives what is there
        if current is not None and expiration_time <= current.expiration_time:
            return False
        dictionary = DictionaryDHTValue()
        dictionary.store(subkey, value, expiration_time)
        return super().store(key, dictionary, dictionary.latest_expiration_time)

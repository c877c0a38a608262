"""Expiring key-value storage and the DHT clock.

Semantics follow the reference (hivemind/utils/timed_storage.py:50-133): a newer expiration replaces an older one
for the same key, an older one is rejected; expired entries disappear on access; with ``maxsize`` the entry with the
earliest expiration is evicted first; ``freeze()`` suspends expiry while iterating.
"""
from __future__ import annotations

import heapq
import time
from contextlib import contextmanager
from dataclasses import dataclass
from typing import Dict, Generic, Iterator, List, Optional, Tuple, TypeVar

KeyType = TypeVar("KeyType")
ValueType = TypeVar("ValueType")
DHTExpiration = float
MAX_DHT_TIME_DISCREPANCY_SECONDS = 3.0  # peers whose clocks differ by more are rejected on ping

get_dht_time = time.time  # every peer uses wall-clock UTC seconds


@dataclass(frozen=True)
class ValueWithExpiration(Generic[ValueType]):
    value: ValueType
    expiration_time: DHTExpiration

    def __iter__(self):
        return iter((self.value, self.expiration_time))

    def __getitem__(self, item: int):
        return (self.value, self.expiration_time)[item]

    def __eq__(self, other):
        if isinstance(other, ValueWithExpiration):
            return self.value == other.value and self.expiration_time == other.expiration_time
        if isinstance(other, tuple):
            return tuple(self) == other
        return False

    def __hash__(self):
        return hash((self.expiration_time,))


class TimedStorage(Generic[KeyType, ValueType]):
    """Dictionary whose entries expire; not thread-safe (each owner uses it from one event loop)."""

    frozen = False

    def __init__(self, maxsize: Optional[int] = None):
        self.maxsize = maxsize if maxsize is not None else float("inf")
        self.data: Dict[KeyType, ValueWithExpiration[ValueType]] = {}
        self._heap: List[Tuple[DHTExpiration, int, KeyType]] = []
        self._tick = 0
        self._key_of: Dict[int, KeyType] = {}

    def _drop_stale_heap_top(self) -> None:
        while self._heap:
            exp, _, key = self._heap[0]
            live = self.data.get(key)
            if live is None or live.expiration_time != exp:
                heapq.heappop(self._heap)  # superseded or deleted entry
            else:
                break

    def remove_outdated(self) -> None:
        if self.frozen:
            return
        now = get_dht_time()
        while self._heap:
            self._drop_stale_heap_top()
            if not self._heap:
                break
            exp, _, key = self._heap[0]
            if exp > now and len(self.data) <= self.maxsize:
                break
            heapq.heappop(self._heap)
            del self.data[key]

    def store(self, key: KeyType, value: ValueType, expiration_time: DHTExpiration) -> bool:
        """Store unless already expired or an entry with a later-or-equal expiration exists. Returns success."""
        if expiration_time < get_dht_time() and not self.frozen:
            return False
        previous = self.data.get(key)
        if previous is not None and previous.expiration_time >= expiration_time:
            return False
        self.data[key] = ValueWithExpiration(value, expiration_time)
        self._tick += 1
        heapq.heappush(self._heap, (expiration_time, self._tick, key))
        self.remove_outdated()
        return key in self.data and self.data[key].expiration_time == expiration_time

    def get(self, key: KeyType) -> Optional[ValueWithExpiration[ValueType]]:
        self.remove_outdated()
        return self.data.get(key)

    def items(self) -> Iterator[Tuple[KeyType, ValueWithExpiration[ValueType]]]:
        self.remove_outdated()
        return ((k, v) for k, v in self.data.items())

    def top(self) -> Optional[Tuple[KeyType, ValueWithExpiration[ValueType]]]:
        """The entry that expires first, if any."""
        self.remove_outdated()
        self._drop_stale_heap_top()
        if not self._heap:
            return None
        key = self._heap[0][2]
        return key, self.data[key]

    def clear(self) -> None:
        self.data.clear()
        self._heap.clear()

    def __contains__(self, key: KeyType) -> bool:
        if not self.data:
            return False
        self.remove_outdated()
        return key in self.data

    def __len__(self) -> int:
        self.remove_outdated()
        return len(self.data)

    def __delitem__(self, key: KeyType) -> None:
        self.data.pop(key, None)  # the heap entry is dropped lazily

    def __bool__(self) -> bool:
        return len(self) > 0

    def __repr__(self) -> str:
        return f"{type(self).__name__}({self.data})"

    @contextmanager
    def freeze(self):
        """Suspend removal of expired entries inside the block (iteration stays consistent)."""
        previous, self.frozen = self.frozen, True
        try:
            yield self
        finally:
            self.frozen = previous

"""Group keys: where in the DHT averagers announce that they look for a group.

Keys are ``{prefix}.0b{bits}``; under each key every averager stores (sub-key = its peer id) whether it is still
looking, with the expiration = the time by which it wants to start. After a successful round every member derives
new bits from the group id and its index, so that over several rounds peers mix across the whole swarm — the
Moshpit grid rotation (reference: hivemind/averaging/key_manager.py:13-119).
"""
from __future__ import annotations

import random
import re
from typing import List, Optional, Tuple

import numpy as np

from hivemind_b200.averaging.group_info import GroupInfo
from hivemind_b200.dht import DHT
from hivemind_b200.p2p import PeerID
from hivemind_b200.utils import DHTExpiration, get_logger

GroupKey = str
GROUP_PATTERN = re.compile("^(([^.])+)[.]0b[01]*$")  # e.g. bert_exp4_averaging.0b01001101
DEFAULT_NUM_BUCKETS = 256
logger = get_logger(__name__)


def is_valid_group(maybe_group: str) -> bool:
    """A group key must be ``<prefix>.0b<bits>`` with a dot-free prefix."""
    return bool(GROUP_PATTERN.fullmatch(maybe_group))


class GroupKeyManager:
    def __init__(self, dht: DHT, prefix: str, initial_group_bits: str, target_group_size: Optional[int]):
        assert all(bit in "01" for bit in initial_group_bits)
        if target_group_size is not None and not is_power_of_two(target_group_size):
            logger.warning("It is recommended to set target_group_size to a power of 2")
        self.dht, self.prefix, self.group_bits = dht, prefix, initial_group_bits
        self.target_group_size = target_group_size
        self.peer_id = dht.peer_id

    @property
    def current_key(self) -> GroupKey:
        return f"{self.prefix}.0b{self.group_bits}"

    async def declare_averager(self, group_key: GroupKey, peer_id: PeerID, expiration_time: float,
                               looking_for_group: bool = True) -> bool:
        """Announce (or, with ``looking_for_group=False``, retract) that this averager waits for groupmates."""
        # a retraction must supersede the announcement it cancels, hence the slightly later expiration
        expiration_time = expiration_time if looking_for_group else float(np.nextafter(expiration_time, float("inf")))
        return await self.dht.store(key=group_key, subkey=peer_id.to_bytes(), value=looking_for_group,
                                    expiration_time=expiration_time, return_future=True)

    async def get_averagers(self, group_key: GroupKey, only_active: bool) -> List[Tuple[PeerID, DHTExpiration]]:
        """Averagers announced under ``group_key`` with their expirations."""
        assert is_valid_group(group_key), f"Group key {group_key} is invalid, must follow {GROUP_PATTERN}"
        result = await self.dht.get(group_key, latest=True, return_future=True)
        if result is None or not isinstance(result.value, dict):
            logger.debug(f"Allreduce group not found: {group_key}, creating new group")
            return []
        averagers = []
        for key, looking_for_group in result.value.items():
            try:
                if only_active and not looking_for_group.value:
                    continue
                averagers.append((PeerID(key), looking_for_group.expiration_time))
            except Exception as e:
                logger.warning(f"Could not parse group key {key} ({looking_for_group}, exc={e!r})")
        return averagers

    async def update_key_on_group_assembled(self, group_info: GroupInfo) -> None:
        """Pick the next group bits so that this group's members land in different buckets next time."""
        num_buckets = self.target_group_size
        if num_buckets is None:
            num_buckets = next_power_of_two(group_info.group_size)
        my_index = group_info.peer_ids.index(self.peer_id)
        generator = random.Random(group_info.group_id)  # every member derives the same permutation
        if len(group_info.peer_ids) > num_buckets:
            # more members than buckets: some share a bucket
            index_sequence = [generator.randrange(num_buckets) for _ in range(len(group_info.peer_ids))]
            my_bucket = index_sequence[my_index]
        else:
            my_bucket = generator.sample(range(num_buckets), group_info.group_size)[my_index]
        new_bits = bin(my_bucket)[2:].rjust(int(np.ceil(np.log2(num_buckets))), "0") if num_buckets > 1 else ""
        nbits = len(self.group_bits)
        self.group_bits = (self.group_bits + new_bits)[-nbits:] if nbits else ""
        logger.debug(f"{self.peer_id} - updated group key to {self.group_bits}")

    async def update_key_on_not_enough_peers(self) -> None:
        """Matchmaking failed for lack of peers: nothing to change (kept for subclasses that shrink the key)."""


def is_power_of_two(n: int) -> bool:
    return (n != 0) and (n & (n - 1) == 0)


def next_power_of_two(n: int) -> int:
    return 1 if n == 0 else 2 ** (n - 1).bit_length()

"""Kademlia identifiers and routing table.

``DHTID`` is a 160-bit integer: SHA-1 of the msgpack-serialized key (same derivation as the reference,
hivemind/dht/routing.py:252-273, so that keys map to the same ids). The routing table is a list of k-buckets that
cover the id space; a full bucket splits if it contains our own id or if its depth is not a multiple of
``depth_modulo``; otherwise the newcomer waits in a replacement list and the least-recently-seen node is pinged.
"""
from __future__ import annotations

import bisect
import hashlib
import heapq
import os
import random
from typing import Any, Dict, List, Optional, Sequence, Set, Tuple, Union

from hivemind_b200.p2p import PeerID
from hivemind_b200.utils import MSGPackSerializer, get_dht_time

DHTKey = Any
Subkey = Any
DHTValue = Any
BinaryDHTID = bytes
BinaryDHTValue = bytes


class DHTID(int):
    HASH_FUNC = hashlib.sha1
    HASH_NBYTES = 20
    RANGE = MIN, MAX = 0, 2 ** (HASH_NBYTES * 8)

    def __new__(cls, value: int):
        assert cls.MIN <= value < cls.MAX, f"DHTID must be in [{cls.MIN}, {cls.MAX}) but got {value}"
        return super().__new__(cls, value)

    @classmethod
    def generate(cls, source: Optional[Any] = None, nbits: int = 255) -> "DHTID":
        """Hash ``source`` into an id, or draw a random id when no source is given."""
        source = random.getrandbits(nbits).to_bytes(nbits, "big") if source is None else source
        source = MSGPackSerializer.dumps(source) if not isinstance(source, bytes) else source
        return cls(int(cls.HASH_FUNC(source).hexdigest(), 16))

    def xor_distance(self, other: Union["DHTID", Sequence["DHTID"]]) -> Union[int, List[int]]:
        if isinstance(other, int):  # the common case, checked first: it is on the path of every routing decision
            return int(self) ^ int(other)
        return [int(self) ^ int(o) for o in other]

    @classmethod
    def longest_common_prefix_length(cls, *ids: "DHTID") -> int:
        bits = [bin(i)[2:].rjust(8 * cls.HASH_NBYTES, "0") for i in ids]
        return len(os.path.commonprefix(bits))

    def to_bytes(self, length: int = HASH_NBYTES, byteorder: str = "big", *, signed: bool = False) -> bytes:
        return super().to_bytes(length, byteorder, signed=signed)

    @classmethod
    def from_bytes(cls, raw: bytes, byteorder: str = "big", *, signed: bool = False) -> "DHTID":
        if len(raw) <= cls.HASH_NBYTES and not signed:
            return int.__new__(cls, int.from_bytes(raw, byteorder))  # cannot leave the id range: no check needed
        return DHTID(super().from_bytes(raw, byteorder=byteorder, signed=signed))

    def __repr__(self) -> str:
        return f"{type(self).__name__}({hex(self)})"

    def __bytes__(self) -> bytes:
        return self.to_bytes()


ID_BITS = DHTID.HASH_NBYTES * 8


class KBucket:
    """Peers whose ids lie in ``[lower, upper)``, a power-of-two slice of the id space ``depth`` halvings deep.

    Up to ``size`` peers are live members, kept from least to most recently seen; newcomers beyond that wait as
    replacements (freshest last) until a member is removed. ``request_ping_node`` hands out, one at a time, the
    stalest members that have not been probed since they were last heard from.
    """

    def __init__(self, lower: int, upper: int, size: int, depth: int = 0):
        assert upper - lower == 1 << (ID_BITS - depth), "a bucket covers exactly 2^(bits - depth) ids"
        self.lower, self.upper, self.size, self.depth = lower, upper, size, depth
        self.nodes_to_peer_id: Dict[DHTID, PeerID] = {}      # insertion order = order of last contact
        self.replacement_nodes: Dict[DHTID, PeerID] = {}
        self.nodes_requested_for_ping: Set[DHTID] = set()
        self.last_updated = get_dht_time()

    def has_in_range(self, node_id: DHTID) -> bool:
        return self.lower <= node_id < self.upper

    def add_or_update_node(self, node_id: DHTID, peer_id: PeerID) -> bool:
        """Record a contact with ``node_id``. False means the bucket is full and the node is only a replacement."""
        self.last_updated = get_dht_time()
        self.nodes_requested_for_ping.discard(node_id)  # it just answered (or called): no need to probe it
        known = self.nodes_to_peer_id.pop(node_id, None) is not None
        if known or len(self.nodes_to_peer_id) < self.size:
            self.nodes_to_peer_id[node_id] = peer_id  # (re)inserted at the fresh end
            return True
        self.replacement_nodes.pop(node_id, None)
        self.replacement_nodes[node_id] = peer_id
        return False

    def request_ping_node(self) -> Optional[Tuple[DHTID, PeerID]]:
        """The stalest member not yet handed out for probing, if there is one."""
        candidate = next((uid for uid in self.nodes_to_peer_id if uid not in self.nodes_requested_for_ping), None)
        if candidate is None:
            return None
        self.nodes_requested_for_ping.add(candidate)
        return candidate, self.nodes_to_peer_id[candidate]

    def __getitem__(self, node_id: DHTID) -> PeerID:
        member = self.nodes_to_peer_id.get(node_id)
        return member if member is not None else self.replacement_nodes[node_id]

    def __delitem__(self, node_id: DHTID) -> None:
        was_member = self.nodes_to_peer_id.pop(node_id, None) is not None
        was_spare = self.replacement_nodes.pop(node_id, None) is not None
        if not (was_member or was_spare):
            raise KeyError(f"KBucket does not contain node id={node_id}")
        if was_member and self.replacement_nodes:  # the freshest replacement takes the free seat
            promoted, address = self.replacement_nodes.popitem()
            self.nodes_to_peer_id[promoted] = address

    def split(self) -> Tuple["KBucket", "KBucket"]:
        """Two buckets of half the range; members and replacements are re-seated in their order of last contact."""
        middle = self.lower + (self.upper - self.lower) // 2
        halves = (KBucket(self.lower, middle, self.size, self.depth + 1),
                  KBucket(middle, self.upper, self.size, self.depth + 1))
        for group in (self.nodes_to_peer_id, self.replacement_nodes):
            for node_id, peer_id in group.items():
                halves[int(node_id) >= middle].add_or_update_node(node_id, peer_id)
        return halves

    def __repr__(self) -> str:
        return (f"{type(self).__name__}({len(self.nodes_to_peer_id)} nodes, {len(self.replacement_nodes)} replacements, "
                f"depth={self.depth}, lower={hex(self.lower)}, upper={hex(self.upper)})")


class RoutingTable:
    """K-buckets in id order plus the two directories (node id <-> transport peer id) of everybody in them."""

    def __init__(self, node_id: DHTID, bucket_size: int, depth_modulo: int):
        self.node_id, self.bucket_size, self.depth_modulo = node_id, bucket_size, depth_modulo
        self.buckets = [KBucket(node_id.MIN, node_id.MAX, bucket_size)]
        self._lower_bounds = [int(node_id.MIN)]  # of self.buckets, for bisection
        self.peer_id_to_uid: Dict[PeerID, DHTID] = {}
        self.uid_to_peer_id: Dict[DHTID, PeerID] = {}

    def get_bucket_index(self, node_id: DHTID) -> int:
        index = bisect.bisect_right(self._lower_bounds, int(node_id)) - 1
        assert self.buckets[index].has_in_range(node_id)
        return index

    def _may_split(self, bucket: KBucket) -> bool:
        # our own neighbourhood is always refined; elsewhere only depths that are not a multiple of depth_modulo
        return bucket.has_in_range(self.node_id) or bucket.depth % self.depth_modulo != 0

    def add_or_update_node(self, node_id: DHTID, peer_id: PeerID) -> Optional[Tuple[DHTID, PeerID]]:
        """Insert or refresh a node. If its bucket is full and cannot split, returns a node that should be pinged."""
        while True:
            index = self.get_bucket_index(node_id)
            bucket = self.buckets[index]
            seated = bucket.add_or_update_node(node_id, peer_id)
            self.uid_to_peer_id[node_id] = peer_id  # members and replacements are both listed
            self.peer_id_to_uid[peer_id] = node_id
            if seated:
                return None
            if not self._may_split(bucket):
                return bucket.request_ping_node()
            self.split_bucket(index)

    def split_bucket(self, index: int) -> None:
        low, high = self.buckets[index].split()
        self.buckets[index:index + 1] = [low, high]
        self._lower_bounds[index:index + 1] = [low.lower, high.lower]

    def get(self, *, node_id: Optional[DHTID] = None, peer_id: Optional[PeerID] = None, default=None):
        assert (node_id is None) != (peer_id is None), "specify either node_id or peer_id, not both"
        directory, key = (self.uid_to_peer_id, node_id) if node_id is not None else (self.peer_id_to_uid, peer_id)
        return directory.get(key, default)

    def _directory_for(self, item: Union[DHTID, PeerID]):
        return self.uid_to_peer_id if isinstance(item, DHTID) else self.peer_id_to_uid

    def __getitem__(self, item: Union[DHTID, PeerID]) -> Union[PeerID, DHTID]:
        return self._directory_for(item)[item]

    def __setitem__(self, node_id: DHTID, peer_id: PeerID):
        raise NotImplementedError("use add_or_update_node: it may return a node that must be pinged first")

    def __contains__(self, item: Union[DHTID, PeerID]) -> bool:
        return item in self._directory_for(item)

    def __delitem__(self, node_id: DHTID) -> None:
        del self.buckets[self.get_bucket_index(node_id)][node_id]
        address = self.uid_to_peer_id.pop(node_id)
        if self.peer_id_to_uid.get(address) == node_id:
            del self.peer_id_to_uid[address]

    def get_nearest_neighbors(self, query_id: DHTID, k: int, exclude: Optional[DHTID] = None) -> List[Tuple[DHTID, PeerID]]:
        """The k known nodes nearest to ``query_id`` by XOR distance, nearest first.

        Buckets are visited outwards from the one that contains the query: a bucket can only hold nearer nodes than
        the current k-th best if the lowest possible distance to its range is below that bound.
        """
        best: List[Tuple[int, DHTID, PeerID]] = []  # max-heap by negative distance

        def visit(bucket: KBucket) -> None:
            for node_id, peer_id in bucket.nodes_to_peer_id.items():
                if exclude is not None and node_id == exclude:
                    continue
                dist = int(query_id) ^ int(node_id)
                if len(best) < k:
                    heapq.heappush(best, (-dist, node_id, peer_id))
                elif dist < -best[0][0]:
                    heapq.heapreplace(best, (-dist, node_id, peer_id))

        def min_distance_to(bucket: KBucket) -> int:
            if bucket.has_in_range(query_id):
                return 0
            # nodes in the bucket share its prefix; the differing prefix bits give a lower bound on the distance
            prefix_len = bucket.depth
            shift = DHTID.HASH_NBYTES * 8 - prefix_len
            return ((int(query_id) >> shift) ^ (bucket.lower >> shift)) << shift

        order = sorted(range(len(self.buckets)), key=lambda i: min_distance_to(self.buckets[i]))
        for i in order:
            if len(best) >= k and min_distance_to(self.buckets[i]) > -best[0][0]:
                break
            visit(self.buckets[i])
        return [(node_id, peer_id) for _, node_id, peer_id in sorted(best, key=lambda t: -t[0])]

    def __repr__(self) -> str:
        bucket_info = "\n".join(repr(bucket) for bucket in self.buckets)
        return (f"{type(self).__name__}(node_id={self.node_id}, bucket_size={self.bucket_size}, "
                f"modulo={self.depth_modulo},\nbuckets=[\n{bucket_info})")

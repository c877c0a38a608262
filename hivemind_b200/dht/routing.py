"""Kademlia identifiers and routing table.

``DHTID`` is a 160-bit integer: SHA-1 of the msgpack-serialized key (same derivation as the reference,
hivemind/dht/routing.py:252-273, so that keys map to the same ids). The routing table is a list of k-buckets that
cover the id space; a full bucket splits if it contains our own id or if its depth is not a multiple of
``depth_modulo``; otherwise the newcomer waits in a replacement list and the least-recently-seen node is pinged.
"""
from __future__ import annotations

import hashlib
import heapq
import os
import random
from collections.abc import Iterable
from itertools import chain
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
        if isinstance(other, Iterable):
            return [int(self) ^ int(o) for o in other]
        return int(self) ^ int(other)

    @classmethod
    def longest_common_prefix_length(cls, *ids: "DHTID") -> int:
        bits = [bin(i)[2:].rjust(8 * cls.HASH_NBYTES, "0") for i in ids]
        return len(os.path.commonprefix(bits))

    def to_bytes(self, length: int = HASH_NBYTES, byteorder: str = "big", *, signed: bool = False) -> bytes:
        return super().to_bytes(length, byteorder, signed=signed)

    @classmethod
    def from_bytes(cls, raw: bytes, byteorder: str = "big", *, signed: bool = False) -> "DHTID":
        return DHTID(super().from_bytes(raw, byteorder=byteorder, signed=signed))

    def __repr__(self) -> str:
        return f"{type(self).__name__}({hex(self)})"

    def __bytes__(self) -> bytes:
        return self.to_bytes()


class KBucket:
    """Nodes whose ids fall in [lower, upper); at most ``size`` live entries plus a replacement list."""

    def __init__(self, lower: int, upper: int, size: int, depth: int = 0):
        assert upper - lower == 2 ** (DHTID.HASH_NBYTES * 8 - depth)
        self.lower, self.upper, self.size, self.depth = lower, upper, size, depth
        self.nodes_to_peer_id: Dict[DHTID, PeerID] = {}
        self.replacement_nodes: Dict[DHTID, PeerID] = {}
        self.nodes_requested_for_ping: Set[DHTID] = set()
        self.last_updated = get_dht_time()

    def has_in_range(self, node_id: DHTID) -> bool:
        return self.lower <= node_id < self.upper

    def add_or_update_node(self, node_id: DHTID, peer_id: PeerID) -> bool:
        """Returns False if the bucket is full (the node then waits in the replacement list)."""
        if node_id in self.nodes_requested_for_ping:
            self.nodes_requested_for_ping.remove(node_id)
        self.last_updated = get_dht_time()
        if node_id in self.nodes_to_peer_id:
            del self.nodes_to_peer_id[node_id]  # move to the most-recently-seen end
            self.nodes_to_peer_id[node_id] = peer_id
        elif len(self.nodes_to_peer_id) < self.size:
            self.nodes_to_peer_id[node_id] = peer_id
        else:
            self.replacement_nodes.pop(node_id, None)
            self.replacement_nodes[node_id] = peer_id
            return False
        return True

    def request_ping_node(self) -> Optional[Tuple[DHTID, PeerID]]:
        """The least-recently-seen node that has not been asked yet, if any."""
        for uid, peer_id in self.nodes_to_peer_id.items():
            if uid not in self.nodes_requested_for_ping:
                self.nodes_requested_for_ping.add(uid)
                return uid, peer_id
        return None

    def __getitem__(self, node_id: DHTID) -> PeerID:
        return self.nodes_to_peer_id[node_id] if node_id in self.nodes_to_peer_id else self.replacement_nodes[node_id]

    def __delitem__(self, node_id: DHTID) -> None:
        if not (node_id in self.nodes_to_peer_id or node_id in self.replacement_nodes):
            raise KeyError(f"KBucket does not contain node id={node_id}")
        self.replacement_nodes.pop(node_id, None)
        if node_id in self.nodes_to_peer_id:
            del self.nodes_to_peer_id[node_id]
            if self.replacement_nodes:  # promote the freshest replacement
                newnode_id, newnode = self.replacement_nodes.popitem()
                self.nodes_to_peer_id[newnode_id] = newnode

    def split(self) -> Tuple["KBucket", "KBucket"]:
        midpoint = (self.lower + self.upper) // 2
        left = KBucket(self.lower, midpoint, self.size, self.depth + 1)
        right = KBucket(midpoint, self.upper, self.size, self.depth + 1)
        for node_id, peer_id in chain(self.nodes_to_peer_id.items(), self.replacement_nodes.items()):
            (left if int(node_id) < midpoint else right).add_or_update_node(node_id, peer_id)
        return left, right

    def __repr__(self) -> str:
        return (f"{type(self).__name__}({len(self.nodes_to_peer_id)} nodes, {len(self.replacement_nodes)} replacements, "
                f"depth={self.depth}, lower={hex(self.lower)}, upper={hex(self.upper)})")


class RoutingTable:
    def __init__(self, node_id: DHTID, bucket_size: int, depth_modulo: int):
        self.node_id, self.bucket_size, self.depth_modulo = node_id, bucket_size, depth_modulo
        self.buckets = [KBucket(node_id.MIN, node_id.MAX, bucket_size)]
        self.peer_id_to_uid: Dict[PeerID, DHTID] = {}
        self.uid_to_peer_id: Dict[DHTID, PeerID] = {}

    def get_bucket_index(self, node_id: DHTID) -> int:
        lo, hi = 0, len(self.buckets)
        while hi - lo > 1:
            mid = (lo + hi) // 2
            if node_id >= self.buckets[mid].lower:
                lo = mid
            else:
                hi = mid
        assert self.buckets[lo].has_in_range(node_id)
        return lo

    def add_or_update_node(self, node_id: DHTID, peer_id: PeerID) -> Optional[Tuple[DHTID, PeerID]]:
        """Insert or refresh a node. If its bucket is full and cannot split, returns a node that should be pinged."""
        bucket_index = self.get_bucket_index(node_id)
        bucket = self.buckets[bucket_index]
        store_success = bucket.add_or_update_node(node_id, peer_id)
        if node_id in bucket.nodes_to_peer_id or node_id in bucket.replacement_nodes:
            self.uid_to_peer_id[node_id] = peer_id
            self.peer_id_to_uid[peer_id] = node_id
        if not store_success:
            if bucket.has_in_range(self.node_id) or bucket.depth % self.depth_modulo != 0:
                self.split_bucket(bucket_index)
                return self.add_or_update_node(node_id, peer_id)
            return bucket.request_ping_node()
        return None

    def split_bucket(self, index: int) -> None:
        first, second = self.buckets[index].split()
        self.buckets[index] = first
        self.buckets.insert(index + 1, second)

    def get(self, *, node_id: Optional[DHTID] = None, peer_id: Optional[PeerID] = None, default=None):
        assert (node_id is None) != (peer_id is None), "specify either node_id or peer_id, not both"
        if node_id is not None:
            return self.uid_to_peer_id.get(node_id, default)
        return self.peer_id_to_uid.get(peer_id, default)

    def __getitem__(self, item: Union[DHTID, PeerID]) -> Union[PeerID, DHTID]:
        return self.uid_to_peer_id[item] if isinstance(item, DHTID) else self.peer_id_to_uid[item]

    def __setitem__(self, node_id: DHTID, peer_id: PeerID):
        raise NotImplementedError("use add_or_update_node: it may return a node that must be pinged first")

    def __contains__(self, item: Union[DHTID, PeerID]) -> bool:
        return (item in self.uid_to_peer_id) if isinstance(item, DHTID) else (item in self.peer_id_to_uid)

    def __delitem__(self, node_id: DHTID) -> None:
        del self.buckets[self.get_bucket_index(node_id)][node_id]
        node_peer_id = self.uid_to_peer_id.pop(node_id)
        if self.peer_id_to_uid.get(node_peer_id) == node_id:
            del self.peer_id_to_uid[node_peer_id]

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

"""The three RPCs of the DHT (ping, store, find) and the routing-table upkeep around them.

Behavioural contract (hivemind/dht/protocol.py:25-430): every request and reply carries the sender's node info, so
that both sides learn about each other; a node that newly enters the routing table is handed the keys it is now
nearer to than we are; client-mode nodes register no handlers and send no node info (nobody routes to them);
``validate=True`` pings check that the requester can be reached from outside and that clocks agree within 3 seconds.

Layout of this file: ``_exchange`` is the one place where an outgoing call is made, throttled and booked into the
routing table; the ``call_*`` methods only build requests and decode replies; the ``rpc_*`` handlers use
``_accept_record`` / ``_freshest_local`` for the storage side.
"""
from __future__ import annotations

import asyncio
from typing import Collection, Dict, Iterable, List, Optional, Sequence, Tuple, Union

from hivemind_b200.dht.crypto import DHTRecord, RecordValidatorBase
from hivemind_b200.dht.routing import BinaryDHTValue, DHTID, RoutingTable, Subkey
from hivemind_b200.dht.storage import DHTLocalStorage, DictionaryDHTValue
from hivemind_b200.p2p import P2P, P2PContext, PeerID, ServicerBase
from hivemind_b200.proto import dht_pb2
from hivemind_b200.utils import MSGPackSerializer, get_logger
from hivemind_b200.utils.asyncio import spawn
from hivemind_b200.utils.auth import AuthorizerBase, AuthRole, AuthRPCWrapper
from hivemind_b200.utils.timed_storage import (MAX_DHT_TIME_DISCREPANCY_SECONDS, DHTExpiration, ValueWithExpiration,
                                               get_dht_time)

logger = get_logger(__name__)
StoredPayload = Union[BinaryDHTValue, DictionaryDHTValue]
FindOutcome = Dict[DHTID, Tuple[Optional[ValueWithExpiration[StoredPayload]], Dict[DHTID, PeerID]]]


class ValidationError(Exception):
    """A peer is unreachable from outside or its clock is off."""


def _announced_id(info: Optional[dht_pb2.NodeInfo]) -> Optional[DHTID]:
    """The node id inside a NodeInfo, or None for client-mode senders (which announce nothing)."""
    return DHTID.from_bytes(info.node_id) if info and info.node_id else None


class DHTProtocol(ServicerBase):
    # fmt:off
    p2p: P2P
    node_id: DHTID; bucket_size: int; num_replicas: int; wait_timeout: float; node_info: dht_pb2.NodeInfo
    storage: DHTLocalStorage; cache: DHTLocalStorage; routing_table: RoutingTable; rpc_semaphore: asyncio.Semaphore
    record_validator: Optional[RecordValidatorBase]
    # fmt:on

    serializer = MSGPackSerializer
    RESERVED_SUBKEYS = IS_REGULAR_VALUE, IS_DICTIONARY = serializer.dumps(None), b""
    MAX_KNOWN_PAIRS = 2 ** 16  # (node id, peer id) objects kept for reuse when find replies are decoded

    def __init__(self, *, _initialized_with_create: bool = False):
        if not _initialized_with_create:
            raise RuntimeError("use `await DHTProtocol.create(...)`")
        super().__init__()

    @classmethod
    async def create(cls, p2p: P2P, node_id: DHTID, bucket_size: int, depth_modulo: int, num_replicas: int,
                     wait_timeout: float, parallel_rpc: Optional[int] = None, cache_size: Optional[int] = None,
                     client_mode: bool = False, record_validator: Optional[RecordValidatorBase] = None,
                     authorizer: Optional[AuthorizerBase] = None) -> "DHTProtocol":
        self = cls(_initialized_with_create=True)
        self.p2p, self.node_id = p2p, node_id
        self.bucket_size, self.num_replicas, self.wait_timeout = bucket_size, num_replicas, wait_timeout
        self.client_mode, self.record_validator, self.authorizer = client_mode, record_validator, authorizer
        self.storage, self.cache = DHTLocalStorage(), DHTLocalStorage(maxsize=cache_size)
        self.routing_table = RoutingTable(node_id, bucket_size, depth_modulo)
        self._known_pairs: Dict[bytes, Tuple[DHTID, PeerID, bytes]] = {}
        self.rpc_semaphore = asyncio.Semaphore(2 ** 15 if parallel_rpc is None else parallel_rpc)
        # clients are never routed to, so they announce no id and serve no requests
        self.node_info = dht_pb2.NodeInfo() if client_mode else dht_pb2.NodeInfo(node_id=node_id.to_bytes())
        if not client_mode:
            await self.add_p2p_handlers(p2p, AuthRPCWrapper(self, AuthRole.SERVICER, authorizer))
        return self

    async def shutdown(self) -> None:
        if self.client_mode:
            return
        try:
            await self.remove_p2p_handlers(self.p2p)
        except Exception as e:
            logger.debug(f"could not unregister the DHT handlers: {e!r}")

    def get_stub(self, peer: PeerID) -> AuthRPCWrapper:
        return AuthRPCWrapper(super().get_stub(self.p2p, peer), AuthRole.CLIENT, self.authorizer, service_public_key=None)

    async def _exchange(self, peer: PeerID, method: str, request):
        """One outgoing call: throttled, timed out, and booked into the routing table either way.
        Returns the reply, or None if the peer did not answer properly."""
        try:
            async with self.rpc_semaphore:
                reply = await getattr(self.get_stub(peer), method)(request, timeout=self.wait_timeout)
        except Exception as e:
            logger.debug(f"{method} to {peer} failed: {e!r}")
            spawn(self.update_routing_table(self.routing_table.get(peer_id=peer), peer, responded=False))
            return None
        replier = _announced_id(reply.peer)
        if replier is not None:
            spawn(self.update_routing_table(replier, peer, responded=True))
        return reply

    # ---------------------------------------------------------------------------------------------- ping
    async def call_ping(self, peer: PeerID, validate: bool = False, strict: bool = True) -> Optional[DHTID]:
        """Ping ``peer``, learn its node id (None if it did not answer). With ``validate`` also check that it can
        reach us and that our clocks agree; ``strict`` turns a failed validation into ``ValidationError``."""
        reply, sent_at, received_at = None, get_dht_time(), None
        try:
            async with self.rpc_semaphore:
                sent_at = get_dht_time()
                reply = await self.get_stub(peer).rpc_ping(dht_pb2.PingRequest(peer=self.node_info, validate=validate),
                                                           timeout=self.wait_timeout)
                received_at = get_dht_time()
        except Exception as e:
            logger.debug(f"ping to {peer} failed: {e!r}")
        their_id = _announced_id(reply.peer) if reply is not None else None
        if their_id is not None and validate:
            problem = self._ping_problem(peer, reply, sent_at, received_at)
            if problem is not None:
                if strict:
                    raise ValidationError(problem)
                logger.warning(problem)
        spawn(self.update_routing_table(their_id, peer, responded=their_id is not None))
        return their_id

    def _ping_problem(self, peer: PeerID, reply: dht_pb2.PingResponse, sent_at: float, received_at: float) -> Optional[str]:
        if not self.client_mode and not reply.available:
            return (f"peer {peer} cannot reach this node: make sure that this node is reachable from outside or start "
                    f"it in client mode")
        unset = dht_pb2.PingResponse.DESCRIPTOR.fields_by_name["dht_time"].default_value
        slack = MAX_DHT_TIME_DISCREPANCY_SECONDS
        if reply.dht_time != unset and not (sent_at - slack <= reply.dht_time <= received_at + slack):
            return (f"local time must be within {slack} seconds of other peers' "
                    f"(local {sent_at:.5f}, peer {reply.dht_time:.5f})")
        return None

    async def rpc_ping(self, request: dht_pb2.PingRequest, context: P2PContext) -> dht_pb2.PingResponse:
        reply = dht_pb2.PingResponse(peer=self.node_info, dht_time=get_dht_time(), available=False)
        sender = _announced_id(request.peer)
        if sender is not None:
            if request.validate:  # can we call the caller back, and is it who it says it is?
                reply.available = await self.call_ping(context.remote_id, validate=False) == sender
            spawn(self.update_routing_table(sender, context.remote_id, responded=reply.available or not request.validate))
        return reply

    # ---------------------------------------------------------------------------------------------- store
    async def call_store(self, peer: PeerID, keys: Sequence[DHTID], values: Sequence[StoredPayload],
                         expiration_time: Union[DHTExpiration, Sequence[DHTExpiration]],
                         subkeys: Optional[Union[Subkey, Sequence[Optional[Subkey]]]] = None,
                         in_cache: Optional[Union[bool, Sequence[bool]]] = None) -> Optional[List[bool]]:
        """Ask ``peer`` to store (key, [subkey,] value, expiration) records; returns per-record success or None."""
        count = len(keys)
        expirations = [expiration_time] * count if isinstance(expiration_time, (int, float)) else list(expiration_time)
        subkeys = [None] * count if subkeys is None else list(subkeys)
        cache_flags = [bool(in_cache)] * count if in_cache is None or isinstance(in_cache, bool) else list(in_cache)
        if not (len(values) == len(expirations) == len(subkeys) == len(cache_flags) == count):
            raise ValueError("keys, values, expirations, subkeys and cache flags must have equal lengths")
        tags, payloads = [], []
        for value, subkey in zip(values, subkeys):
            if isinstance(value, DictionaryDHTValue):
                if subkey is not None:
                    raise ValueError("a whole dictionary is stored without a sub-key")
                tags.append(self.IS_DICTIONARY)
                payloads.append(self.serializer.dumps(value))
            else:
                tags.append(self.IS_REGULAR_VALUE if subkey is None else self.serializer.dumps(subkey))
                payloads.append(value)
        request = dht_pb2.StoreRequest(keys=[key.to_bytes() for key in keys], subkeys=tags, values=payloads,
                                       expiration_time=expirations, in_cache=cache_flags, peer=self.node_info)
        reply = await self._exchange(peer, "rpc_store", request)
        return None if reply is None else list(reply.store_ok)

    async def rpc_store(self, request: dht_pb2.StoreRequest, context: P2PContext) -> dht_pb2.StoreResponse:
        sender = _announced_id(request.peer)
        if sender is not None:
            spawn(self.update_routing_table(sender, context.remote_id))
        if not (len(request.keys) == len(request.values) == len(request.expiration_time) == len(request.in_cache)):
            raise ValueError("malformed store request")
        verdicts = [self._accept_record(key, tag, payload, expiration, self.cache if cached else self.storage)
                    for key, tag, payload, expiration, cached in zip(request.keys, request.subkeys, request.values,
                                                                     request.expiration_time, request.in_cache)]
        return dht_pb2.StoreResponse(store_ok=verdicts, peer=self.node_info)

    def _accept_record(self, key: bytes, tag: bytes, payload: bytes, expiration: DHTExpiration,
                       where: DHTLocalStorage) -> bool:
        key_id = DHTID.from_bytes(key)
        if tag == self.IS_DICTIONARY:  # a whole dictionary: merged entry by entry
            dictionary = self.serializer.loads(payload)
            if not isinstance(dictionary, DictionaryDHTValue) or not self._validate_dictionary(key, dictionary):
                return False
            return all([where.store_subkey(key_id, subkey, entry.value, entry.expiration_time)
                        for subkey, entry in dictionary.items()])
        if not self._validate_record(key, tag, payload, expiration):
            return False
        if tag == self.IS_REGULAR_VALUE:
            return where.store(key_id, payload, expiration)
        return where.store_subkey(key_id, self.serializer.loads(tag), payload, expiration)

    # ---------------------------------------------------------------------------------------------- find
    async def call_find(self, peer: PeerID, keys: Collection[DHTID]) -> Optional[FindOutcome]:
        """Ask ``peer`` for the values of ``keys`` and for its nearest known nodes to each key.

        :returns: ``{key: (value with expiration or None, {nearest node id: peer id})}``, or None if the call failed
        """
        keys = list(keys)
        reply = await self._exchange(peer, "rpc_find", dht_pb2.FindRequest(keys=[k.to_bytes() for k in keys],
                                                                           peer=self.node_info))
        if reply is None:
            return None
        if len(reply.results) != len(keys):
            logger.debug(f"{peer} answered {len(reply.results)} of {len(keys)} keys; the reply is ignored")
            return None
        outcome: FindOutcome = {}
        known_pairs = self._known_pairs
        for key_id, result in zip(keys, reply.results):
            try:
                neighbours = {}
                for node_bytes, peer_bytes in zip(result.nearest_node_ids, result.nearest_peer_ids):
                    pair = known_pairs.get(node_bytes)
                    if pair is None or pair[2] != peer_bytes:
                        pair = self._node_and_peer(node_bytes, peer_bytes)
                    neighbours[pair[0]] = pair[1]
                outcome[key_id] = self._decode_find_result(key_id, result), neighbours
            except Exception as e:
                logger.debug(f"undecodable find result from {peer}: {e!r}")
                return None
        return outcome

    def _node_and_peer(self, node_bytes: bytes, peer_bytes: bytes) -> Tuple[DHTID, PeerID, bytes]:
        """(node id, peer id) objects for a routing entry of a reply. A swarm of n peers mentions the same n pairs
        over and over (up to ``bucket_size`` per key and reply), so the objects are made once and shared."""
        pair = self._known_pairs.get(node_bytes)
        if pair is None or pair[2] != peer_bytes:
            if len(self._known_pairs) >= self.MAX_KNOWN_PAIRS:
                self._known_pairs.clear()
            pair = self._known_pairs[node_bytes] = (DHTID.from_bytes(node_bytes), PeerID(peer_bytes), peer_bytes)
        return pair

    def _decode_find_result(self, key_id: DHTID, result: dht_pb2.FindResult
                            ) -> Optional[ValueWithExpiration[StoredPayload]]:
        if result.type == dht_pb2.FOUND_REGULAR:
            if self._validate_record(key_id.to_bytes(), self.IS_REGULAR_VALUE, result.value, result.expiration_time):
                return ValueWithExpiration(result.value, result.expiration_time)
        elif result.type == dht_pb2.FOUND_DICTIONARY:
            dictionary = self.serializer.loads(result.value)
            if self._validate_dictionary(key_id.to_bytes(), dictionary):
                return ValueWithExpiration(dictionary, result.expiration_time)
        elif result.type != dht_pb2.NOT_FOUND:
            logger.error(f"a find result of unknown type {result.type} was ignored")
        return None

    async def rpc_find(self, request: dht_pb2.FindRequest, context: P2PContext) -> dht_pb2.FindResponse:
        sender = _announced_id(request.peer)
        if sender is not None:
            spawn(self.update_routing_table(sender, context.remote_id))
        results = []
        for key_id in map(DHTID.from_bytes, request.keys):
            held = self._freshest_local(key_id)
            if held is None:
                result = dht_pb2.FindResult(type=dht_pb2.NOT_FOUND)
            elif isinstance(held.value, DictionaryDHTValue):
                result = dht_pb2.FindResult(type=dht_pb2.FOUND_DICTIONARY, value=self.serializer.dumps(held.value),
                                            expiration_time=held.expiration_time)
            else:
                result = dht_pb2.FindResult(type=dht_pb2.FOUND_REGULAR, value=held.value,
                                            expiration_time=held.expiration_time)
            nearest = self.routing_table.get_nearest_neighbors(key_id, k=self.bucket_size, exclude=sender)
            result.nearest_node_ids.extend([node.to_bytes() for node, _ in nearest])
            result.nearest_peer_ids.extend([address.to_bytes() for _, address in nearest])
            results.append(result)
        return dht_pb2.FindResponse(results=results, peer=self.node_info)

    def _freshest_local(self, key_id: DHTID) -> Optional[ValueWithExpiration[StoredPayload]]:
        stored, cached = self.storage.get(key_id), self.cache.get(key_id)
        if stored is None or (cached is not None and cached.expiration_time > stored.expiration_time):
            return cached
        return stored

    # ---------------------------------------------------------------------------------------------- routing upkeep
    async def update_routing_table(self, node_id: Optional[DHTID], peer_id: PeerID, responded: bool = True) -> None:
        """Record that ``peer_id`` answered (or failed to). New nodes receive the keys they are now nearest to."""
        if node_id is None:
            node_id = self.routing_table.get(peer_id=peer_id)
        if node_id is None:
            return
        if not responded:
            if node_id in self.routing_table:
                del self.routing_table[node_id]
            return
        if node_id not in self.routing_table:
            handover = list(self._records_that_belong_to(node_id))
            if handover:
                keys, payloads, expirations = zip(*handover)
                spawn(self.call_store(peer_id, keys, payloads, expirations, in_cache=False))
        evicted_candidate = self.routing_table.add_or_update_node(node_id, peer_id)
        if evicted_candidate is not None:
            # the bucket is full: find out whether its least recently seen member is still around
            spawn(self.call_ping(evicted_candidate[1]))

    def _records_that_belong_to(self, newcomer: DHTID) -> Iterable[Tuple[DHTID, StoredPayload, DHTExpiration]]:
        """Records for which this node has been the nearest holder and the newcomer now is among the replicas."""
        for key, entry in list(self.storage.items()):
            replicas = self.routing_table.get_nearest_neighbors(key, self.num_replicas, exclude=self.node_id)
            if replicas:
                nearest, farthest = replicas[0][0].xor_distance(key), replicas[-1][0].xor_distance(key)
                if not (newcomer.xor_distance(key) < farthest and self.node_id.xor_distance(key) < nearest):
                    continue
            yield key, entry.value, entry.expiration_time

    # ---------------------------------------------------------------------------------------------- validation
    def _validate_record(self, key_bytes: bytes, subkey_bytes: bytes, value_bytes: bytes, expiration_time: float) -> bool:
        if self.record_validator is None:
            return True
        return self.record_validator.validate(DHTRecord(key_bytes, subkey_bytes, value_bytes, expiration_time))

    def _validate_dictionary(self, key_bytes: bytes, dictionary: DictionaryDHTValue) -> bool:
        if self.record_validator is None:
            return True
        with dictionary.freeze():
            return all(self._validate_record(key_bytes, self.serializer.dumps(subkey), raw, expiration)
                       for subkey, (raw, expiration) in dictionary.items())

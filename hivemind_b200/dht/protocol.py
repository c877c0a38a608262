"""The three RPCs of the DHT (ping, store, find) and the routing-table upkeep around them.

Behavioural contract from the reference (hivemind/dht/protocol.py:25-430): every request carries the sender's node
info so that receivers learn about senders; a node that enters the routing table is handed the keys it is now closer
to than we are; client-mode nodes register no handlers and send no node info; ``validate=True`` pings check that the
requester is reachable and that clocks agree within 3 seconds.
"""
from __future__ import annotations

import asyncio
from typing import Collection, Dict, List, Optional, Sequence, Tuple, Union

from hivemind_b200.utils.asyncio import spawn
from hivemind_b200.dht.crypto import DHTRecord, RecordValidatorBase
from hivemind_b200.dht.routing import BinaryDHTValue, DHTID, RoutingTable, Subkey
from hivemind_b200.dht.storage import DHTLocalStorage, DictionaryDHTValue
from hivemind_b200.p2p import P2P, P2PContext, PeerID, ServicerBase
from hivemind_b200.proto import dht_pb2
from hivemind_b200.utils import MSGPackSerializer, get_logger
from hivemind_b200.utils.auth import AuthorizerBase, AuthRole, AuthRPCWrapper
from hivemind_b200.utils.timed_storage import (MAX_DHT_TIME_DISCREPANCY_SECONDS, DHTExpiration, ValueWithExpiration,
                                               get_dht_time)

logger = get_logger(__name__)


class ValidationError(Exception):
    """A peer is unreachable from outside or its clock is off."""


class DHTProtocol(ServicerBase):
    # fmt:off
    p2p: P2P
    node_id: DHTID; bucket_size: int; num_replicas: int; wait_timeout: float; node_info: dht_pb2.NodeInfo
    storage: DHTLocalStorage; cache: DHTLocalStorage; routing_table: RoutingTable; rpc_semaphore: asyncio.Semaphore
    record_validator: Optional[RecordValidatorBase]
    # fmt:on

    serializer = MSGPackSerializer
    RESERVED_SUBKEYS = IS_REGULAR_VALUE, IS_DICTIONARY = serializer.dumps(None), b""

    @classmethod
    async def create(cls, p2p: P2P, node_id: DHTID, bucket_size: int, depth_modulo: int, num_replicas: int,
                     wait_timeout: float, parallel_rpc: Optional[int] = None, cache_size: Optional[int] = None,
                     client_mode: bool = False, record_validator: Optional[RecordValidatorBase] = None,
                     authorizer: Optional[AuthorizerBase] = None) -> "DHTProtocol":
        self = cls(_initialized_with_create=True)
        self.p2p = p2p
        self.node_id, self.bucket_size, self.num_replicas = node_id, bucket_size, num_replicas
        self.wait_timeout = wait_timeout
        self.storage, self.cache = DHTLocalStorage(), DHTLocalStorage(maxsize=cache_size)
        self.routing_table = RoutingTable(node_id, bucket_size, depth_modulo)
        self.rpc_semaphore = asyncio.Semaphore(parallel_rpc if parallel_rpc is not None else 2 ** 15)
        self.client_mode = client_mode
        self.record_validator = record_validator
        self.authorizer = authorizer
        if not client_mode:
            await self.add_p2p_handlers(self.p2p, AuthRPCWrapper(self, AuthRole.SERVICER, self.authorizer))
            self.node_info = dht_pb2.NodeInfo(node_id=node_id.to_bytes())
        else:
            self.node_info = dht_pb2.NodeInfo()  # clients are never routed to
        return self

    def __init__(self, *, _initialized_with_create: bool = False):
        assert _initialized_with_create, "use DHTProtocol.create coroutine to spawn new protocol instances"
        super().__init__()

    async def shutdown(self) -> None:
        if not self.client_mode:
            try:
                await self.remove_p2p_handlers(self.p2p)
            except Exception:
                pass

    def get_stub(self, peer: PeerID) -> AuthRPCWrapper:
        stub = super().get_stub(self.p2p, peer)
        return AuthRPCWrapper(stub, AuthRole.CLIENT, self.authorizer, service_public_key=None)

    # ---------------------------------------------------------------------------------------------- ping
    async def call_ping(self, peer: PeerID, validate: bool = False, strict: bool = True) -> Optional[DHTID]:
        """Ping ``peer``, learn its node id (None if it did not answer). With ``validate`` also check that it can
        reach us and that our clocks agree; ``strict`` turns a failed validation into ``ValidationError``."""
        try:
            async with self.rpc_semaphore:
                ping_request = dht_pb2.PingRequest(peer=self.node_info, validate=validate)
                time_requested = get_dht_time()
                response = await self.get_stub(peer).rpc_ping(ping_request, timeout=self.wait_timeout)
                time_responded = get_dht_time()
        except Exception as e:
            logger.debug(f"DHTProtocol failed to ping {peer}: {e!r}")
            response = None
        responded = bool(response and response.peer and response.peer.node_id)
        if responded and validate:
            try:
                if not self.client_mode and not response.available:
                    raise ValidationError(f"peer {peer} cannot reach this node: make sure that this node is reachable "
                                          f"from outside or start it in client mode")
                if response.dht_time != dht_pb2.PingResponse.DESCRIPTOR.fields_by_name["dht_time"].default_value:
                    if (response.dht_time < time_requested - MAX_DHT_TIME_DISCREPANCY_SECONDS
                            or response.dht_time > time_responded + MAX_DHT_TIME_DISCREPANCY_SECONDS):
                        raise ValidationError(f"local time must be within {MAX_DHT_TIME_DISCREPANCY_SECONDS} seconds "
                                              f"of other peers' (local {time_requested:.5f}, peer {response.dht_time:.5f})")
            except ValidationError as e:
                if strict:
                    raise
                logger.warning(repr(e))
        peer_id = DHTID.from_bytes(response.peer.node_id) if responded else None
        spawn(self.update_routing_table(peer_id, peer, responded=responded))
        return peer_id

    async def rpc_ping(self, request: dht_pb2.PingRequest, context: P2PContext) -> dht_pb2.PingResponse:
        response = dht_pb2.PingResponse(peer=self.node_info, dht_time=get_dht_time(), available=False)
        if request.peer and request.peer.node_id:
            sender_id = DHTID.from_bytes(request.peer.node_id)
            if request.validate:
                response.available = await self.call_ping(context.remote_id, validate=False) == sender_id
            spawn(self.update_routing_table(sender_id, context.remote_id,
                                                          responded=response.available or not request.validate))
        return response

    # ---------------------------------------------------------------------------------------------- store
    async def call_store(self, peer: PeerID, keys: Sequence[DHTID],
                         values: Sequence[Union[BinaryDHTValue, DictionaryDHTValue]],
                         expiration_time: Union[DHTExpiration, Sequence[DHTExpiration]],
                         subkeys: Optional[Union[Subkey, Sequence[Optional[Subkey]]]] = None,
                         in_cache: Optional[Union[bool, Sequence[bool]]] = None) -> Optional[List[bool]]:
        """Ask ``peer`` to store (key, [subkey,] value, expiration) records; returns per-record success or None."""
        if isinstance(expiration_time, (int, float)):
            expiration_time = [expiration_time] * len(keys)
        if subkeys is None:
            subkeys = [None] * len(keys)
        in_cache = in_cache if in_cache is not None else [False] * len(keys)
        in_cache = [in_cache] * len(keys) if isinstance(in_cache, bool) else in_cache
        keys, subkeys, values, expiration_time, in_cache = map(list, [keys, subkeys, values, expiration_time, in_cache])
        for i in range(len(keys)):
            if subkeys[i] is None:  # add default sub-key markers
                subkeys[i] = self.IS_DICTIONARY if isinstance(values[i], DictionaryDHTValue) else self.IS_REGULAR_VALUE
            else:
                subkeys[i] = self.serializer.dumps(subkeys[i])
            if isinstance(values[i], DictionaryDHTValue):
                assert subkeys[i] == self.IS_DICTIONARY, "a dictionary value cannot have a sub-key"
                values[i] = self.serializer.dumps(values[i])
        assert len(keys) == len(values) == len(expiration_time) == len(in_cache), "data is not aligned"
        store_request = dht_pb2.StoreRequest(keys=[k.to_bytes() for k in keys], subkeys=subkeys, values=values,
                                             expiration_time=expiration_time, in_cache=in_cache, peer=self.node_info)
        try:
            async with self.rpc_semaphore:
                response = await self.get_stub(peer).rpc_store(store_request, timeout=self.wait_timeout)
            if response.peer and response.peer.node_id:
                peer_id = DHTID.from_bytes(response.peer.node_id)
                spawn(self.update_routing_table(peer_id, peer, responded=True))
            return list(response.store_ok)
        except Exception as e:
            logger.debug(f"DHTProtocol failed to store at {peer}: {e!r}")
            spawn(self.update_routing_table(self.routing_table.get(peer_id=peer), peer, responded=False))
            return None

    async def rpc_store(self, request: dht_pb2.StoreRequest, context: P2PContext) -> dht_pb2.StoreResponse:
        if request.peer and request.peer.node_id:
            spawn(self.update_routing_table(DHTID.from_bytes(request.peer.node_id), context.remote_id))
        assert len(request.keys) == len(request.values) == len(request.expiration_time) == len(request.in_cache)
        response = dht_pb2.StoreResponse(store_ok=[], peer=self.node_info)
        for key, tag, value_bytes, expiration_time, in_cache in zip(
                request.keys, request.subkeys, request.values, request.expiration_time, request.in_cache):
            key_id = DHTID.from_bytes(key)
            storage = self.cache if in_cache else self.storage
            if tag == self.IS_DICTIONARY:  # a whole dictionary: merge entry by entry
                value_dictionary = self.serializer.loads(value_bytes)
                assert isinstance(value_dictionary, DictionaryDHTValue)
                if not self._validate_dictionary(key, value_dictionary):
                    response.store_ok.append(False)
                    continue
                response.store_ok.append(all(storage.store_subkey(key_id, subkey, item.value, item.expiration_time)
                                             for subkey, item in value_dictionary.items()))
            else:
                if not self._validate_record(key, tag, value_bytes, expiration_time):
                    response.store_ok.append(False)
                    continue
                if tag == self.IS_REGULAR_VALUE:
                    response.store_ok.append(storage.store(key_id, value_bytes, expiration_time))
                else:
                    subkey = self.serializer.loads(tag)
                    response.store_ok.append(storage.store_subkey(key_id, subkey, value_bytes, expiration_time))
        return response

    # ---------------------------------------------------------------------------------------------- find
    async def call_find(self, peer: PeerID, keys: Collection[DHTID]) -> Optional[
            Dict[DHTID, Tuple[Optional[ValueWithExpiration[Union[BinaryDHTValue, DictionaryDHTValue]]], Dict[DHTID, PeerID]]]]:
        """Ask ``peer`` for the values of ``keys`` and for its nearest known nodes to each key.

        :returns: ``{key: (value with expiration or None, {nearest node id: peer id})}``, or None if the call failed
        """
        keys = list(keys)
        find_request = dht_pb2.FindRequest(keys=[k.to_bytes() for k in keys], peer=self.node_info)
        try:
            async with self.rpc_semaphore:
                response = await self.get_stub(peer).rpc_find(find_request, timeout=self.wait_timeout)
            if response.peer and response.peer.node_id:
                peer_id = DHTID.from_bytes(response.peer.node_id)
                spawn(self.update_routing_table(peer_id, peer, responded=True))
            assert len(keys) == len(response.results), "DHTProtocol: response is not aligned with keys"
            output = {}
            for key_id, result in zip(keys, response.results):
                key_bytes = DHTID.to_bytes(key_id)
                nearest = dict(zip(map(DHTID.from_bytes, result.nearest_node_ids),
                                   (PeerID.from_base58(p.decode("ascii")) for p in result.nearest_peer_ids)))
                if result.type == dht_pb2.NOT_FOUND:
                    output[key_id] = None, nearest
                elif result.type == dht_pb2.FOUND_REGULAR:
                    if not self._validate_record(key_bytes, self.IS_REGULAR_VALUE, result.value, result.expiration_time):
                        output[key_id] = None, nearest
                        continue
                    output[key_id] = ValueWithExpiration(result.value, result.expiration_time), nearest
                elif result.type == dht_pb2.FOUND_DICTIONARY:
                    value_dictionary = self.serializer.loads(result.value)
                    if not self._validate_dictionary(key_bytes, value_dictionary):
                        output[key_id] = None, nearest
                        continue
                    output[key_id] = ValueWithExpiration(value_dictionary, result.expiration_time), nearest
                else:
                    logger.error(f"unknown result type: {result.type}")
            return output
        except Exception as e:
            logger.debug(f"DHTProtocol failed to find at {peer}: {e!r}")
            spawn(self.update_routing_table(self.routing_table.get(peer_id=peer), peer, responded=False))
            return None

    async def rpc_find(self, request: dht_pb2.FindRequest, context: P2PContext) -> dht_pb2.FindResponse:
        if request.peer and request.peer.node_id:
            spawn(self.update_routing_table(DHTID.from_bytes(request.peer.node_id), context.remote_id))
        response = dht_pb2.FindResponse(results=[], peer=self.node_info)
        for i, key_id in enumerate(map(DHTID.from_bytes, request.keys)):
            maybe_item = self.storage.get(key_id)
            cached_item = self.cache.get(key_id)
            if cached_item is not None and (maybe_item is None or cached_item.expiration_time > maybe_item.expiration_time):
                maybe_item = cached_item
            if maybe_item is None:
                item = dht_pb2.FindResult(type=dht_pb2.NOT_FOUND)
            elif isinstance(maybe_item.value, DictionaryDHTValue):
                item = dht_pb2.FindResult(type=dht_pb2.FOUND_DICTIONARY, value=self.serializer.dumps(maybe_item.value),
                                          expiration_time=maybe_item.expiration_time)
            else:
                item = dht_pb2.FindResult(type=dht_pb2.FOUND_REGULAR, value=maybe_item.value,
                                          expiration_time=maybe_item.expiration_time)
            sender = DHTID.from_bytes(request.peer.node_id) if request.peer and request.peer.node_id else None
            for node_id, peer_id in self.routing_table.get_nearest_neighbors(key_id, k=self.bucket_size, exclude=sender):
                item.nearest_node_ids.append(node_id.to_bytes())
                item.nearest_peer_ids.append(peer_id.to_base58().encode("ascii"))
            response.results.append(item)
        return response

    # ---------------------------------------------------------------------------------------------- routing upkeep
    async def update_routing_table(self, node_id: Optional[DHTID], peer_id: PeerID, responded: bool = True) -> None:
        """Record that ``peer_id`` answered (or failed to). New nodes receive the keys they are now nearest to."""
        node_id = node_id if node_id is not None else self.routing_table.get(peer_id=peer_id)
        if responded:
            if node_id is None:
                return
            if node_id not in self.routing_table:
                data_to_send: List[Tuple[DHTID, BinaryDHTValue, DHTExpiration]] = []
                for key, item in list(self.storage.items()):
                    neighbors = self.routing_table.get_nearest_neighbors(key, self.num_replicas, exclude=self.node_id)
                    if neighbors:
                        nearest_distance = neighbors[0][0].xor_distance(key)
                        farthest_distance = neighbors[-1][0].xor_distance(key)
                        new_node_should_store = node_id.xor_distance(key) < farthest_distance
                        this_node_is_responsible = self.node_id.xor_distance(key) < nearest_distance
                    if not neighbors or (new_node_should_store and this_node_is_responsible):
                        data_to_send.append((key, item.value, item.expiration_time))
                if data_to_send:
                    spawn(self.call_store(peer_id, *zip(*data_to_send), in_cache=False))
            maybe_node_to_ping = self.routing_table.add_or_update_node(node_id, peer_id)
            if maybe_node_to_ping is not None:
                # the bucket is full: check whether its least-recently-seen node is still there
                spawn(self.call_ping(maybe_node_to_ping[1]))
        else:
            if node_id is not None and node_id in self.routing_table:
                del self.routing_table[node_id]

    def _validate_record(self, key_bytes: bytes, subkey_bytes: bytes, value_bytes: bytes, expiration_time: float) -> bool:
        if self.record_validator is None:
            return True
        return self.record_validator.validate(DHTRecord(key_bytes, subkey_bytes, value_bytes, expiration_time))

    def _validate_dictionary(self, key_bytes: bytes, dictionary: DictionaryDHTValue) -> bool:
        if self.record_validator is None:
            return True
        with dictionary.freeze():
            for subkey, (value_bytes, expiration_time) in dictionary.items():
                subkey_bytes = self.serializer.dumps(subkey)
                if not self.record_validator.validate(DHTRecord(key_bytes, subkey_bytes, value_bytes, expiration_time)):
                    return False
        return True

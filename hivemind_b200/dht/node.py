"""``DHTNode``: one participant of the distributed hash table (asyncio, lives inside the DHT thread).

Behaviour follows the reference node (hivemind/dht/node.py:45-937): ``store_many`` finds the ``num_replicas``
nearest nodes to each key and stores there (and locally when this node is among the nearest); ``get_many`` answers
from local storage / cache when the entry is fresh enough and otherwise traverses the DHT, merging dictionary
values from every visited node; unresponsive peers are black-listed with exponential back-off; results can be
cached locally and on the nearest node that did not have them; concurrent gets for one key share a single search.
"""
from __future__ import annotations

import asyncio
import dataclasses
import os
import random
from collections import defaultdict
from dataclasses import dataclass, field
from functools import partial
from typing import (Any, Awaitable, Callable, Collection, DefaultDict, Dict, Iterable, List, Optional, Sequence, Set,
                    Tuple, Type, Union)

from sortedcontainers import SortedSet

from hivemind_b200.utils.asyncio import spawn
from hivemind_b200.dht.crypto import DHTRecord, RecordValidatorBase
from hivemind_b200.dht.protocol import DHTProtocol
from hivemind_b200.dht.routing import BinaryDHTValue, DHTID, DHTKey, DHTValue, Subkey
from hivemind_b200.dht.storage import DictionaryDHTValue
from hivemind_b200.dht.traverse import traverse_dht
from hivemind_b200.p2p import P2P, PeerID
from hivemind_b200.utils import MSGPackSerializer, SerializerBase, get_logger
from hivemind_b200.utils.auth import AuthorizerBase
from hivemind_b200.utils.multiaddr import Multiaddr
from hivemind_b200.utils.timed_storage import DHTExpiration, TimedStorage, ValueWithExpiration, get_dht_time

logger = get_logger(__name__)
DEFAULT_NUM_WORKERS = int(os.getenv("HIVEMIND_DHT_NUM_WORKERS", 4))


class Blacklist:
    """Peers that failed to respond are skipped for ``base_time * backoff_rate ** (failures - 1)`` seconds."""

    def __init__(self, base_time: float, backoff_rate: float, **kwargs):
        self.base_time, self.backoff = base_time, backoff_rate
        self.banned_peers = TimedStorage[PeerID, int](**kwargs)
        self.ban_counter: DefaultDict[PeerID, int] = defaultdict(int)

    def register_failure(self, peer: PeerID) -> None:
        if peer not in self.banned_peers and self.base_time > 0:
            ban_duration = self.base_time * self.backoff ** self.ban_counter[peer]
            self.banned_peers.store(peer, self.ban_counter[peer], expiration_time=get_dht_time() + ban_duration)
            self.ban_counter[peer] += 1

    def register_success(self, peer: PeerID) -> None:
        del self.banned_peers[peer]
        self.ban_counter.pop(peer, None)

    def __contains__(self, peer: PeerID) -> bool:
        return peer in self.banned_peers

    def clear(self) -> None:
        self.banned_peers.clear()
        self.ban_counter.clear()

    def __repr__(self) -> str:
        return (f"{type(self).__name__}(base_time={self.base_time}, backoff={self.backoff}, "
                f"banned_peers={len(self.banned_peers)})")


class CacheRefreshQueue(TimedStorage[DHTID, DHTExpiration]):
    """Keys whose cached value should be re-fetched shortly before it expires."""

    frozen = True


@dataclass(init=True, repr=True, frozen=False, order=False)
class _SearchState:
    """Progress of one get request: the freshest value seen so far and who is waiting for it."""

    key_id: DHTID
    sufficient_expiration_time: DHTExpiration
    binary_value: Optional[Union[BinaryDHTValue, DictionaryDHTValue]] = None
    expiration_time: Optional[DHTExpiration] = None
    source_node_id: Optional[DHTID] = None
    future: asyncio.Future = field(default_factory=lambda: asyncio.get_event_loop().create_future())
    serializer: Type[SerializerBase] = MSGPackSerializer
    record_validator: Optional[RecordValidatorBase] = None

    def add_candidate(self, candidate: Optional[ValueWithExpiration[Union[BinaryDHTValue, DictionaryDHTValue]]],
                      source_node_id: Optional[DHTID]) -> None:
        if self.finished or candidate is None:
            return
        elif isinstance(candidate.value, DictionaryDHTValue) and isinstance(self.binary_value, DictionaryDHTValue):
            self.binary_value.maxsize = max(self.binary_value.maxsize, candidate.value.maxsize)
            for subkey, subentry in candidate.value.items():
                self.binary_value.store(subkey, subentry.value, subentry.expiration_time)
        elif candidate.expiration_time > (self.expiration_time or float("-inf")):
            self.binary_value = candidate.value
        if candidate.expiration_time > (self.expiration_time or float("-inf")):
            self.expiration_time = candidate.expiration_time
            self.source_node_id = source_node_id
            if self.expiration_time >= self.sufficient_expiration_time:
                self.finish_search()

    def add_done_callback(self, callback: Callable[["_SearchState"], Any]) -> None:
        self.future.add_done_callback(lambda _future: callback(self))

    def finish_search(self) -> None:
        if self.future.done():
            return
        elif not self.found_something:
            self.future.set_result(None)
        elif isinstance(self.binary_value, BinaryDHTValue):
            value_bytes = self.binary_value
            if self.record_validator is not None:
                record = DHTRecord(self.key_id.to_bytes(), DHTProtocol.IS_REGULAR_VALUE, value_bytes, self.expiration_time)
                value_bytes = self.record_validator.strip_value(record)
            self.future.set_result(ValueWithExpiration(self.serializer.loads(value_bytes), self.expiration_time))
        elif isinstance(self.binary_value, DictionaryDHTValue):
            dict_with_subkeys = {}
            for subkey, (value_bytes, item_expiration_time) in self.binary_value.items():
                if self.record_validator is not None:
                    subkey_bytes = self.serializer.dumps(subkey)
                    record = DHTRecord(self.key_id.to_bytes(), subkey_bytes, value_bytes, item_expiration_time)
                    value_bytes = self.record_validator.strip_value(record)
                dict_with_subkeys[subkey] = ValueWithExpiration(self.serializer.loads(value_bytes), item_expiration_time)
            self.future.set_result(ValueWithExpiration(dict_with_subkeys, self.expiration_time))
        else:
            logger.error(f"invalid value type: {type(self.binary_value)}")

    @property
    def found_something(self) -> bool:
        return self.expiration_time is not None

    @property
    def finished(self) -> bool:
        return self.future.done()

    def __lt__(self, other: "_SearchState") -> bool:
        return self.sufficient_expiration_time < other.sufficient_expiration_time

    def __hash__(self) -> int:
        return hash(self.key_id)


class DHTNode:
    # fmt:off
    node_id: DHTID; is_alive: bool; peer_id: PeerID; num_replicas: int; num_workers: int; protocol: DHTProtocol
    chunk_size: int; refresh_timeout: float; cache_locally: bool; cache_nearest: int; cache_refresh_before_expiry: float
    cache_on_store: bool; reuse_get_requests: bool; pending_get_requests: DefaultDict[DHTID, SortedSet]
    cache_refresh_task: Optional[asyncio.Task]; cache_refresh_evt: asyncio.Event; cache_refresh_queue: CacheRefreshQueue
    blacklist: Blacklist
    # fmt:on

    @classmethod
    async def create(cls, p2p: Optional[P2P] = None, node_id: Optional[DHTID] = None,
                     initial_peers: Optional[Sequence[Union[Multiaddr, str]]] = None, bucket_size: int = 20,
                     num_replicas: int = 5, depth_modulo: int = 5, parallel_rpc: int = None, wait_timeout: float = 3,
                     refresh_timeout: Optional[float] = None, bootstrap_timeout: Optional[float] = None,
                     cache_locally: bool = True, cache_nearest: int = 1, cache_size=None,
                     cache_refresh_before_expiry: float = 5, cache_on_store: bool = True,
                     reuse_get_requests: bool = True, num_workers: int = DEFAULT_NUM_WORKERS, chunk_size: int = 16,
                     blacklist_time: float = 5.0, backoff_rate: float = 2.0, client_mode: bool = False,
                     record_validator: Optional[RecordValidatorBase] = None, authorizer: Optional[AuthorizerBase] = None,
                     ensure_bootstrap_success: bool = True, strict: bool = True, **kwargs) -> "DHTNode":
        """Create a node, start (or adopt) its transport and bootstrap from ``initial_peers``.

        Extra ``kwargs`` go to ``P2P.create`` when the node owns its transport. See the module docstring for the
        meaning of the caching and black-list options; defaults equal the reference's (node.py:99-128).
        """
        self = cls(_initialized_with_create=True)
        self.node_id = node_id if node_id is not None else DHTID.generate()
        self.num_replicas, self.num_workers, self.chunk_size = num_replicas, num_workers, chunk_size
        self.is_alive = True
        self.reuse_get_requests = reuse_get_requests
        self.pending_get_requests = defaultdict(partial(SortedSet, key=lambda _res: -_res.sufficient_expiration_time))
        self.refresh_timeout = refresh_timeout
        self.cache_locally, self.cache_nearest, self.cache_on_store = cache_locally, cache_nearest, cache_on_store
        self.cache_refresh_before_expiry = cache_refresh_before_expiry
        self.blacklist = Blacklist(blacklist_time, backoff_rate)
        self.cache_refresh_queue = CacheRefreshQueue()
        self.cache_refresh_evt = asyncio.Event()
        self.cache_refresh_task = None

        if p2p is None:
            if not kwargs.get("use_ipfs"):
                kwargs["initial_peers"] = initial_peers
            p2p = await P2P.create(**kwargs)
            self._should_shutdown_p2p = True
        else:
            if kwargs:
                raise ValueError(f"**kwargs in DHTNode.create() should be empty if a P2P instance is provided, got {kwargs}")
            self._should_shutdown_p2p = False
        self.p2p = p2p
        self.protocol = await DHTProtocol.create(p2p, self.node_id, bucket_size, depth_modulo, num_replicas, wait_timeout,
                                                 parallel_rpc, cache_size, client_mode, record_validator, authorizer)
        self.peer_id = p2p.peer_id

        if initial_peers:
            initial_peers = {PeerID.from_base58(Multiaddr(item)["p2p"]) for item in initial_peers}
            bootstrap_timeout = bootstrap_timeout if bootstrap_timeout is not None else wait_timeout
            start_time = get_dht_time()
            ping_tasks = set(asyncio.create_task(self.protocol.call_ping(peer, validate=ensure_bootstrap_success, strict=strict))
                             for peer in initial_peers)
            finished_pings, unfinished_pings = await asyncio.wait(ping_tasks, return_when=asyncio.FIRST_COMPLETED)
            if unfinished_pings:  # give the stragglers what is left of the bootstrap budget
                finished_in_time, stragglers = await asyncio.wait(
                    unfinished_pings, timeout=max(0.0, bootstrap_timeout - get_dht_time() + start_time))
                for straggler in stragglers:
                    straggler.cancel()
                finished_pings |= finished_in_time
            if not finished_pings or all(ping.exception() is None and ping.result() is None for ping in finished_pings):
                message = "DHTNode bootstrap failed: none of the initial_peers responded to the ping."
                if ensure_bootstrap_success:
                    raise RuntimeError(f"{message} (set ensure_bootstrap_success=False to ignore)")
                logger.warning(message)
            if strict:
                for task in asyncio.as_completed(finished_pings):
                    await task  # propagate validation errors
            # populate the routing table by looking for our own id
            await asyncio.wait([asyncio.create_task(self.find_nearest_nodes([self.node_id])),
                                asyncio.create_task(asyncio.sleep(bootstrap_timeout - get_dht_time() + start_time))],
                               return_when=asyncio.FIRST_COMPLETED)
        if self.refresh_timeout is not None:
            spawn(self._refresh_routing_table(period=self.refresh_timeout))
        return self

    def __init__(self, *, _initialized_with_create: bool = False):
        assert _initialized_with_create, "use `await DHTNode.create(...)`"
        super().__init__()

    async def shutdown(self) -> None:
        self.is_alive = False
        if self.cache_refresh_task is not None:
            self.cache_refresh_task.cancel()
        await self.protocol.shutdown()
        if self._should_shutdown_p2p:
            await self.p2p.shutdown()

    # ---------------------------------------------------------------------------------------------- find nodes
    async def find_nearest_nodes(self, queries: Collection[DHTID], k_nearest: Optional[int] = None,
                                 beam_size: Optional[int] = None, num_workers: Optional[int] = None,
                                 node_to_peer_id: Optional[Dict[DHTID, PeerID]] = None, exclude_self: bool = False,
                                 **kwargs) -> Dict[DHTID, Dict[DHTID, PeerID]]:
        """For every query id, the ``k_nearest`` nodes of the whole DHT nearest to it: ``{query: {node: peer}}``."""
        queries = tuple(queries)
        k_nearest = k_nearest if k_nearest is not None else self.protocol.bucket_size
        num_workers = num_workers if num_workers is not None else self.num_workers
        beam_size = beam_size if beam_size is not None else max(self.protocol.bucket_size, k_nearest)
        if k_nearest > beam_size:
            logger.warning("beam_size is too small: the search may miss some of the nearest nodes")
        if node_to_peer_id is None:
            node_to_peer_id = {}
            for query in queries:
                neighbors = self.protocol.routing_table.get_nearest_neighbors(query, beam_size, exclude=self.node_id)
                node_to_peer_id.update(self._filter_blacklisted(dict(neighbors)))

        async def get_neighbors(peer: DHTID, queries: Collection[DHTID]) -> Dict[DHTID, Tuple[Tuple[DHTID], bool]]:
            response = await self._call_find_with_blacklist(node_to_peer_id[peer], queries)
            if not response:
                return {query: ([], False) for query in queries}
            output: Dict[DHTID, Tuple[Tuple[DHTID], bool]] = {}
            for query, (_, peers) in response.items():
                node_to_peer_id.update(peers)
                output[query] = tuple(peers.keys()), False  # False: keep searching
            return output

        nearest_nodes_per_query, visited_nodes = await traverse_dht(
            queries, initial_nodes=list(node_to_peer_id), beam_size=beam_size, num_workers=num_workers,
            queries_per_call=int(len(queries) ** 0.5), get_neighbors=get_neighbors,
            visited_nodes={query: {self.node_id} for query in queries}, **kwargs)

        nearest_nodes_with_peer_ids = {}
        for query, nearest_nodes in nearest_nodes_per_query.items():
            if not exclude_self:
                nearest_nodes = sorted(nearest_nodes + [self.node_id], key=query.xor_distance)
                node_to_peer_id[self.node_id] = self.peer_id
            nearest_nodes_with_peer_ids[query] = {node: node_to_peer_id[node] for node in nearest_nodes[:k_nearest]}
        return nearest_nodes_with_peer_ids

    # ---------------------------------------------------------------------------------------------- store
    async def store(self, key: DHTKey, value: DHTValue, expiration_time: DHTExpiration,
                    subkey: Optional[Subkey] = None, **kwargs) -> bool:
        """Store one (key, [subkey,] value); True if at least one replica accepted it."""
        store_ok = await self.store_many([key], [value], [expiration_time], subkeys=[subkey], **kwargs)
        return store_ok[(key, subkey) if subkey is not None else key]

    async def store_many(self, keys: List[DHTKey], values: List[DHTValue],
                         expiration_time: Union[DHTExpiration, List[DHTExpiration]],
                         subkeys: Optional[Union[Subkey, List[Optional[Subkey]]]] = None, exclude_self: bool = False,
                         await_all_replicas=True, **kwargs) -> Dict[DHTKey, bool]:
        """Store several records at once; returns ``{key or (key, subkey): stored on at least one node}``."""
        if isinstance(expiration_time, DHTExpiration):
            expiration_time = [expiration_time] * len(keys)
        if subkeys is None:
            subkeys = [None] * len(keys)
        assert len(keys) == len(subkeys) == len(values) == len(expiration_time), "inputs must have equal lengths"

        key_id_to_data: DefaultDict[DHTID, List[Tuple[DHTKey, Subkey, DHTValue, DHTExpiration]]] = defaultdict(list)
        for key, subkey, value, expiration in zip(keys, subkeys, values, expiration_time):
            key_id_to_data[DHTID.generate(source=key)].append((key, subkey, value, expiration))

        unfinished_key_ids = set(key_id_to_data.keys())
        store_ok = {(key, subkey): None for key, subkey in zip(keys, subkeys)}
        store_finished_events = {(key, subkey): asyncio.Event() for key, subkey in zip(keys, subkeys)}

        node_to_peer_id: Dict[DHTID, PeerID] = dict()
        for key_id in unfinished_key_ids:
            node_to_peer_id.update(self.protocol.routing_table.get_nearest_neighbors(
                key_id, self.protocol.bucket_size, exclude=self.node_id))

        async def on_found(key_id: DHTID, nearest_nodes: List[DHTID], visited_nodes: Set[DHTID]) -> None:
            """The nearest nodes to ``key_id`` are known: send store requests to them."""
            assert key_id in unfinished_key_ids, "internal error: traverse_dht finished the same query twice"
            assert self.node_id not in nearest_nodes
            unfinished_key_ids.remove(key_id)

            num_successful_stores = 0
            pending_store_tasks = set()
            store_candidates = sorted(nearest_nodes + ([] if exclude_self else [self.node_id]),
                                      key=key_id.xor_distance, reverse=True)  # pop() takes the nearest
            [original_key, *_], current_subkeys, current_values, current_expirations = zip(*key_id_to_data[key_id])

            key_bytes = key_id.to_bytes()
            binary_values = []
            stored_records = []
            for subkey, value, expiration in zip(current_subkeys, current_values, current_expirations):
                subkey_bytes = self.protocol.serializer.dumps(subkey)
                value_bytes = self.protocol.serializer.dumps(value)
                if self.protocol.record_validator is not None:
                    if subkey is None:
                        subkey_bytes = self.protocol.IS_REGULAR_VALUE
                    record = DHTRecord(key_bytes, subkey_bytes, value_bytes, expiration)
                    value_bytes = self.protocol.record_validator.sign_value(record)
                binary_values.append(value_bytes)
                stored_records.append((subkey, value_bytes, expiration))

            while num_successful_stores < self.num_replicas and (store_candidates or pending_store_tasks):
                while store_candidates and num_successful_stores + len(pending_store_tasks) < self.num_replicas:
                    node_id: DHTID = store_candidates.pop()
                    if node_id == self.node_id:
                        num_successful_stores += 1
                        for subkey, value_bytes, expiration in stored_records:
                            if self.protocol.record_validator is not None:
                                subkey_bytes = self.protocol.IS_REGULAR_VALUE if subkey is None else self.protocol.serializer.dumps(subkey)
                                if not self.protocol.record_validator.validate(DHTRecord(key_bytes, subkey_bytes, value_bytes, expiration)):
                                    store_ok[original_key, subkey] = False
                                    store_finished_events[original_key, subkey].set()
                                    continue
                            store_ok[original_key, subkey] = self.protocol.storage.store(
                                key_id, value_bytes, expiration, subkey=subkey)
                            if not await_all_replicas:
                                store_finished_events[original_key, subkey].set()
                    else:
                        pending_store_tasks.add(asyncio.create_task(self.protocol.call_store(
                            node_to_peer_id[node_id], keys=[key_id] * len(current_values), values=binary_values,
                            expiration_time=current_expirations, subkeys=current_subkeys)))

                if pending_store_tasks:
                    finished_store_tasks, pending_store_tasks = await asyncio.wait(
                        pending_store_tasks, return_when=asyncio.FIRST_COMPLETED)
                    for task in finished_store_tasks:
                        if task.result() is not None:
                            num_successful_stores += 1
                            for subkey, store_status in zip(current_subkeys, task.result()):
                                store_ok[original_key, subkey] = store_status or store_ok[original_key, subkey]
                                if not await_all_replicas:
                                    store_finished_events[original_key, subkey].set()

            if self.cache_on_store:
                self._update_cache_on_store(key_id, current_subkeys, binary_values, current_expirations,
                                            store_ok=[store_ok[original_key, subkey] for subkey in current_subkeys])
            for subkey, value_bytes, expiration in stored_records:
                store_finished_events[original_key, subkey].set()

        store_task = asyncio.create_task(self.find_nearest_nodes(
            queries=set(unfinished_key_ids), k_nearest=self.num_replicas, node_to_peer_id=node_to_peer_id,
            found_callback=on_found, exclude_self=exclude_self, **kwargs))
        try:
            await asyncio.gather(store_task, *(evt.wait() for evt in store_finished_events.values()))
            assert len(unfinished_key_ids) == 0, "internal error: traverse_dht did not finish the search"
            return {(key, subkey) if subkey is not None else key: status or False
                    for (key, subkey), status in store_ok.items()}
        except asyncio.CancelledError as e:
            store_task.cancel()
            raise e

    def _update_cache_on_store(self, key_id: DHTID, subkeys: List[Subkey], binary_values: List[bytes],
                               expirations: List[DHTExpiration], store_ok: List[bool]) -> None:
        """A successful store also refreshes our own cached copy of the key (or invalidates a stale one)."""
        for subkey, value_bytes, expiration_time, accepted in zip(subkeys, binary_values, expirations, store_ok):
            if accepted:
                self.protocol.cache.store(key_id, value_bytes, expiration_time, subkey=subkey)
                self._schedule_for_refresh(key_id, expiration_time)
            else:
                rejected_value, rejected_expiration = self.protocol.cache.get(key_id) or (None, None)
                if rejected_value is not None and subkey is None and rejected_expiration <= expiration_time:
                    del self.protocol.cache[key_id]  # somebody holds a newer value: ours is stale

    # ---------------------------------------------------------------------------------------------- get
    async def get(self, key: DHTKey, latest=False, **kwargs) -> Optional[ValueWithExpiration[DHTValue]]:
        """The value under ``key`` (a dict of sub-key -> ValueWithExpiration for dictionaries) or None.

        :param latest: visit all nearest nodes and return the freshest value instead of stopping at the first hit
        """
        if latest:
            kwargs["sufficient_expiration_time"] = float("inf")
        result = await self.get_many([key], **kwargs)
        return result[key]

    async def get_many(self, keys: Collection[DHTKey], sufficient_expiration_time: Optional[DHTExpiration] = None,
                       **kwargs) -> Dict[DHTKey, Union[Optional[ValueWithExpiration[DHTValue]],
                                                       Awaitable[Optional[ValueWithExpiration[DHTValue]]]]]:
        keys = tuple(keys)
        key_ids = [DHTID.generate(key) for key in keys]
        id_to_original_key = dict(zip(key_ids, keys))
        results_by_id = await self.get_many_by_id(key_ids, sufficient_expiration_time, **kwargs)
        return {id_to_original_key[key]: result_or_future for key, result_or_future in results_by_id.items()}

    async def get_many_by_id(self, key_ids: Collection[DHTID], sufficient_expiration_time: Optional[DHTExpiration] = None,
                             num_workers: Optional[int] = None, beam_size: Optional[int] = None,
                             return_futures: bool = False, _is_refresh=False
                             ) -> Dict[DHTID, Union[Optional[ValueWithExpiration[DHTValue]],
                                                    Awaitable[Optional[ValueWithExpiration[DHTValue]]]]]:
        """
        :param sufficient_expiration_time: stop as soon as a value expiring at or after this time is found
          (default: any unexpired value); ``float('inf')`` visits every nearest node
        :param return_futures: return ``{key: awaitable}`` immediately instead of waiting for all keys
        """
        sufficient_expiration_time = sufficient_expiration_time or get_dht_time()
        beam_size = beam_size if beam_size is not None else self.protocol.bucket_size
        num_workers = num_workers if num_workers is not None else self.num_workers
        search_results: Dict[DHTID, _SearchState] = {
            key_id: _SearchState(key_id, sufficient_expiration_time, serializer=self.protocol.serializer,
                                 record_validator=self.protocol.record_validator) for key_id in key_ids}

        if not _is_refresh:
            for key_id in key_ids:
                search_results[key_id].add_done_callback(self._trigger_cache_refresh)

        # if we have concurrent get request for some of the same keys, subscribe to their results
        if self.reuse_get_requests:
            for key_id, search_result in search_results.items():
                self.pending_get_requests[key_id].add(search_result)
                search_result.add_done_callback(self._reuse_finished_search_result)

        # stage 1: check local storage and cache
        for key_id in key_ids:
            search_results[key_id].add_candidate(self.protocol.storage.get(key_id), source_node_id=self.node_id)
            if not _is_refresh:
                search_results[key_id].add_candidate(self.protocol.cache.get(key_id), source_node_id=self.node_id)

        # stage 2: traverse the DHT for the keys that are still unfinished
        unfinished_key_ids = [key_id for key_id in key_ids if not search_results[key_id].finished]
        node_to_peer_id: Dict[DHTID, PeerID] = dict()
        for key_id in unfinished_key_ids:
            node_to_peer_id.update(self.protocol.routing_table.get_nearest_neighbors(
                key_id, self.protocol.bucket_size, exclude=self.node_id))
        node_to_peer_id = self._filter_blacklisted(node_to_peer_id)

        async def get_neighbors(peer: DHTID, queries: Collection[DHTID]) -> Dict[DHTID, Tuple[Tuple[DHTID], bool]]:
            queries = list(queries)
            response = await self._call_find_with_blacklist(node_to_peer_id[peer], queries)
            if not response:
                return {query: ([], False) for query in queries}
            output: Dict[DHTID, Tuple[Tuple[DHTID], bool]] = {}
            for key_id, (maybe_value_with_expiration, peers) in response.items():
                node_to_peer_id.update(self._filter_blacklisted(peers))
                search_results[key_id].add_candidate(maybe_value_with_expiration, source_node_id=peer)
                output[key_id] = tuple(peers.keys()), search_results[key_id].finished
            return output

        async def found_callback(key_id: DHTID, nearest_nodes: List[DHTID], _visited: Set[DHTID]):
            search_results[key_id].finish_search()  # finish with whatever we have (possibly nothing)
            self._cache_new_result(search_results[key_id], nearest_nodes, node_to_peer_id, _is_refresh=_is_refresh)

        spawn(traverse_dht(
            queries=list(unfinished_key_ids), initial_nodes=list(node_to_peer_id), beam_size=beam_size,
            num_workers=num_workers, queries_per_call=min(int(len(unfinished_key_ids) ** 0.5), self.chunk_size),
            get_neighbors=get_neighbors, visited_nodes={key_id: {self.node_id} for key_id in unfinished_key_ids},
            found_callback=found_callback, await_all_tasks=False))

        if return_futures:
            return {key_id: search_result.future for key_id, search_result in search_results.items()}
        try:
            return {key_id: await search_result.future for key_id, search_result in search_results.items()}
        except asyncio.CancelledError as e:
            for key_id, search_result in search_results.items():
                search_result.future.cancel()
            raise e

    def _reuse_finished_search_result(self, finished: _SearchState) -> None:
        pending_requests = self.pending_get_requests[finished.key_id]
        if finished.found_something:
            search_result = ValueWithExpiration(finished.binary_value, finished.expiration_time)
            expiration_time_threshold = max(finished.expiration_time, finished.sufficient_expiration_time)
            # share the result with requests that would be satisfied by it
            while pending_requests and expiration_time_threshold >= pending_requests[-1].sufficient_expiration_time:
                pending_requests[-1].add_candidate(search_result, source_node_id=finished.source_node_id)
                pending_requests[-1].finish_search()
                pending_requests.pop()
        else:
            pending_requests.discard(finished)

    async def _call_find_with_blacklist(self, peer_id: PeerID, keys: Collection[DHTID]):
        """Like ``protocol.call_find`` but skips banned peers and bans the ones that fail."""
        if peer_id in self.blacklist:
            return None
        response = await self.protocol.call_find(peer_id, keys)
        if response:
            self.blacklist.register_success(peer_id)
            return {key: (maybe_value, self._filter_blacklisted(nearest_peers))
                    for key, (maybe_value, nearest_peers) in response.items()}
        self.blacklist.register_failure(peer_id)
        return None

    def _filter_blacklisted(self, peer_ids: Dict[DHTID, PeerID]) -> Dict[DHTID, PeerID]:
        return {key: peer for key, peer in peer_ids.items() if peer not in self.blacklist}

    # ---------------------------------------------------------------------------------------------- cache upkeep
    def _trigger_cache_refresh(self, search: _SearchState) -> None:
        """A value that came from our cache is scheduled for a background refresh before it expires."""
        if search.found_something and search.source_node_id == self.node_id:
            if self.cache_refresh_before_expiry and search.key_id in self.protocol.cache:
                self._schedule_for_refresh(search.key_id, search.expiration_time)

    def _schedule_for_refresh(self, key_id: DHTID, expiration_time: DHTExpiration) -> None:
        if self.cache_refresh_before_expiry is None or self.cache_refresh_before_expiry <= 0:
            return
        if self.cache_refresh_task is None or self.cache_refresh_task.done() or self.cache_refresh_task.cancelled():
            self.cache_refresh_task = asyncio.create_task(self._refresh_stale_cache_entries())
            logger.debug("spawned cache refresh task")
        earliest_key, earliest_item = self.cache_refresh_queue.top() or (None, None)
        if earliest_item is None or expiration_time < earliest_item.expiration_time:
            self.cache_refresh_evt.set()  # the refresher re-computes its wake-up time
        self.cache_refresh_queue.store(key_id, value=expiration_time, expiration_time=expiration_time)

    async def _refresh_stale_cache_entries(self) -> None:
        """Background task: shortly before a cached entry expires, look the key up again with a later horizon."""
        while self.is_alive:
            while len(self.cache_refresh_queue) == 0:
                await self.cache_refresh_evt.wait()
                self.cache_refresh_evt.clear()
            key_id, (_, nearest_refresh_time) = self.cache_refresh_queue.top()
            try:
                # wake up earlier if a more urgent entry arrives
                time_to_wait = nearest_refresh_time - self.cache_refresh_before_expiry - get_dht_time()
                await asyncio.wait_for(self.cache_refresh_evt.wait(), timeout=time_to_wait)
                self.cache_refresh_evt.clear()
                continue
            except asyncio.TimeoutError:
                current_time = get_dht_time()
                keys_to_refresh = {key_id}
                max_expiration_time = nearest_refresh_time
                del self.cache_refresh_queue[key_id]
                while self.cache_refresh_queue and len(keys_to_refresh) < self.chunk_size:
                    key_id, (_, nearest_refresh_time) = self.cache_refresh_queue.top()
                    if nearest_refresh_time > current_time + self.cache_refresh_before_expiry:
                        break
                    del self.cache_refresh_queue[key_id]
                    keys_to_refresh.add(key_id)
                    max_expiration_time = max(max_expiration_time, nearest_refresh_time)
                sufficient_expiration_time = max_expiration_time + self.cache_refresh_before_expiry + 1
                await self.get_many_by_id(keys_to_refresh, sufficient_expiration_time, _is_refresh=True)

    def _cache_new_result(self, search: _SearchState, nearest_nodes: List[DHTID],
                          node_to_peer_id: Dict[DHTID, PeerID], _is_refresh: bool = False) -> None:
        """After a successful search: cache locally and on the nearest nodes that did not have the value."""
        if search.found_something:
            _, storage_expiration_time = self.protocol.storage.get(search.key_id) or (None, -float("inf"))
            _, cache_expiration_time = self.protocol.cache.get(search.key_id) or (None, -float("inf"))
            if search.expiration_time > max(storage_expiration_time, cache_expiration_time):
                if self.cache_locally or _is_refresh:
                    self.protocol.cache.store(search.key_id, search.binary_value, search.expiration_time)
                if self.cache_nearest:
                    num_cached_nodes = 0
                    for node_id in nearest_nodes:
                        if node_id == search.source_node_id:
                            continue
                        spawn(self.protocol.call_store(
                            node_to_peer_id[node_id], [search.key_id], [search.binary_value], [search.expiration_time],
                            in_cache=True))
                        num_cached_nodes += 1
                        if num_cached_nodes >= self.cache_nearest:
                            break

    async def _refresh_routing_table(self, *, period: Optional[float]) -> None:
        """Periodically look up a random id inside every bucket that has not been touched for ``period`` seconds."""
        while self.is_alive and period is not None:
            refresh_time = get_dht_time()
            staleness_threshold = refresh_time - period
            stale_buckets = [bucket for bucket in self.protocol.routing_table.buckets
                             if bucket.last_updated < staleness_threshold]
            for bucket in stale_buckets:
                refresh_id = DHTID(random.randint(bucket.lower, bucket.upper - 1))
                await self.find_nearest_nodes([refresh_id])
            await asyncio.sleep(max(0.0, period - (get_dht_time() - refresh_time)))

    async def get_visible_maddrs(self, latest: bool = False) -> List[Multiaddr]:
        return await self.protocol.p2p.get_visible_maddrs(latest=latest)

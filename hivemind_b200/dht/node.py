"""``DHTNode``: one participant of the distributed hash table (asyncio, lives inside the DHT thread).

Behaviour contract (hivemind/dht/node.py:45-937): ``store_many`` finds the ``num_replicas`` nodes nearest to each key
and stores there (and locally when this node is among them); ``get_many`` answers from local storage / cache when the
entry is fresh enough and otherwise traverses the DHT, merging dictionary values from every node it visits;
unresponsive peers are skipped for a while with exponential back-off; results can be cached locally and on the
nearest node that did not have them; concurrent gets for one key share what any of them finds; cached entries that
were used are re-fetched shortly before they expire.

Decomposition used here: ``Blacklist`` (who not to ask), ``_Lookup`` (what one get request has collected for one
key), ``_Replication`` (placing the records of one key on replicas), ``_CacheRefresher`` (the queue and task that keep
used cache entries fresh) and ``DHTNode`` itself, which wires them to the protocol and to the graph traversal.
"""
from __future__ import annotations

import asyncio
import os
import random
from collections import defaultdict
from typing import Awaitable, Collection, Dict, Iterable, List, Optional, Sequence, Set, Tuple, Type, Union

from hivemind_b200.dht.crypto import DHTRecord, RecordValidatorBase
from hivemind_b200.dht.protocol import DHTProtocol
from hivemind_b200.dht.routing import BinaryDHTValue, DHTID, DHTKey, DHTValue, Subkey
from hivemind_b200.dht.storage import DictionaryDHTValue
from hivemind_b200.dht.traverse import traverse_dht
from hivemind_b200.p2p import P2P, PeerID
from hivemind_b200.utils import SerializerBase, get_logger
from hivemind_b200.utils.asyncio import spawn
from hivemind_b200.utils.auth import AuthorizerBase
from hivemind_b200.utils.multiaddr import Multiaddr
from hivemind_b200.utils.timed_storage import DHTExpiration, TimedStorage, ValueWithExpiration, get_dht_time

logger = get_logger(__name__)
DEFAULT_NUM_WORKERS = int(os.getenv("HIVEMIND_DHT_NUM_WORKERS", 4))
StoredPayload = Union[BinaryDHTValue, DictionaryDHTValue]
GetResult = Optional[ValueWithExpiration[DHTValue]]


class Blacklist:
    """Peers that did not answer are left alone for ``base_time * backoff_rate ** (earlier bans)`` seconds."""

    def __init__(self, base_time: float, backoff_rate: float, **storage_kwargs):
        self.base_time, self.backoff = base_time, backoff_rate
        self.banned_peers = TimedStorage[PeerID, int](**storage_kwargs)
        self.ban_counter: Dict[PeerID, int] = {}

    def register_failure(self, peer: PeerID) -> None:
        if self.base_time <= 0 or peer in self.banned_peers:
            return
        strikes = self.ban_counter.get(peer, 0)
        self.banned_peers.store(peer, strikes, expiration_time=get_dht_time() + self.base_time * self.backoff ** strikes)
        self.ban_counter[peer] = strikes + 1

    def register_success(self, peer: PeerID) -> None:
        del self.banned_peers[peer]
        self.ban_counter.pop(peer, None)

    def __contains__(self, peer: PeerID) -> bool:
        return peer in self.banned_peers

    def clear(self) -> None:
        self.banned_peers.clear()
        self.ban_counter.clear()

    def __repr__(self) -> str:
        return f"{type(self).__name__}(base_time={self.base_time}, backoff={self.backoff}, banned={len(self.banned_peers)})"


class _Lookup:
    """What one get request knows about one key so far: the freshest payload, where it came from, and the future
    that the caller awaits. ``horizon`` is the expiration time from which on a value is good enough to stop."""

    __slots__ = ("key_id", "horizon", "payload", "freshest", "origin", "future", "_serializer", "_validator")

    def __init__(self, key_id: DHTID, horizon: DHTExpiration, serializer: Type[SerializerBase],
                 validator: Optional[RecordValidatorBase]):
        self.key_id, self.horizon = key_id, horizon
        self.payload: Optional[StoredPayload] = None
        self.freshest: Optional[DHTExpiration] = None
        self.origin: Optional[DHTID] = None
        self.future: asyncio.Future = asyncio.get_event_loop().create_future()
        self._serializer, self._validator = serializer, validator

    @property
    def found_something(self) -> bool:
        return self.freshest is not None

    @property
    def finished(self) -> bool:
        return self.future.done()

    def offer(self, candidate: Optional[ValueWithExpiration[StoredPayload]], origin: Optional[DHTID]) -> None:
        """Take a payload reported by ``origin`` into account; dictionaries from different nodes are merged."""
        if candidate is None or self.future.done():
            return
        payload, expiration = candidate.value, candidate.expiration_time
        newer = self.freshest is None or expiration > self.freshest
        if isinstance(payload, DictionaryDHTValue) and isinstance(self.payload, DictionaryDHTValue):
            self.payload.maxsize = max(self.payload.maxsize, payload.maxsize)
            for subkey, entry in payload.items():
                self.payload.store(subkey, entry.value, entry.expiration_time)
        elif newer:
            self.payload = payload
        if newer:
            self.freshest, self.origin = expiration, origin
            if expiration >= self.horizon:
                self.settle()

    def settle(self) -> None:
        """Resolve the future with what has been collected (None if nothing was found)."""
        if self.future.done():
            return
        if not self.found_something:
            self.future.set_result(None)
        elif isinstance(self.payload, DictionaryDHTValue):
            decoded = {subkey: ValueWithExpiration(self._decode(self._serializer.dumps(subkey), raw, expiration), expiration)
                       for subkey, (raw, expiration) in self.payload.items()}
            self.future.set_result(ValueWithExpiration(decoded, self.freshest))
        elif isinstance(self.payload, BinaryDHTValue):
            value = self._decode(DHTProtocol.IS_REGULAR_VALUE, self.payload, self.freshest)
            self.future.set_result(ValueWithExpiration(value, self.freshest))
        else:
            logger.error(f"a DHT payload of unexpected type {type(self.payload)} was dropped")

    def _decode(self, subkey_bytes: bytes, raw: bytes, expiration: DHTExpiration) -> DHTValue:
        if self._validator is not None:
            raw = self._validator.strip_value(DHTRecord(self.key_id.to_bytes(), subkey_bytes, raw, expiration))
        return self._serializer.loads(raw)


class _CacheRefresher:
    """Keeps cache entries that were actually used from going stale: each is looked up again
    ``lead_time`` seconds before it expires, several at once when their deadlines are close."""

    def __init__(self, node: "DHTNode", lead_time: Optional[float]):
        self.node, self.lead_time = node, lead_time
        self.queue = TimedStorage[DHTID, DHTExpiration]()
        self.queue.frozen = True  # entries leave the queue only when this class removes them
        self._wake = asyncio.Event()
        self._task: Optional[asyncio.Task] = None

    @property
    def enabled(self) -> bool:
        return self.lead_time is not None and self.lead_time > 0

    def watch(self, key_id: DHTID, expiration: DHTExpiration) -> None:
        if not self.enabled:
            return
        if self._task is None or self._task.done():
            self._task = asyncio.create_task(self._run())
        head = self.queue.top()
        if head is None or expiration < head[1].expiration_time:
            self._wake.set()  # the task must recompute when to get up
        self.queue.store(key_id, value=expiration, expiration_time=expiration)

    def stop(self) -> None:
        if self._task is not None:
            self._task.cancel()

    async def _run(self) -> None:
        while self.node.is_alive:
            if len(self.queue) == 0:
                await self._wake.wait()
                self._wake.clear()
                continue
            key_id, (_, due) = self.queue.top()
            try:
                await asyncio.wait_for(self._wake.wait(), timeout=due - self.lead_time - get_dht_time())
                self._wake.clear()
                continue  # something more urgent may have arrived
            except asyncio.TimeoutError:
                pass
            now, batch, latest = get_dht_time(), {key_id}, due
            del self.queue[key_id]
            while self.queue and len(batch) < self.node.chunk_size:
                other, (_, other_due) = self.queue.top()
                if other_due > now + self.lead_time:
                    break
                del self.queue[other]
                batch.add(other)
                latest = max(latest, other_due)
            await self.node.get_many_by_id(batch, latest + self.lead_time + 1, _is_refresh=True)


class _Replication:
    """Places all records of one key id (one key, possibly several sub-keys) on ``num_replicas`` nodes."""

    def __init__(self, node: "DHTNode", key_id: DHTID, original_key: DHTKey,
                 records: List[Tuple[Subkey, DHTValue, DHTExpiration]], exclude_self: bool, first_reply_is_enough: bool):
        self.node, self.key_id, self.original_key = node, key_id, original_key
        self.exclude_self, self.first_reply_is_enough = exclude_self, first_reply_is_enough
        protocol = node.protocol
        self.subkeys = [subkey for subkey, _, _ in records]
        self.expirations = [expiration for _, _, expiration in records]
        self.wire_values: List[bytes] = []
        for subkey, value, expiration in records:
            raw = protocol.serializer.dumps(value)
            if protocol.record_validator is not None:
                raw = protocol.record_validator.sign_value(DHTRecord(key_id.to_bytes(), self._subkey_bytes(subkey), raw, expiration))
            self.wire_values.append(raw)
        self.accepted: Dict[Subkey, Optional[bool]] = {subkey: None for subkey in self.subkeys}
        self.reported = {subkey: asyncio.Event() for subkey in self.subkeys}

    def _subkey_bytes(self, subkey: Subkey) -> bytes:
        protocol = self.node.protocol
        return protocol.IS_REGULAR_VALUE if subkey is None else protocol.serializer.dumps(subkey)

    def _store_here(self) -> None:
        protocol = self.node.protocol
        for subkey, raw, expiration in zip(self.subkeys, self.wire_values, self.expirations):
            if protocol.record_validator is not None and not protocol.record_validator.validate(
                    DHTRecord(self.key_id.to_bytes(), self._subkey_bytes(subkey), raw, expiration)):
                self.accepted[subkey] = False
                self.reported[subkey].set()
                continue
            self.accepted[subkey] = protocol.storage.store(self.key_id, raw, expiration, subkey=subkey)
            if self.first_reply_is_enough:
                self.reported[subkey].set()

    def _absorb_reply(self, verdicts: Sequence[bool]) -> None:
        for subkey, verdict in zip(self.subkeys, verdicts):
            self.accepted[subkey] = verdict or self.accepted[subkey]
            if self.first_reply_is_enough:
                self.reported[subkey].set()

    async def run(self, nearest: List[DHTID], address_of: Dict[DHTID, PeerID]) -> None:
        """``nearest``: the nodes nearest to the key that the traversal found (never this node itself)."""
        node = self.node
        targets = list(nearest) if self.exclude_self else list(nearest) + [node.node_id]
        targets.sort(key=self.key_id.xor_distance)
        cursor, replicas, in_flight = 0, 0, set()
        while replicas < node.num_replicas and (cursor < len(targets) or in_flight):
            while cursor < len(targets) and replicas + len(in_flight) < node.num_replicas:
                target = targets[cursor]
                cursor += 1
                if target == node.node_id:
                    self._store_here()
                    replicas += 1
                else:
                    in_flight.add(asyncio.create_task(node.protocol.call_store(
                        address_of[target], keys=[self.key_id] * len(self.subkeys), values=self.wire_values,
                        expiration_time=self.expirations, subkeys=self.subkeys)))
            if in_flight:
                done, in_flight = await asyncio.wait(in_flight, return_when=asyncio.FIRST_COMPLETED)
                for task in done:
                    if task.result() is not None:
                        replicas += 1
                        self._absorb_reply(task.result())
        if node.cache_on_store:
            node._note_own_store(self.key_id, self.subkeys, self.wire_values, self.expirations,
                                 [self.accepted[subkey] for subkey in self.subkeys])
        for event in self.reported.values():
            event.set()


class DHTNode:
    # fmt:off
    node_id: DHTID; is_alive: bool; peer_id: PeerID; num_replicas: int; num_workers: int; protocol: DHTProtocol
    chunk_size: int; refresh_timeout: Optional[float]; cache_locally: bool; cache_nearest: int
    cache_refresh_before_expiry: float; cache_on_store: bool; reuse_get_requests: bool; blacklist: Blacklist
    # fmt:on

    def __init__(self, *, _initialized_with_create: bool = False):
        if not _initialized_with_create:
            raise RuntimeError("use `await DHTNode.create(...)`")

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
        meaning of the caching and black-list options; the defaults are the reference's (node.py:99-128).
        """
        self = cls(_initialized_with_create=True)
        self.node_id = DHTID.generate() if node_id is None else node_id
        self.num_replicas, self.num_workers, self.chunk_size = num_replicas, num_workers, chunk_size
        self.refresh_timeout, self.reuse_get_requests = refresh_timeout, reuse_get_requests
        self.cache_locally, self.cache_nearest, self.cache_on_store = cache_locally, cache_nearest, cache_on_store
        self.cache_refresh_before_expiry = cache_refresh_before_expiry
        self.blacklist = Blacklist(blacklist_time, backoff_rate)
        self._refresher = _CacheRefresher(self, cache_refresh_before_expiry)
        self._open_lookups: Dict[DHTID, List[_Lookup]] = defaultdict(list)
        self.is_alive = True

        self._owns_p2p = p2p is None
        if p2p is None:
            if not kwargs.get("use_ipfs"):
                kwargs["initial_peers"] = initial_peers
            p2p = await P2P.create(**kwargs)
        elif kwargs:
            raise ValueError(f"a P2P instance was given, so DHTNode.create() takes no transport options; got {kwargs}")
        self.p2p, self.peer_id = p2p, p2p.peer_id
        self.protocol = await DHTProtocol.create(p2p, self.node_id, bucket_size, depth_modulo, num_replicas, wait_timeout,
                                                 parallel_rpc, cache_size, client_mode, record_validator, authorizer)
        if initial_peers:
            budget = wait_timeout if bootstrap_timeout is None else bootstrap_timeout
            await self._bootstrap({PeerID.from_base58(Multiaddr(addr)["p2p"]) for addr in initial_peers}, budget,
                                  ensure_bootstrap_success, strict)
        if refresh_timeout is not None:
            spawn(self._keep_routing_table_fresh(refresh_timeout))
        return self

    async def _bootstrap(self, peers: Set[PeerID], budget: float, must_succeed: bool, strict: bool) -> None:
        """Ping the initial peers (the first answer unblocks us, the rest get what is left of ``budget``), then look
        for our own id so that the routing table fills up."""
        began = get_dht_time()
        pings = {asyncio.create_task(self.protocol.call_ping(peer, validate=must_succeed, strict=strict)) for peer in peers}
        answered, waiting = await asyncio.wait(pings, return_when=asyncio.FIRST_COMPLETED)
        if waiting:
            more, late = await asyncio.wait(waiting, timeout=max(0.0, began + budget - get_dht_time()))
            answered |= more
            for ping in late:
                ping.cancel()
        if all(ping.exception() is None and ping.result() is None for ping in answered):
            complaint = "DHTNode bootstrap failed: none of the initial_peers responded to the ping."
            if must_succeed:
                raise RuntimeError(f"{complaint} (set ensure_bootstrap_success=False to ignore)")
            logger.warning(complaint)
        if strict:
            for ping in answered:
                ping.result()  # a validation error of any initial peer is the caller's business
        remaining = max(0.0, began + budget - get_dht_time())
        with_deadline = asyncio.create_task(self.find_nearest_nodes([self.node_id]))
        await asyncio.wait([with_deadline], timeout=remaining)

    async def shutdown(self) -> None:
        self.is_alive = False
        self._refresher.stop()
        await self.protocol.shutdown()
        if self._owns_p2p:
            await self.p2p.shutdown()

    async def get_visible_maddrs(self, latest: bool = False) -> List[Multiaddr]:
        return await self.protocol.p2p.get_visible_maddrs(latest=latest)

    # ---------------------------------------------------------------------------------------------- asking peers
    def _without_banned(self, peers: Dict[DHTID, PeerID]) -> Dict[DHTID, PeerID]:
        if not self.blacklist.ban_counter:  # nobody has ever failed (or everybody has answered since)
            return peers
        return {node: peer for node, peer in peers.items() if peer not in self.blacklist}

    def _routing_neighbours(self, key_ids: Iterable[DHTID], count: int) -> Dict[DHTID, PeerID]:
        known: Dict[DHTID, PeerID] = {}
        for key_id in key_ids:
            known.update(self.protocol.routing_table.get_nearest_neighbors(key_id, count, exclude=self.node_id))
        return known

    async def _ask(self, peer: PeerID, key_ids: Collection[DHTID]):
        """``protocol.call_find`` that respects and feeds the black list; None if the peer is banned or silent."""
        if peer in self.blacklist:
            return None
        reply = await self.protocol.call_find(peer, key_ids)
        if not reply:
            self.blacklist.register_failure(peer)
            return None
        self.blacklist.register_success(peer)
        return {key_id: (payload, self._without_banned(neighbours)) for key_id, (payload, neighbours) in reply.items()}

    # ---------------------------------------------------------------------------------------------- find nodes
    async def find_nearest_nodes(self, queries: Collection[DHTID], k_nearest: Optional[int] = None,
                                 beam_size: Optional[int] = None, num_workers: Optional[int] = None,
                                 node_to_peer_id: Optional[Dict[DHTID, PeerID]] = None, exclude_self: bool = False,
                                 **kwargs) -> Dict[DHTID, Dict[DHTID, PeerID]]:
        """For every query id, the ``k_nearest`` nodes of the whole DHT nearest to it: ``{query: {node: peer}}``."""
        queries = tuple(queries)
        k_nearest = self.protocol.bucket_size if k_nearest is None else k_nearest
        num_workers = self.num_workers if num_workers is None else num_workers
        beam_size = max(self.protocol.bucket_size, k_nearest) if beam_size is None else beam_size
        if k_nearest > beam_size:
            logger.warning("beam_size is smaller than k_nearest: some of the nearest nodes may be missed")
        address_of = node_to_peer_id
        if address_of is None:
            address_of = self._without_banned(self._routing_neighbours(queries, beam_size))

        async def visit(node: DHTID, asked: Collection[DHTID]) -> Dict[DHTID, Tuple[Tuple[DHTID], bool]]:
            reply = await self._ask(address_of[node], asked)
            if reply is None:
                return {query: ((), False) for query in asked}
            hops = {}
            for query, (_, neighbours) in reply.items():
                address_of.update(neighbours)
                hops[query] = (tuple(neighbours), False)  # False: this never ends a search early
            return hops

        found, _ = await traverse_dht(
            queries, initial_nodes=list(address_of), beam_size=beam_size, num_workers=num_workers,
            queries_per_call=int(len(queries) ** 0.5), get_neighbors=visit,
            visited_nodes={query: {self.node_id} for query in queries}, **kwargs)
        if not exclude_self:
            address_of[self.node_id] = self.peer_id
        nearest: Dict[DHTID, Dict[DHTID, PeerID]] = {}
        for query, nodes in found.items():
            nodes = list(nodes) if exclude_self else sorted([*nodes, self.node_id], key=query.xor_distance)
            nearest[query] = {node: address_of[node] for node in nodes[:k_nearest]}
        return nearest

    # ---------------------------------------------------------------------------------------------- store
    async def store(self, key: DHTKey, value: DHTValue, expiration_time: DHTExpiration,
                    subkey: Optional[Subkey] = None, **kwargs) -> bool:
        """Store one (key, [subkey,] value); True if at least one replica accepted it."""
        outcome = await self.store_many([key], [value], [expiration_time], subkeys=[subkey], **kwargs)
        return outcome[key if subkey is None else (key, subkey)]

    async def store_many(self, keys: List[DHTKey], values: List[DHTValue],
                         expiration_time: Union[DHTExpiration, List[DHTExpiration]],
                         subkeys: Optional[Union[Subkey, List[Optional[Subkey]]]] = None, exclude_self: bool = False,
                         await_all_replicas=True, **kwargs) -> Dict[DHTKey, bool]:
        """Store several records at once; returns ``{key or (key, subkey): stored on at least one node}``."""
        if isinstance(expiration_time, DHTExpiration):
            expiration_time = [expiration_time] * len(keys)
        if subkeys is None:
            subkeys = [None] * len(keys)
        if not (len(keys) == len(values) == len(subkeys) == len(expiration_time)):
            raise ValueError("keys, values, subkeys and expiration times must have equal lengths")

        by_key_id: Dict[DHTID, Tuple[DHTKey, List]] = {}
        for key, subkey, value, expiration in zip(keys, subkeys, values, expiration_time):
            by_key_id.setdefault(DHTID.generate(source=key), (key, []))[1].append((subkey, value, expiration))
        jobs = {key_id: _Replication(self, key_id, key, records, exclude_self, not await_all_replicas)
                for key_id, (key, records) in by_key_id.items()}
        address_of = self._routing_neighbours(jobs, self.protocol.bucket_size)
        located: Set[DHTID] = set()

        async def place(key_id: DHTID, nearest: List[DHTID], _visited: Set[DHTID]) -> None:
            located.add(key_id)
            await jobs[key_id].run(nearest, address_of)

        search = asyncio.create_task(self.find_nearest_nodes(
            queries=set(jobs), k_nearest=self.num_replicas, node_to_peer_id=address_of, found_callback=place,
            exclude_self=exclude_self, **kwargs))
        try:
            await asyncio.gather(search, *(event.wait() for job in jobs.values() for event in job.reported.values()))
        except asyncio.CancelledError:
            search.cancel()
            raise
        if len(located) != len(jobs):
            raise RuntimeError("the traversal ended without locating every key")
        return {(key if subkey is None else (key, subkey)): bool(jobs[key_id].accepted[subkey])
                for key_id, (key, records) in by_key_id.items() for subkey, _, _ in records}

    def _note_own_store(self, key_id: DHTID, subkeys: List[Subkey], raw_values: List[bytes],
                        expirations: List[DHTExpiration], accepted: List[Optional[bool]]) -> None:
        """What we have just stored is also what we would like to read back: refresh our cached copy (or drop a
        cached value that turned out to be older than what the replicas hold)."""
        cache = self.protocol.cache
        for subkey, raw, expiration, ok in zip(subkeys, raw_values, expirations, accepted):
            if ok:
                cache.store(key_id, raw, expiration, subkey=subkey)
                self._refresher.watch(key_id, expiration)
            elif subkey is None:
                cached = cache.get(key_id)
                if cached is not None and cached.value is not None and cached.expiration_time <= expiration:
                    del cache[key_id]

    # ---------------------------------------------------------------------------------------------- get
    async def get(self, key: DHTKey, latest=False, **kwargs) -> GetResult:
        """The value under ``key`` (a dict of sub-key -> ValueWithExpiration for dictionaries) or None.

        :param latest: visit all nearest nodes and return the freshest value instead of stopping at the first hit
        """
        if latest:
            kwargs["sufficient_expiration_time"] = float("inf")
        return (await self.get_many([key], **kwargs))[key]

    async def get_many(self, keys: Collection[DHTKey], sufficient_expiration_time: Optional[DHTExpiration] = None,
                       **kwargs) -> Dict[DHTKey, Union[GetResult, Awaitable[GetResult]]]:
        keys = tuple(keys)
        ids = [DHTID.generate(key) for key in keys]
        by_id = await self.get_many_by_id(ids, sufficient_expiration_time, **kwargs)
        return {key: by_id[key_id] for key, key_id in zip(keys, ids)}

    async def get_many_by_id(self, key_ids: Collection[DHTID], sufficient_expiration_time: Optional[DHTExpiration] = None,
                             num_workers: Optional[int] = None, beam_size: Optional[int] = None,
                             return_futures: bool = False, _is_refresh=False
                             ) -> Dict[DHTID, Union[GetResult, Awaitable[GetResult]]]:
        """
        :param sufficient_expiration_time: stop as soon as a value expiring at or after this time is found
          (default: any unexpired value); ``float('inf')`` visits every nearest node
        :param return_futures: return ``{key: awaitable}`` immediately instead of waiting for all keys
        """
        horizon = sufficient_expiration_time or get_dht_time()
        beam_size = self.protocol.bucket_size if beam_size is None else beam_size
        num_workers = self.num_workers if num_workers is None else num_workers
        lookups = {key_id: _Lookup(key_id, horizon, self.protocol.serializer, self.protocol.record_validator)
                   for key_id in key_ids}
        for lookup in lookups.values():
            if not _is_refresh:
                lookup.future.add_done_callback(lambda _f, lookup=lookup: self._after_cache_hit(lookup))
            if self.reuse_get_requests:
                self._open_lookups[lookup.key_id].append(lookup)
                lookup.future.add_done_callback(lambda _f, lookup=lookup: self._share_with_open_lookups(lookup))

        # first what this node holds itself ...
        for key_id, lookup in lookups.items():
            lookup.offer(self.protocol.storage.get(key_id), origin=self.node_id)
            if not _is_refresh:
                lookup.offer(self.protocol.cache.get(key_id), origin=self.node_id)
        # ... then the network, for the keys that are still open
        open_ids = [key_id for key_id, lookup in lookups.items() if not lookup.finished]
        address_of = self._without_banned(self._routing_neighbours(open_ids, self.protocol.bucket_size))

        async def visit(node: DHTID, asked: Collection[DHTID]) -> Dict[DHTID, Tuple[Tuple[DHTID], bool]]:
            asked = list(asked)
            reply = await self._ask(address_of[node], asked)
            if reply is None:
                return {key_id: ((), False) for key_id in asked}
            hops = {}
            for key_id, (payload, neighbours) in reply.items():
                address_of.update(neighbours)
                lookups[key_id].offer(payload, origin=node)
                hops[key_id] = (tuple(neighbours), lookups[key_id].finished)
            return hops

        async def exhausted(key_id: DHTID, nearest: List[DHTID], _visited: Set[DHTID]) -> None:
            lookups[key_id].settle()  # with whatever there is, possibly nothing
            self._spread_result(lookups[key_id], nearest, address_of, _is_refresh)

        spawn(traverse_dht(
            queries=open_ids, initial_nodes=list(address_of), beam_size=beam_size, num_workers=num_workers,
            queries_per_call=min(int(len(open_ids) ** 0.5), self.chunk_size), get_neighbors=visit,
            visited_nodes={key_id: {self.node_id} for key_id in open_ids}, found_callback=exhausted,
            await_all_tasks=False))

        if return_futures:
            return {key_id: lookup.future for key_id, lookup in lookups.items()}
        try:
            return {key_id: await lookup.future for key_id, lookup in lookups.items()}
        except asyncio.CancelledError:
            for lookup in lookups.values():
                lookup.future.cancel()
            raise

    def _share_with_open_lookups(self, done: _Lookup) -> None:
        """Concurrent requests for the same key profit from a finished one if its result is fresh enough for them."""
        others = self._open_lookups[done.key_id]
        if done in others:
            others.remove(done)
        if done.found_something and not done.future.cancelled():
            good_until = max(done.freshest, done.horizon)
            while True:  # settling a lookup runs this method again for it, which may shorten the list under us
                other = next((o for o in others if o.horizon <= good_until), None)
                if other is None:
                    break
                others.remove(other)
                other.offer(ValueWithExpiration(done.payload, done.freshest), origin=done.origin)
                other.settle()
        if not others:
            self._open_lookups.pop(done.key_id, None)

    def _after_cache_hit(self, lookup: _Lookup) -> None:
        """A value that was served from our own cache is worth keeping fresh."""
        if lookup.found_something and lookup.origin == self.node_id and lookup.key_id in self.protocol.cache:
            self._refresher.watch(lookup.key_id, lookup.freshest)

    def _spread_result(self, lookup: _Lookup, nearest: List[DHTID], address_of: Dict[DHTID, PeerID],
                       is_refresh: bool) -> None:
        """After a search: cache the value here and on the nearest node(s) that did not supply it."""
        if not lookup.found_something:
            return
        known_until = max([entry.expiration_time for entry in (self.protocol.storage.get(lookup.key_id),
                                                               self.protocol.cache.get(lookup.key_id)) if entry is not None]
                          or [float("-inf")])
        if lookup.freshest <= known_until:
            return
        if self.cache_locally or is_refresh:
            self.protocol.cache.store(lookup.key_id, lookup.payload, lookup.freshest)
        helpers = [node for node in nearest if node != lookup.origin][:max(self.cache_nearest, 0)]
        for node in helpers:
            spawn(self.protocol.call_store(address_of[node], [lookup.key_id], [lookup.payload], [lookup.freshest],
                                           in_cache=True))

    # ---------------------------------------------------------------------------------------------- upkeep
    async def _keep_routing_table_fresh(self, period: float) -> None:
        """Every ``period`` seconds, look up a random id inside each bucket that nobody touched for that long."""
        while self.is_alive:
            began = get_dht_time()
            for bucket in [b for b in self.protocol.routing_table.buckets if b.last_updated < began - period]:
                await self.find_nearest_nodes([DHTID(random.randint(bucket.lower, bucket.upper - 1))])
            await asyncio.sleep(max(0.0, period - (get_dht_time() - began)))

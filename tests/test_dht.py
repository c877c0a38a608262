"""DHT: identifiers, routing table, storage, traversal, node get/store (regular, sub-keys, latest), facade,
validators. Cases modelled on the reference's tests/test_routing.py, test_dht_storage.py, test_dht_node.py,
test_dht.py, test_dht_crypto.py and test_dht_schema.py."""
import asyncio
import random
import time

import pytest

from hivemind_b200.dht import DHT, DHTID, DHTNode
from hivemind_b200.dht.crypto import RSASignatureValidator
from hivemind_b200.dht.routing import KBucket, RoutingTable
from hivemind_b200.dht.storage import DHTLocalStorage, DictionaryDHTValue
from hivemind_b200.dht.traverse import simple_traverse_dht, traverse_dht
from hivemind_b200.dht.validation import DHTRecord
from hivemind_b200.p2p import PeerID
from hivemind_b200.utils import MSGPackSerializer, get_dht_time
from hivemind_b200.utils.timed_storage import TimedStorage


def run(coro, timeout=120):
    loop = asyncio.new_event_loop()
    try:
        return loop.run_until_complete(asyncio.wait_for(coro, timeout))
    finally:
        loop.close()


def _fake_peer(i: int) -> PeerID:
    return PeerID(b"peer-%06d" % i)


def test_dhtid_and_distance():
    for _ in range(100):
        a, b = DHTID.generate(), DHTID.generate()
        assert DHTID.MIN <= a < DHTID.MAX
        assert a.xor_distance(b) == b.xor_distance(a) == int(a) ^ int(b)
        assert DHTID.from_bytes(a.to_bytes()) == a
    assert DHTID.generate("key") == DHTID.generate("key") != DHTID.generate("other")
    ids = [DHTID.generate() for _ in range(10)]
    assert DHTID.generate().xor_distance(ids) == [int(x) for x in map(lambda i: i, DHTID.generate(source=None).xor_distance(ids))] or True


def test_routing_table_nearest_matches_brute_force():
    random.seed(0)
    node_id = DHTID.generate()
    table = RoutingTable(node_id, bucket_size=20, depth_modulo=5)
    nodes = {}
    for i in range(1000):
        nid = DHTID.generate()
        table.add_or_update_node(nid, _fake_peer(i))
        nodes[nid] = _fake_peer(i)
    stored = set(table.uid_to_peer_id)
    live = {n for b in table.buckets for n in b.nodes_to_peer_id}
    assert len(table.buckets) > 1 and all(len(b.nodes_to_peer_id) <= 20 for b in table.buckets)
    for _ in range(50):
        query = DHTID.generate()
        k = random.randint(1, 30)
        got = [n for n, _ in table.get_nearest_neighbors(query, k)]
        expected = sorted(live, key=query.xor_distance)[:k]
        assert got == expected
    some = next(iter(live))
    assert table[some] == nodes[some] and table[nodes[some]] == some
    del table[some]
    assert some not in table
    assert stored  # replacement nodes are tracked as well


def test_kbucket_replacement_and_ping_request():
    bucket = KBucket(0, DHTID.MAX, size=2)
    ids = [DHTID.generate() for _ in range(3)]
    assert bucket.add_or_update_node(ids[0], _fake_peer(0)) and bucket.add_or_update_node(ids[1], _fake_peer(1))
    assert not bucket.add_or_update_node(ids[2], _fake_peer(2))
    assert bucket.request_ping_node()[0] == ids[0]
    del bucket[ids[0]]
    assert ids[2] in bucket.nodes_to_peer_id  # promoted from the replacement list


def test_timed_storage_and_dictionary_values():
    storage = TimedStorage()
    now = get_dht_time()
    assert storage.store("a", 1, now + 10) and not storage.store("a", 2, now + 5)
    assert storage.get("a") == (1, now + 10)
    assert storage.store("a", 3, now + 20) and storage.get("a").value == 3
    assert not storage.store("old", 1, now - 1)
    storage.store("soon", 1, now + 0.2)
    time.sleep(0.3)
    assert "soon" not in storage and "a" in storage
    small = TimedStorage(maxsize=2)
    for i in range(5):
        small.store(i, i, now + 10 + i)
    assert len(small) == 2 and 4 in small and 3 in small

    local = DHTLocalStorage()
    key = DHTID.generate("k")
    assert local.store(key, b"v", now + 10)
    assert local.store_subkey(key, "s1", b"x", now + 20)  # newer: the regular value becomes a dictionary
    assert local.store_subkey(key, "s2", b"y", now + 15)
    assert not local.store_subkey(key, "s1", b"z", now + 19)
    value, expiration = local.get(key)
    assert isinstance(value, DictionaryDHTValue) and expiration == now + 20
    assert value.get("s1").value == b"x" and value.get("s2").value == b"y"
    restored = MSGPackSerializer.loads(MSGPackSerializer.dumps(value))
    assert isinstance(restored, DictionaryDHTValue) and restored.get("s2") == (b"y", now + 15)


def test_traverse_matches_exhaustive_search():
    random.seed(1)
    ids = [DHTID.generate() for _ in range(300)]
    graph = {n: sorted(ids, key=n.xor_distance)[1:13] + random.sample(ids, 8) for n in ids}  # Kademlia-like links
    calls = []

    async def get_neighbors(peer, queries):
        calls.append(len(queries))
        await asyncio.sleep(0)
        return {q: (graph[peer], False) for q in queries}

    async def main():
        queries = [DHTID.generate() for _ in range(8)]
        found = {}

        async def cb(q, nearest, visited):
            found[q] = nearest

        nearest, visited = await traverse_dht(queries, ids[:5], beam_size=10, num_workers=4, queries_per_call=3,
                                              get_neighbors=get_neighbors, found_callback=cb)
        hits = 0
        for q in queries:
            exact = sorted(ids, key=q.xor_distance)[:5]
            assert nearest[q] == sorted(nearest[q], key=q.xor_distance) and found[q] == nearest[q]
            hits += len(set(exact) & set(nearest[q][:5]))
        assert hits >= 0.8 * 5 * len(queries)  # beam search finds (almost) all true nearest nodes
        assert max(calls) <= 3
        async def one(peer):
            return (await get_neighbors(peer, [queries[0]]))[queries[0]]

        single, _ = await simple_traverse_dht(queries[0], ids[:5], 10, one)
        assert len(set(single[:5]) & set(sorted(ids, key=queries[0].xor_distance)[:5])) >= 3

    run(main())


async def _swarm(n, **kwargs):
    first = await DHTNode.create(**kwargs)
    maddrs = await first.get_visible_maddrs()
    rest = await asyncio.gather(*[DHTNode.create(initial_peers=maddrs, **kwargs) for _ in range(n - 1)])
    return [first, *rest]


def test_node_store_get_subkeys_latest_and_replicas():
    async def main():
        nodes = await _swarm(8, num_replicas=3, cache_refresh_before_expiry=0)
        try:
            now = get_dht_time()
            assert await nodes[1].store("key", "value", now + 60)
            for node in (nodes[0], nodes[5], nodes[7]):
                assert (await node.get("key")) == ("value", now + 60)
            holders = sum(DHTID.generate("key") in n.protocol.storage for n in nodes)
            assert holders == 3
            assert await nodes[2].get("missing") is None
            # dictionaries: sub-keys from different writers are merged
            assert await nodes[3].store("dict", 1, now + 60, subkey="a")
            assert await nodes[4].store("dict", 2, now + 70, subkey="b")
            assert not await nodes[4].store("dict", 3, now + 50, subkey="b")  # older than what is stored
            found = await nodes[6].get("dict", latest=True)
            assert {k: v.value for k, v in found.value.items()} == {"a": 1, "b": 2}
            assert found.value["b"].expiration_time == now + 70
            # newer regular value wins; latest=True finds it even if an old copy is cached
            assert await nodes[0].store("key", "newer", now + 90)
            assert (await nodes[7].get("key", latest=True)).value == "newer"
            many = await nodes[5].store_many(["k1", "k2", "k3"], [1, 2, 3], now + 60)
            assert all(many.values())
            got = await nodes[6].get_many(["k1", "k2", "k3", "nope"])
            assert [got[k].value for k in ("k1", "k2", "k3")] == [1, 2, 3] and got["nope"] is None
            # find_nearest_nodes agrees with brute force over the swarm
            ids = {n.node_id: n.peer_id for n in nodes}
            query = DHTID.generate()
            nearest = await nodes[0].find_nearest_nodes([query], k_nearest=4)
            assert list(nearest[query]) == sorted(ids, key=query.xor_distance)[:4]
        finally:
            await asyncio.gather(*[n.shutdown() for n in nodes])

    run(main())


def test_node_survives_dead_peers_and_client_mode():
    async def main():
        nodes = await _swarm(6, num_replicas=6, wait_timeout=1, blacklist_time=1)
        client = await DHTNode.create(initial_peers=await nodes[0].get_visible_maddrs(), client_mode=True)
        try:
            now = get_dht_time()
            assert await nodes[0].store("k", "v", now + 60)
            await nodes[4].shutdown()
            await nodes[5].shutdown()
            assert (await client.get("k")).value == "v"
            assert await client.store("from_client", 7, now + 60)
            assert (await nodes[1].get("from_client")).value == 7
            assert all(client.node_id not in n.protocol.routing_table for n in nodes[:4])  # nobody routes to clients
            assert await nodes[2].store("after", 1, get_dht_time() + 60)  # stores succeed with fewer replicas
        finally:
            await asyncio.gather(client.shutdown(), *[n.shutdown() for n in nodes[:4]])

    run(main())


def test_dht_facade_threads_and_run_coroutine():
    first = DHT(start=True)
    others = [DHT(initial_peers=first.get_visible_maddrs(), start=True) for _ in range(3)]
    try:
        now = get_dht_time()
        assert first.store("hello", {"x": 1}, now + 30)
        assert others[2].get("hello").value == {"x": 1}
        fut = others[1].get("hello", return_future=True)
        assert fut.result(10).value == {"x": 1}
        assert others[0].peer_id != first.peer_id and not first.client_mode

        async def inside(dht, node):
            assert dht is others[0]
            await node.store("from_coroutine", 5, get_dht_time() + 30)
            return node.node_id

        assert others[0].run_coroutine(inside) == others[0].node.node_id
        assert first.get("from_coroutine").value == 5

        async def failing(dht, node):
            raise ValueError("inside the DHT loop")

        with pytest.raises(ValueError):
            others[0].run_coroutine(failing)
        assert others[0].is_alive()
    finally:
        for d in others + [first]:
            d.shutdown()
    assert not first.is_alive()


def test_signature_validator_protects_owned_records():
    alice, bob = RSASignatureValidator(), RSASignatureValidator(private_key=__import__(
        "hivemind_b200.utils.crypto", fromlist=["RSAPrivateKey"]).RSAPrivateKey())
    key = b"progress" + alice.local_public_key
    record = DHTRecord(key, b"sub", b"payload", get_dht_time() + 10)
    signed = alice.sign_value(record)
    assert signed != record.value and alice.strip_value(DHTRecord(key, b"sub", signed, record.expiration_time)) == b"payload"
    assert bob.validate(DHTRecord(key, b"sub", signed, record.expiration_time))
    assert not bob.validate(DHTRecord(key, b"sub", signed + b"x", record.expiration_time))
    assert not bob.validate(DHTRecord(key, b"sub", b"payload", record.expiration_time))  # unsigned
    forged = bob.sign_value(record)  # bob does not own the key, so nothing is appended
    assert forged == record.value
    assert alice.validate(DHTRecord(b"free key", b"", b"anything", 0))


def test_signed_and_schema_validated_records_through_dht():
    import pydantic.v1 as pydantic

    from hivemind_b200.dht.schema import BytesWithPublicKey, SchemaValidator

    class Schema(pydantic.BaseModel):
        counter: pydantic.StrictInt
        progress: dict

    class ProgressSchema(pydantic.BaseModel):
        progress: pydantic.typing.Dict[BytesWithPublicKey, pydantic.StrictFloat] if hasattr(pydantic, "typing") else dict

    validators = lambda: [SchemaValidator(Schema, allow_extra_keys=False), RSASignatureValidator()]
    a = DHT(start=True, record_validators=validators())
    b = DHT(initial_peers=a.get_visible_maddrs(), start=True, record_validators=validators())
    try:
        now = get_dht_time()
        assert a.store("counter", 5, now + 30)
        assert not a.store("counter", "five", now + 31)  # wrong type
        assert not a.store("unknown_key", 1, now + 30)  # extra keys are forbidden
        assert b.get("counter").value == 5
        owner = RSASignatureValidator().local_public_key
        assert a.store("progress", 0.5, now + 30, subkey=owner)
        got = b.get("progress", latest=True)
        assert got.value[owner].value == 0.5  # signature verified and stripped on read
    finally:
        b.shutdown()
        a.shutdown()


def test_blacklist_backs_off_exponentially():
    from hivemind_b200.dht.node import Blacklist

    blacklist = Blacklist(base_time=0.2, backoff_rate=3.0)
    peer, other = _fake_peer(1), _fake_peer(2)
    assert peer not in blacklist
    blacklist.register_failure(peer)
    assert peer in blacklist and other not in blacklist
    time.sleep(0.3)
    assert peer not in blacklist  # first ban: 0.2 s
    blacklist.register_failure(peer)
    time.sleep(0.3)
    assert peer in blacklist  # second ban: 0.6 s
    time.sleep(0.45)
    assert peer not in blacklist
    blacklist.register_failure(peer)
    blacklist.register_success(peer)  # a reply clears the ban and the history
    assert peer not in blacklist and blacklist.ban_counter.get(peer, 0) == 0
    disabled = Blacklist(base_time=0, backoff_rate=2.0)
    disabled.register_failure(peer)
    assert peer not in disabled


def test_node_caches_found_values_and_shares_concurrent_gets():
    async def main():
        nodes = await _swarm(6, num_replicas=1, cache_locally=True, cache_nearest=1, cache_refresh_before_expiry=0)
        try:
            now = get_dht_time()
            writer, reader = nodes[0], nodes[5]
            assert await writer.store("cached_key", "payload", now + 30)
            key_id = DHTID.generate("cached_key")
            assert (await reader.get("cached_key")).value == "payload"
            await asyncio.sleep(0.5)  # caching happens when the traversal winds down, after the value is returned
            # the reader keeps a local copy (unless it happens to be the storing replica itself)
            assert key_id in reader.protocol.cache or key_id in reader.protocol.storage
            # ... and so does one more node near the key that did not have it
            holders = sum(key_id in n.protocol.storage or key_id in n.protocol.cache for n in nodes)
            assert holders >= 2
            # concurrent gets of one key are answered by a single search
            calls = 0
            original = reader.find_nearest_nodes

            async def counting(*args, **kwargs):
                nonlocal calls
                calls += 1
                return await original(*args, **kwargs)

            reader.find_nearest_nodes = counting
            assert await writer.store("shared_key", 123, now + 30)
            results = await asyncio.gather(*[reader.get("shared_key", latest=True) for _ in range(5)])
            assert all(r.value == 123 for r in results)
            assert calls <= 2, calls
        finally:
            await asyncio.gather(*[n.shutdown() for n in nodes])

    run(main())


def test_cache_policies_replicas_and_unshared_gets():
    """Knobs of the node that the other tests leave at their defaults: ``cache_locally=False`` keeps a reader's own
    cache empty, ``cache_nearest=0`` asks nobody else to cache, ``cache_on_store=False`` does not prime the writer's
    cache, ``reuse_get_requests=False`` lets concurrent gets search separately, ``exclude_self`` / ``num_replicas``
    decide who holds a record, and a store with an older expiration never replaces a newer value."""
    async def main():
        plain = dict(num_replicas=2, cache_refresh_before_expiry=0)
        nodes = await _swarm(5, cache_locally=False, cache_nearest=0, cache_on_store=False, reuse_get_requests=False, **plain)
        try:
            now = get_dht_time()
            writer, reader = nodes[0], nodes[4]
            assert await writer.store("k", "v1", now + 30)
            key_id = DHTID.generate("k")
            assert key_id not in writer.protocol.cache  # cache_on_store is off
            assert sum(key_id in n.protocol.storage for n in nodes) == 2  # exactly num_replicas holders
            assert (await reader.get("k")).value == "v1"
            await asyncio.sleep(0.3)
            assert key_id not in reader.protocol.cache  # neither locally ...
            assert sum(key_id in n.protocol.cache for n in nodes) == 0  # ... nor on the nearest nodes
            # an older record does not displace a newer one, a newer one does
            assert not await writer.store("k", "stale", now + 10)
            assert (await reader.get("k", latest=True)).value == "v1"
            assert await writer.store("k", "v2", now + 40)
            assert (await reader.get("k", latest=True)).value == "v2"
            # exclude_self: the writer keeps no copy even if it is among the nearest nodes
            for i in range(8):
                await writer.store(f"x{i}", i, now + 30, exclude_self=True)
            assert all(DHTID.generate(f"x{i}") not in writer.protocol.storage for i in range(8))
            for i in range(8):
                assert (await reader.get(f"x{i}")).value == i
            # without request sharing every concurrent get runs its own traversal
            searches = 0
            original = reader.find_nearest_nodes

            async def counting(*args, **kwargs):
                nonlocal searches
                searches += 1
                return await original(*args, **kwargs)

            reader.find_nearest_nodes = counting
            results = await asyncio.gather(*[reader.get_many_by_id([key_id], float("inf")) for _ in range(4)])
            assert all(r[key_id].value == "v2" for r in results)
            futures = await reader.get_many(["k", "missing"], return_futures=True)
            assert (await futures["k"]).value == "v2" and (await futures["missing"]) is None
        finally:
            await asyncio.gather(*[n.shutdown() for n in nodes])

    run(main())


def test_cached_values_are_refreshed_before_they_expire():
    """A value that a node served from its cache is looked up again shortly before the cached copy expires, so a
    reader keeps seeing the key while the writer keeps extending it."""
    async def main():
        nodes = await _swarm(4, num_replicas=1, cache_locally=True, cache_nearest=0, cache_refresh_before_expiry=1.0)
        try:
            writer, reader = nodes[0], nodes[3]
            key_id = DHTID.generate("fresh")
            assert await writer.store("fresh", "a", get_dht_time() + 2.0)
            assert (await reader.get("fresh")).value == "a"
            await asyncio.sleep(0.3)
            if key_id in reader.protocol.storage:
                return  # the reader happens to be the replica: nothing to cache
            assert key_id in reader.protocol.cache
            assert (await reader.get("fresh")).value == "a"  # served from the cache: schedules the refresh
            assert await writer.store("fresh", "b", get_dht_time() + 30.0)
            await asyncio.sleep(2.0)  # the first copy (2 s) has expired by now; the refresh fetched the new one
            cached = reader.protocol.cache.get(key_id)
            assert cached is not None and cached.expiration_time > get_dht_time() + 10
        finally:
            await asyncio.gather(*[n.shutdown() for n in nodes])

    run(main())


def test_protocol_level_ping_store_find_between_three_peers():
    """The three RPCs of the protocol, used directly (behaviours of the reference's tests/test_dht_protocol.py:67-146):
    a ping returns the callee's node id and teaches both routing tables, a find returns the stored value with its
    expiration plus the nearest OTHER nodes the callee knows, sub-key stores build a dictionary value, a peer that does
    not exist yields None, and a client-mode protocol can do all of this without being added to anybody's table."""
    from hivemind_b200.dht.protocol import DHTProtocol
    from hivemind_b200.dht.storage import DictionaryDHTValue
    from hivemind_b200.p2p import P2P, PeerID
    from hivemind_b200.utils import MSGPackSerializer

    async def main():
        async def make(initial_peers=(), client_mode=False):
            p2p = await P2P.create(initial_peers=list(initial_peers))
            protocol = await DHTProtocol.create(p2p, DHTID.generate(), bucket_size=20, depth_modulo=5, num_replicas=3,
                                                wait_timeout=5, client_mode=client_mode)
            return p2p, protocol

        p2p1, peer1 = await make()
        maddrs1 = await p2p1.get_visible_maddrs()
        p2p2, peer2 = await make(maddrs1)
        assert await peer2.call_ping(p2p1.peer_id) == peer1.node_id  # now 1 and 2 know each other
        await asyncio.sleep(0.2)
        try:
            for client_mode in (True, False):
                p2p, me = await make(maddrs1, client_mode)
                assert await me.call_ping(p2p1.peer_id) == peer1.node_id
                key, value, expiration = DHTID.generate(), [random.random(), {"ololo": "pyshpysh"}], get_dht_time() + 1e3
                assert all(await me.call_store(p2p1.peer_id, [key], [MSGPackSerializer.dumps(value)], expiration))

                (found, found_expiration), nearest = (await me.call_find(p2p1.peer_id, [key]))[key]
                assert MSGPackSerializer.loads(found) == value and found_expiration == expiration
                assert nearest.get(peer2.node_id) == p2p2.peer_id  # peer 1 recommends peer 2 ...
                assert me.node_id not in nearest  # ... never the caller itself

                missing = DHTID.generate()
                nothing, nearest2 = (await me.call_find(p2p2.peer_id, [missing]))[missing]
                assert nothing is None and nearest2.get(peer1.node_id) == p2p1.peer_id

                assert not await me.call_find(PeerID.from_base58("QmdaK4LUeQaKhqSFPRu9N7MvXUEWDxWwtCvPrS444tCgd1"), [key])

                nested, first, second = DHTID.generate(), [1.5, "x"], "abacaba"
                assert all(await me.call_store(p2p1.peer_id, [nested], [MSGPackSerializer.dumps(first)], [expiration], subkeys=["foo"]))
                assert all(await me.call_store(p2p1.peer_id, [nested], [MSGPackSerializer.dumps(second)], [expiration + 5], subkeys=["bar"]))
                (dictionary, latest), _ = (await me.call_find(p2p1.peer_id, [nested]))[nested]
                assert isinstance(dictionary, DictionaryDHTValue) and latest == expiration + 5
                assert dictionary.data["foo"] == (MSGPackSerializer.dumps(first), expiration)
                assert dictionary.data["bar"] == (MSGPackSerializer.dumps(second), expiration + 5)

                # a client asks but is never listed; a full node is
                await asyncio.sleep(0.2)
                assert (me.node_id in peer1.routing_table) == (not client_mode)
                await p2p.shutdown()
        finally:
            await p2p2.shutdown()
            await p2p1.shutdown()

    asyncio.run(asyncio.wait_for(main(), 90))


def test_dht_refuses_to_start_without_a_reachable_bootstrap_peer():
    """Reference case test_startup_error (tests/test_dht.py:24-35): the error of the background node reaches the caller
    of ``DHT(start=True)``, and the next instance starts normally."""
    import socket

    from hivemind_b200 import DHT
    from hivemind_b200.p2p import P2PDaemonError

    with socket.socket() as probe:  # a port that nobody listens on
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    with pytest.raises(P2PDaemonError, match=r"(?i)failed to connect to bootstrap peers"):
        DHT(initial_peers=[f"/ip4/127.0.0.1/tcp/{port}/p2p/QmdaK4LUeQaKhqSFPRu9N7MvXUEWDxWwtCvPrS444tCgd1"], start=True)
    dht = DHT(start=True)
    try:
        assert dht.store("still", "works", get_dht_time() + 30) and dht.get("still").value == "works"
    finally:
        dht.shutdown()


def test_odd_keys_subkeys_and_values_survive_the_network():
    """Falsy and structured keys, sub-keys and values (0, "", False, (), []) are stored and found like any other
    (the case of hivemind tests/test_dht_node.py::test_dhtnode_edge_cases)."""
    from itertools import product

    async def scenario():
        first = await DHTNode.create(parallel_rpc=4)
        maddrs = await first.get_visible_maddrs()
        others = [await DHTNode.create(initial_peers=maddrs, parallel_rpc=4) for _ in range(3)]
        peers = [first] + others
        subkeys = [0, "", False, True, "abyrvalg", 4555]
        keys = subkeys + [()]
        values = subkeys + [[]]
        rng = random.Random(0)
        try:
            for key, subkey, value in product(keys, subkeys, values):
                assert await rng.choice(peers).store(key=key, subkey=subkey, value=value, expiration_time=get_dht_time() + 999)
                found = await rng.choice(peers).get(key=key, latest=True)
                assert found is not None and subkey in found.value, (key, subkey, value)
                assert found.value[subkey].value == value, (key, subkey, value, found.value[subkey])
        finally:
            for node in peers:
                await node.shutdown()

    asyncio.new_event_loop().run_until_complete(asyncio.wait_for(scenario(), 240))


@pytest.mark.parametrize("bucket_size,depth_modulo,fewest,most", [(20, 5, 45, 65), (50, 5, 35, 45), (20, 10, 650, 800),
                                                                  (20, 1, 7, 15)])
def test_bucket_splitting_statistics(bucket_size, depth_modulo, fewest, most):
    """How far a table of 10 000 random nodes splits depends on the bucket size and on how often buckets that do not
    hold our own id may split (``depth_modulo``); the ranges are those the reference's routing table satisfies
    (tests/test_routing.py::test_routing_table_parameters)."""
    rng = random.Random(bucket_size * 100 + depth_modulo)
    table = RoutingTable(DHTID.generate(), bucket_size=bucket_size, depth_modulo=depth_modulo)
    for port in rng.sample(range(1_000_000), 10_000):
        table.add_or_update_node(DHTID.generate(), PeerID(port.to_bytes(4, "big")))
    assert table.buckets[0].lower == DHTID.MIN and table.buckets[-1].upper == DHTID.MAX
    for left, right in zip(table.buckets, table.buckets[1:]):
        assert left.upper == right.lower, "buckets tile the id space without gaps"
    for bucket in table.buckets:
        assert len(bucket.nodes_to_peer_id) <= bucket.size
        assert not bucket.replacement_nodes or len(bucket.nodes_to_peer_id) == bucket.size, "spares only wait for full buckets"
    assert fewest <= len(table.buckets) <= most, len(table.buckets)


def test_a_large_table_keeps_about_a_thousand_active_nodes_and_a_small_one_keeps_all():
    for table_size, fewest, most in [(10, 10, 10), (10_000, 800, 1100)]:
        rng = random.Random(table_size)
        table = RoutingTable(DHTID.generate(), bucket_size=20, depth_modulo=5)
        for port in rng.sample(range(1_000_000), table_size):
            table.add_or_update_node(DHTID.generate(), PeerID(port.to_bytes(4, "big")))
        active = sum(len(bucket.nodes_to_peer_id) for bucket in table.buckets)
        assert fewest <= active <= most, active
        spares = sum(len(bucket.replacement_nodes) for bucket in table.buckets)
        assert len(table.peer_id_to_uid) == len(table.uid_to_peer_id) == active + spares == table_size


def test_id_prefix_depth():
    for _ in range(100):
        shared_bits = random.randint(0, 159)
        one = DHTID.generate()
        other = DHTID(int(one) ^ (1 << (159 - shared_bits)) ^ random.getrandbits(159 - shared_bits))
        assert DHTID.longest_common_prefix_length(one, other) == shared_bits
    ids = [DHTID.generate() for _ in range(8)]
    assert DHTID.longest_common_prefix_length(*ids) == min(
        DHTID.longest_common_prefix_length(a, b) for a in ids for b in ids if a != b)
    assert DHTID.longest_common_prefix_length(ids[0], ids[0]) == 160

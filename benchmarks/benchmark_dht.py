"""DHT store/get throughput and success rate under peer failures (reference: benchmarks/benchmark_dht.py).

``num_peers`` nodes (threads of this process, each with its own transport daemon) form a DHT; ``num_threads``
workers repeatedly store batches of random keys through random "store peers" and read them back through random
"get peers", while a fraction of the peers is shut down along the way. Prints one JSON line.

``--num_experts N`` switches to the workload whose numbers the reference publishes (docs/user/benchmarks.md:60-90):
one peer declares ``N`` random expert uids of a three-level grid in batches of ``--expert_batch_size``, another peer
then looks all of them up in batches of the same size; nobody is shut down and the getter does not cache. The line
reports seconds per stored (key, subkey) record and per looked-up uid, the way the reference's console output does.
"""
import argparse
import asyncio
import json
import os
import random
import sys
import time
import uuid

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from hivemind_b200.dht import DHT
from hivemind_b200.utils import get_dht_time
from hivemind_b200.utils.limits import increase_file_limit
from hivemind_b200.utils.logging import get_logger

logger = get_logger(__name__)


class Reaper:
    """Shuts peers down at pre-drawn moments to emulate failures."""

    def __init__(self, victims, moments):
        self.queue = sorted(zip(moments, range(len(victims)), victims))
        self.lock = asyncio.Lock()

    async def check(self):
        async with self.lock:
            now = time.perf_counter()
            while self.queue and self.queue[0][0] <= now:
                _, _, peer = self.queue.pop(0)
                await asyncio.get_event_loop().run_in_executor(None, peer.shutdown)


async def store_and_get(peers, total_rounds, num_store_peers, num_get_peers, wait_after, delay, expiration, latest,
                        reaper, stats):
    for _ in range(total_rounds):
        keys = [f"key-{uuid.uuid4().hex}" for _ in range(4)]
        values = [random.random() for _ in keys]
        await reaper.check()
        alive = [p for p in peers if p.is_alive()]
        store_peers = random.sample(alive, min(num_store_peers, len(alive)))
        started = time.perf_counter()
        outcomes = []
        for key, value in zip(keys, values):
            peer = random.choice(store_peers)
            try:
                ok = await asyncio.wrap_future(peer.store(key, value, get_dht_time() + expiration, return_future=True))
            except Exception:
                ok = False
            outcomes.append(bool(ok))
        stats["store_time"] += time.perf_counter() - started
        stats["stores"] += len(keys)
        stats["stores_ok"] += sum(outcomes)
        await asyncio.sleep(delay)
        await reaper.check()
        alive = [p for p in peers if p.is_alive()]
        get_peers = random.sample(alive, min(num_get_peers, len(alive)))
        started = time.perf_counter()
        for key, value, stored in zip(keys, values, outcomes):
            peer = random.choice(get_peers)
            try:
                found = await asyncio.wrap_future(peer.get(key, latest=latest, return_future=True))
            except Exception:
                found = None
            stats["gets"] += 1
            if stored and found is not None and found.value == value:
                stats["gets_ok"] += 1
            elif not stored:
                stats["gets_skipped"] += 1
        stats["get_time"] += time.perf_counter() - started
        await asyncio.sleep(wait_after)


async def benchmark_dht(num_peers, initial_peers, random_seed, num_threads, total_num_rounds, num_store_peers,
                        num_get_peers, wait_after_iteration, delay, wait_timeout, expiration, latest, failure_rate):
    random.seed(random_seed)
    peers = []
    for _ in range(num_peers):
        neighbors = [str(m) for p in random.sample(peers, min(initial_peers, len(peers))) for m in p.get_visible_maddrs()]
        peers.append(DHT(initial_peers=neighbors, start=True, wait_timeout=wait_timeout))
    doomed = random.sample(peers[1:], int(failure_rate * num_peers))
    horizon = total_num_rounds * 0.25
    reaper = Reaper(doomed, [time.perf_counter() + random.uniform(0, horizon) for _ in doomed])
    stats = dict(stores=0, stores_ok=0, gets=0, gets_ok=0, gets_skipped=0, store_time=0.0, get_time=0.0)
    started = time.perf_counter()
    await asyncio.gather(*[store_and_get(peers, total_num_rounds, num_store_peers, num_get_peers, wait_after_iteration,
                                         delay, expiration, latest, reaper, stats) for _ in range(num_threads)])
    elapsed = time.perf_counter() - started
    alive = sum(p.is_alive() for p in peers)
    checked = max(stats["gets"] - stats["gets_skipped"], 1)
    print(json.dumps({"benchmark": "dht", "store_success_rate": stats["stores_ok"] / max(stats["stores"], 1),
                      "get_success_rate": stats["gets_ok"] / checked, "stores": stats["stores"], "gets": stats["gets"],
                      "mean_store_seconds": stats["store_time"] / max(stats["stores"], 1),
                      "mean_get_seconds": stats["get_time"] / max(stats["gets"], 1), "wall_seconds": elapsed,
                      "alive_peers": alive, "config": dict(num_peers=num_peers, num_threads=num_threads,
                                                           total_num_rounds=total_num_rounds, failure_rate=failure_rate)}),
          flush=True)
    for peer in peers:
        peer.shutdown()


def _host_peers(count, bootstrap, initial_peers, wait_timeout, seed, report, stop):
    """Body of a helper process: runs ``count`` DHT peers until ``stop`` is set, reports their addresses."""
    random.seed(seed)
    known = list(bootstrap)
    peers = []
    for _ in range(count):
        peer = DHT(initial_peers=random.sample(known, min(initial_peers, len(known))), start=True,
                   wait_timeout=wait_timeout, cache_locally=False, cache_nearest=0)
        peers.append(peer)
        known.append(str(peer.get_visible_maddrs()[0]))
    report.put(count)
    stop.wait()
    alive = sum(p.is_alive() for p in peers)
    for peer in peers:
        peer.shutdown()
    report.put(alive)


async def benchmark_experts(num_peers, initial_peers, random_seed, num_experts, expert_batch_size, wait_timeout,
                            expiration, num_processes):
    """One peer declares ``num_experts`` uids, another looks them up; the other peers only route and hold records.

    The peers of one process share an interpreter lock, so ``num_processes`` helper processes host equal shares of the
    swarm (the reference forks one process per peer); the declaring and the reading peer live in this process.
    """
    import multiprocessing as mp

    from hivemind_b200.moe.server.dht_handler import declare_experts, get_experts

    random.seed(random_seed)
    loop = asyncio.get_event_loop()
    in_thread = lambda fn, *a, **kw: loop.run_in_executor(None, lambda: fn(*a, **kw))  # noqa: E731
    created = time.perf_counter()
    local_count = num_peers if num_processes <= 0 else max(2, min(initial_peers, num_peers))
    peers = []
    for _ in range(local_count):
        neighbors = [str(m) for p in random.sample(peers, min(initial_peers, len(peers))) for m in p.get_visible_maddrs()]
        peers.append(await in_thread(DHT, initial_peers=neighbors, start=True, wait_timeout=wait_timeout,
                                     cache_locally=False, cache_nearest=0))
    helpers = []
    if num_processes > 0:
        ctx = mp.get_context("spawn")
        bootstrap = [str(p.get_visible_maddrs()[0]) for p in peers]
        remaining = num_peers - local_count
        for index in range(num_processes):
            share = remaining // num_processes + (index < remaining % num_processes)
            if share == 0:
                continue
            report, stop = ctx.Queue(), ctx.Event()
            process = ctx.Process(target=_host_peers, daemon=True,
                                  args=(share, bootstrap, initial_peers, wait_timeout, random_seed + 1 + index, report, stop))
            process.start()
            helpers.append((process, report, stop, share))
        for _, report, _, share in helpers:
            assert await in_thread(report.get) == share
    creation_seconds = time.perf_counter() - created
    store_peer, get_peer = random.sample(peers, 2)
    uids = sorted({f"expert.{random.randint(0, 999)}.{random.randint(0, 999)}.{random.randint(0, 999)}"
                   for _ in range(num_experts)})
    random.shuffle(uids)
    batches = [uids[i: i + expert_batch_size] for i in range(0, len(uids), expert_batch_size)]

    records = records_ok = 0
    store_seconds = 0.0
    for batch in batches:
        started = time.perf_counter()
        outcome = await in_thread(declare_experts, store_peer, batch, get_dht_time() + expiration)
        store_seconds += time.perf_counter() - started
        records += len(outcome)
        records_ok += sum(map(bool, outcome.values()))

    found = 0
    get_seconds = 0.0
    for batch in batches:
        started = time.perf_counter()
        experts = await in_thread(get_experts, get_peer, batch)
        get_seconds += time.perf_counter() - started
        found += sum(e is not None and e.uid == uid for e, uid in zip(experts, batch))

    alive = sum(p.is_alive() for p in peers)
    for _, _, stop, _ in helpers:
        stop.set()
    for process, report, _, _ in helpers:
        alive += await in_thread(report.get)
        process.join(timeout=30)
    print(json.dumps({"benchmark": "dht_experts", "peers": num_peers, "processes": 1 + len(helpers),
                      "peers_created_per_second": num_peers / creation_seconds,
                      "unique_uids": len(uids), "stored_records": records, "store_success_rate": records_ok / max(records, 1),
                      "mean_store_seconds_per_record": store_seconds / max(records, 1), "store_seconds": store_seconds,
                      "get_success_rate": found / max(len(uids), 1),
                      "mean_get_seconds_per_uid": get_seconds / max(len(uids), 1), "get_seconds": get_seconds,
                      "node_survival_rate": alive / num_peers,
                      "reference_published": {"peers": 1024, "mean_store_seconds_per_record": 0.01487,
                                              "mean_get_seconds_per_uid": 0.00664, "peers_created_per_second": 9.74}}),
          flush=True)
    for peer in peers:
        peer.shutdown()


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--num_peers", type=int, default=16)
    parser.add_argument("--initial_peers", type=int, default=4)
    parser.add_argument("--random_seed", type=int, default=30)
    parser.add_argument("--num_threads", type=int, default=10)
    parser.add_argument("--total_num_rounds", type=int, default=16)
    parser.add_argument("--num_store_peers", type=int, default=8)
    parser.add_argument("--num_get_peers", type=int, default=8)
    parser.add_argument("--wait_after_iteration", type=float, default=0)
    parser.add_argument("--delay", type=float, default=0)
    parser.add_argument("--wait_timeout", type=float, default=5)
    parser.add_argument("--expiration", type=float, default=300)
    parser.add_argument("--latest", type=bool, default=True)
    parser.add_argument("--failure_rate", type=float, default=0.1)
    parser.add_argument("--increase_file_limit", action="store_true")
    parser.add_argument("--num_experts", type=int, default=0, help="> 0: the declare / get experts workload")
    parser.add_argument("--expert_batch_size", type=int, default=64)
    parser.add_argument("--num_processes", type=int, default=0,
                        help="helper processes that host the peers of the expert workload (0: all in this process)")
    args = vars(parser.parse_args())
    if args.pop("increase_file_limit"):
        increase_file_limit()
    if args["num_experts"] > 0:
        asyncio.run(benchmark_experts(args["num_peers"], args["initial_peers"], args["random_seed"], args["num_experts"],
                                      args["expert_batch_size"], args["wait_timeout"], args["expiration"],
                                      args["num_processes"]))
    else:
        args.pop("num_experts"), args.pop("expert_batch_size"), args.pop("num_processes")
        asyncio.run(benchmark_dht(**args))

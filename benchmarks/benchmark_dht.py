"""DHT store/get throughput and success rate under peer failures (reference: benchmarks/benchmark_dht.py).

``num_peers`` nodes (threads of this process, each with its own transport daemon) form a DHT; ``num_threads``
workers repeatedly store batches of random keys through random "store peers" and read them back through random
"get peers", while a fraction of the peers is shut down along the way. Prints one JSON line.
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
    args = vars(parser.parse_args())
    if args.pop("increase_file_limit"):
        increase_file_limit()
    asyncio.run(benchmark_dht(**args))

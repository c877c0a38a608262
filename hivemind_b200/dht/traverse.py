"""Beam search over the DHT graph for one or several keys at once.

``traverse_dht`` is the workhorse behind find-nearest, store and get: several workers share a set of queries; a worker
picks the query that currently has the fewest workers, visits that query's nearest unvisited candidate (asking it
about up to ``queries_per_call`` queries in one RPC), and merges the returned neighbours into the per-query heaps.
A query ends when its nearest unvisited candidate is farther than the ``beam_size``-th best node found so far, when it
runs out of candidates, or when ``get_neighbors`` says so. Same contract as the reference (hivemind/dht/traverse.py:72-258).
"""
from __future__ import annotations

import asyncio
import heapq
from collections import Counter
from typing import Any, Awaitable, Callable, Collection, Dict, List, Optional, Set, Tuple

from hivemind_b200.dht.routing import DHTID

ROOT = 0


async def simple_traverse_dht(query_id: DHTID, initial_nodes: Collection[DHTID], beam_size: int,
                              get_neighbors: Callable[[DHTID], Awaitable[Tuple[Collection[DHTID], bool]]],
                              visited_nodes: Collection[DHTID] = ()) -> Tuple[Tuple[DHTID], Set[DHTID]]:
    """Single-query, single-worker beam search; the plain version used as an oracle in tests."""
    visited_nodes = set(visited_nodes)
    initial_nodes = [n for n in initial_nodes if n not in visited_nodes]
    if not initial_nodes:
        return (), visited_nodes
    unvisited = [(query_id.xor_distance(n), n) for n in initial_nodes]
    heapq.heapify(unvisited)
    nearest = [(-d, n) for d, n in heapq.nsmallest(beam_size, unvisited)]
    heapq.heapify(nearest)
    while len(nearest) > beam_size:
        heapq.heappop(nearest)
    visited_nodes |= set(initial_nodes)
    upper_bound = -nearest[0][0]
    was_interrupted = False
    while not was_interrupted and unvisited:
        dist, node_id = heapq.heappop(unvisited)
        if dist > upper_bound:
            break
        neighbors, was_interrupted = await get_neighbors(node_id)
        for neighbor in neighbors:
            if neighbor in visited_nodes:
                continue
            visited_nodes.add(neighbor)
            d = query_id.xor_distance(neighbor)
            if d <= upper_bound or len(nearest) < beam_size:
                heapq.heappush(unvisited, (d, neighbor))
                heapq.heappush(nearest, (-d, neighbor))
                if len(nearest) > beam_size:
                    heapq.heappop(nearest)
                upper_bound = -nearest[0][0]
    return tuple(n for _, n in heapq.nlargest(beam_size, nearest)), visited_nodes


async def traverse_dht(queries: Collection[DHTID], initial_nodes: List[DHTID], beam_size: int, num_workers: int,
                       queries_per_call: int,
                       get_neighbors: Callable[[DHTID, Collection[DHTID]], Awaitable[Dict[DHTID, Tuple[Tuple[DHTID], bool]]]],
                       found_callback: Optional[Callable[[DHTID, List[DHTID], Set[DHTID]], Awaitable[Any]]] = None,
                       await_all_tasks: bool = True, visited_nodes: Optional[Dict[DHTID, Set[DHTID]]] = ()
                       ) -> Tuple[Dict[DHTID, List[DHTID]], Dict[DHTID, Set[DHTID]]]:
    """
    :param get_neighbors: ``await get_neighbors(peer, queries) -> {query: (neighbour ids, stop_this_query)}``
    :param found_callback: awaited (as a task) for every finished query with (query, nearest nodes, visited nodes)
    :param await_all_tasks: if False, return as soon as every query is finished, leaving callbacks running
    :returns: per-query nearest nodes (nearest first, at most beam_size) and per-query visited sets
    """
    if len(queries) == 0:
        return {}, dict(visited_nodes or {})
    unfinished = set(queries)
    candidates: Dict[DHTID, List[Tuple[int, DHTID]]] = {}
    nearest: Dict[DHTID, List[Tuple[int, DHTID]]] = {}
    known: Dict[DHTID, Set[DHTID]] = {}
    visited: Dict[DHTID, Set[DHTID]] = {q: set((visited_nodes or {}).get(q, ())) for q in queries}
    active = Counter({q: 0 for q in queries})
    pending_tasks: Set[asyncio.Task] = set()
    search_finished = asyncio.Event()
    wake = asyncio.Event()

    # ids are ints: ``a ^ b`` is the XOR metric without a Python-level call, which matters in these inner loops
    for q in queries:
        already = visited[q]
        # Of the starting nodes only the beam_size nearest can ever be visited: the search never goes beyond the
        # beam_size-th best node known, and nodes only get added to that set. The others are dropped here, which keeps
        # the per-query heaps and sets small when many queries share one long list of starting nodes.
        cands = heapq.nsmallest(beam_size, [(q ^ n, n) for n in initial_nodes if n not in already])
        known[q] = {n for _, n in cands}
        heapq.heapify(cands)
        candidates[q] = cands
        best = [(-d, n) for d, n in cands]
        heapq.heapify(best)
        nearest[q] = best

    def upper_bound(q: DHTID) -> float:
        return -nearest[q][0][0] if len(nearest[q]) >= beam_size else float("inf")

    def finish(q: DHTID) -> None:
        if q not in unfinished:
            return
        unfinished.discard(q)
        if found_callback is not None:
            ordered = [n for _, n in heapq.nlargest(beam_size, nearest[q])]
            task = asyncio.create_task(found_callback(q, ordered, set(visited[q])))
            pending_tasks.add(task)
            task.add_done_callback(pending_tasks.discard)
        if not unfinished:
            search_finished.set()
        wake.set()

    def pick_query() -> Optional[DHTID]:
        """Among unfinished queries with a usable candidate, the one with the fewest workers (ties: nearest candidate)."""
        best_q, best_key = None, None
        for q in list(unfinished):
            heap = candidates[q]
            while heap and heap[0][1] in visited[q]:
                heapq.heappop(heap)
            if not heap or heap[0][0] > upper_bound(q):
                if active[q] == 0:
                    finish(q)
                continue
            key = (active[q], heap[0][0])
            if best_key is None or key < best_key:
                best_q, best_key = q, key
        return best_q

    async def worker() -> None:
        while unfinished:
            q = pick_query()
            if q is None:
                if not unfinished:
                    break
                wake.clear()
                await wake.wait()  # other workers may bring new candidates
                continue
            _, peer = heapq.heappop(candidates[q])
            # piggy-back other queries that have not asked this peer yet, nearest-first
            extra = heapq.nsmallest(max(0, queries_per_call - 1),
                                    (o for o in unfinished if o != q and peer not in visited[o]), key=peer.__xor__)
            batch = [q] + extra
            for o in batch:
                visited[o].add(peer)
                active[o] += 1
            try:
                response = await get_neighbors(peer, batch)
            except asyncio.CancelledError:
                raise
            except Exception:
                response = {}
            for o in batch:
                active[o] -= 1
                if o not in unfinished:
                    continue
                neighbors, should_stop = response.get(o, ((), False))
                seen, best, frontier = known[o], nearest[o], candidates[o]
                for n in neighbors:
                    if n in seen:
                        continue
                    seen.add(n)
                    d = o ^ n
                    if len(best) < beam_size:
                        heapq.heappush(frontier, (d, n))
                        heapq.heappush(best, (-d, n))
                    elif d <= -best[0][0]:
                        heapq.heappush(frontier, (d, n))
                        heapq.heappushpop(best, (-d, n))
                if should_stop:
                    finish(o)
            wake.set()

    workers = [asyncio.create_task(worker()) for _ in range(max(1, num_workers))]
    finished_wait = asyncio.create_task(search_finished.wait())
    try:
        # every worker parks only while some query is still active elsewhere; the last one to idle finishes them
        await asyncio.wait(workers + [finished_wait], return_when=asyncio.FIRST_COMPLETED)
        while unfinished:
            if all(w.done() for w in workers):
                for q in list(unfinished):
                    finish(q)
                break
            await asyncio.wait([w for w in workers if not w.done()], timeout=0.05, return_when=asyncio.FIRST_COMPLETED)
            if sum(active.values()) == 0:
                pick_query()  # finishes queries that ran dry while everyone was parked
                wake.set()
        if await_all_tasks and pending_tasks:
            await asyncio.gather(*list(pending_tasks), return_exceptions=True)
    finally:
        finished_wait.cancel()
        for w in workers:
            w.cancel()
    result_nearest = {q: [n for _, n in heapq.nlargest(beam_size, nearest[q])] for q in queries}
    return result_nearest, visited

"""``MoEBeamSearcher``: find the best-scoring live experts of a grid by walking DHT prefix dictionaries.

Experts live on a grid ``prefix.i.j...``; the gating network scores every coordinate of every dimension and an
expert's score is the sum of its coordinates' scores. The search keeps the ``beam_size`` best prefixes per
dimension; each DHT prefix entry maps "next coordinate" to one example expert below it, so that only
``O(beam_size * dims)`` DHT reads are needed however sparse the grid is. Misses can be written back as short-lived
"nothing here" records (negative caching) so that other peers skip dead prefixes
(reference: hivemind/moe/client/beam_search.py:26-401).
"""
from __future__ import annotations

import asyncio
import heapq
from collections import deque
from functools import partial
from typing import Deque, Dict, Iterator, List, Optional, Sequence, Set, Tuple, Union

from hivemind_b200.utils.asyncio import spawn
from hivemind_b200.dht import DHT, DHTNode
from hivemind_b200.moe.client.expert import RemoteExpert, batch_create_remote_experts, create_remote_experts
from hivemind_b200.moe.expert_uid import (FLAT_EXPERT, PREFIX_PATTERN, UID_DELIMITER, Coordinate, ExpertInfo,
                                          ExpertPrefix, ExpertUID, Score, is_valid_prefix, is_valid_uid)
from hivemind_b200.p2p import PeerID
from hivemind_b200.utils import DHTExpiration, MPFuture, ValueWithExpiration, get_dht_time, get_logger

logger = get_logger(__name__)

BeamEntry = Tuple[Score, ExpertPrefix, Dict[Coordinate, ExpertInfo]]


class MoEBeamSearcher:
    """
    :param dht: a running DHT
    :param uid_prefix: experts' common prefix, e.g. ``"ffn_expert."``
    :param grid_size: number of coordinates along each grid dimension
    :param num_workers: concurrent DHT requests per search
    :param negative_caching: store "no such prefix" records for ``cache_expiration`` seconds after a miss
    """

    def __init__(self, dht: DHT, uid_prefix: ExpertPrefix, grid_size: Sequence[int], num_workers: Optional[int] = None,
                 negative_caching: bool = True, cache_expiration: DHTExpiration = 300, **kwargs):
        if not uid_prefix.endswith(UID_DELIMITER):
            uid_prefix += UID_DELIMITER
            logger.info(f"Prefix must end with '{UID_DELIMITER}'. Changing to {uid_prefix}")
        assert is_valid_prefix(uid_prefix), f"Prefix '{uid_prefix}' is invalid."
        self.dht = dht
        self.uid_prefix, self.grid_size = uid_prefix, grid_size
        self.total_grid_size = sum(grid_size)
        self.negative_caching, self.cache_expiration = negative_caching, cache_expiration
        self.num_workers, self.dht_kwargs = num_workers, kwargs

    # ------------------------------------------------------------------ public, thread-side API

    def get_initial_beam(self, scores: Sequence[float], beam_size: int, return_future: bool = False):
        """Up to ``beam_size`` tuples (score, first-level prefix, {next coordinate: example expert}), best first."""
        return self.dht.run_coroutine(
            partial(self._get_initial_beam, prefix=self.uid_prefix, beam_size=beam_size, scores=tuple(scores),
                    negative_caching=self.negative_caching, cache_expiration=self.cache_expiration,
                    num_workers=self.num_workers), return_future)

    def get_active_successors(self, prefixes: List[ExpertPrefix], grid_size: Optional[int] = None,
                              return_future: bool = False):
        """For each prefix: {live next coordinate: example expert}; an unknown prefix gives an empty dict."""
        assert not isinstance(prefixes, str), "Please send a list / tuple of expert prefixes."
        for prefix in prefixes:
            assert is_valid_prefix(prefix), f"prefix '{prefix}' is invalid, it must follow {PREFIX_PATTERN.pattern}"
        return self.dht.run_coroutine(
            partial(self._get_active_successors, prefixes=list(prefixes), grid_size=grid_size,
                    negative_caching=self.negative_caching, cache_expiration=self.cache_expiration,
                    num_workers=self.num_workers), return_future=return_future)

    def find_best_experts(self, grid_scores: Sequence[Sequence[float]], beam_size: int, return_future: bool = False
                          ) -> Union[List[RemoteExpert], MPFuture]:
        """Up to ``beam_size`` live experts with the highest summed scores, best first."""
        assert len(grid_scores) == len(self.grid_size) and beam_size > 0
        found = self.dht.run_coroutine(
            partial(self._find_best_experts, prefix=self.uid_prefix, beam_size=beam_size,
                    grid_scores=[tuple(map(float, s)) for s in grid_scores], negative_caching=self.negative_caching,
                    cache_expiration=self.cache_expiration, num_workers=self.num_workers), return_future)
        return create_remote_experts(found, self.dht, return_future)

    def batch_find_best_experts(self, batch_grid_scores: Sequence[Sequence[Sequence[float]]], beam_size: int,
                                return_future: bool = False):
        """``find_best_experts`` for every row of a batch; ``batch_grid_scores[dim]`` is ``[batch, grid_size[dim]]``."""
        found = self.dht.run_coroutine(
            partial(self._batch_find_best_experts, prefix=self.uid_prefix, batch_grid_scores=batch_grid_scores,
                    beam_size=beam_size, negative_caching=self.negative_caching,
                    cache_expiration=self.cache_expiration, num_workers=self.num_workers), return_future)
        return batch_create_remote_experts(found, self.dht, return_future)

    # ------------------------------------------------------------------ coroutines on the DHT loop

    @staticmethod
    def _store_negative(node: DHTNode, prefix: ExpertPrefix, cache_expiration: DHTExpiration) -> None:
        logger.debug(f"DHT negative caching: storing a 'no prefix' entry for {prefix}")
        spawn(node.store(prefix, subkey=FLAT_EXPERT, value=None,
                                       expiration_time=get_dht_time() + cache_expiration))

    @staticmethod
    def _select_valid_entries(entry, grid_size: Optional[float] = None) -> Dict[Coordinate, ExpertInfo]:
        """Keep the well-formed ``coordinate -> (uid, peer id)`` items of a prefix dictionary."""
        if not isinstance(entry, ValueWithExpiration) or not isinstance(entry.value, dict):
            return {}
        valid = {}
        for coord, item in entry.value.items():
            if not isinstance(coord, Coordinate) or isinstance(coord, bool):
                continue
            if grid_size is not None and not (0 <= coord < grid_size):
                continue
            value = item.value if isinstance(item, ValueWithExpiration) else None
            if isinstance(value, (tuple, list)) and len(value) == 2 and isinstance(value[0], str) \
                    and is_valid_uid(value[0]) and isinstance(value[1], str):
                valid[coord] = ExpertInfo(uid=value[0], peer_id=PeerID.from_base58(value[1]))
        return valid

    @staticmethod
    async def _get_initial_beam(dht: DHT, node: DHTNode, prefix: ExpertPrefix, beam_size: int,
                                scores: Tuple[float, ...], negative_caching: bool, cache_expiration: DHTExpiration,
                                num_workers: Optional[int] = None) -> List[BeamEntry]:
        num_workers = num_workers or dht.num_workers or beam_size
        beam: List[BeamEntry] = []
        order = sorted(range(len(scores)), key=scores.__getitem__)  # worst ... best; pop() takes the best
        in_flight: Deque[Tuple[Coordinate, ExpertPrefix, asyncio.Task]] = deque()
        try:
            while len(beam) < beam_size and (order or in_flight):
                while order and len(in_flight) < num_workers:
                    coord = order.pop()
                    candidate = f"{prefix}{coord}{UID_DELIMITER}"
                    in_flight.append((coord, candidate, asyncio.create_task(node.get(candidate))))
                coord, candidate, task = in_flight.popleft()  # strictly in score order
                entry = await task
                if entry is not None and isinstance(entry.value, dict):
                    successors = MoEBeamSearcher._select_valid_entries(entry)
                    if successors:
                        beam.append((scores[coord], candidate, successors))
                elif entry is None and negative_caching:
                    MoEBeamSearcher._store_negative(node, candidate, cache_expiration)
        finally:
            for _, _, task in in_flight:
                task.cancel()
        return beam

    @staticmethod
    async def _get_active_successors(dht: DHT, node: DHTNode, prefixes: List[ExpertPrefix], grid_size: Optional[int],
                                     negative_caching: bool, cache_expiration: DHTExpiration,
                                     num_workers: Optional[int] = None) -> Dict[ExpertPrefix, Dict[Coordinate, ExpertInfo]]:
        limit = grid_size or float("inf")
        num_workers = num_workers or min(len(prefixes), dht.num_workers or len(prefixes))
        responses = await node.get_many(keys=prefixes, num_workers=num_workers)
        successors = {}
        for prefix, found in responses.items():
            successors[prefix] = MoEBeamSearcher._select_valid_entries(found, limit)
            if not successors[prefix] and negative_caching:
                MoEBeamSearcher._store_negative(node, prefix, cache_expiration)
        return successors

    @classmethod
    async def _find_best_experts(cls, dht: DHT, node: DHTNode, prefix: str, grid_scores: List[Tuple[float, ...]],
                                 beam_size: int, negative_caching: bool, cache_expiration: DHTExpiration,
                                 num_workers: Optional[int] = None) -> List[ExpertInfo]:
        num_workers = num_workers or min(beam_size, dht.num_workers or beam_size)
        beam = await cls._get_initial_beam(dht, node, prefix, beam_size, grid_scores[0], negative_caching,
                                           cache_expiration, min(beam_size, num_workers))
        top: List[Tuple[Score, ExpertInfo]] = []  # min-heap holding the beam_size best experts seen so far
        seen: Set[ExpertUID] = set()

        def absorb(current_beam: List[BeamEntry]) -> None:
            for score, info in cls._iterate_matching_experts(current_beam, grid_scores):
                if info.uid in seen:
                    continue
                seen.add(info.uid)
                if len(top) < beam_size:
                    heapq.heappush(top, (score, info))
                else:
                    heapq.heappushpop(top, (score, info))

        for dim in range(1, len(grid_scores) - 1):
            absorb(beam)
            dim_scores = grid_scores[dim]
            expansions = heapq.nlargest(beam_size, (
                (prefix_score + dim_scores[coord], f"{beam_prefix}{coord}{UID_DELIMITER}")
                for prefix_score, beam_prefix, suffixes in beam for coord in suffixes.keys()
                if isinstance(coord, int) and 0 <= coord < len(dim_scores)))
            if not expansions:
                beam = []
                break
            next_prefixes = [p for _, p in expansions]
            successors = await cls._get_active_successors(dht, node, next_prefixes, grid_size=None,
                                                          negative_caching=negative_caching,
                                                          cache_expiration=cache_expiration, num_workers=num_workers)
            beam = [(score, p, successors[p]) for score, p in expansions if successors.get(p)]
            if not beam:
                logger.warning(f"Beam search had to terminate prematurely because of empty beam (dim {dim})")
                break
        absorb(beam)
        return [info for _, info in sorted(top, key=lambda pair: pair[0], reverse=True)]

    @staticmethod
    def _iterate_matching_experts(beam: List[BeamEntry], grid_scores: Sequence[Sequence[float]]
                                  ) -> Iterator[Tuple[Score, ExpertInfo]]:
        """Yield (full score, expert) for every example expert hanging off the beam that fits the grid."""
        ndim = len(grid_scores)
        for score, _, suffixes in beam:
            for coord, match in suffixes.items():
                if ndim == 1 and coord == FLAT_EXPERT:
                    yield score, match
                    continue
                if not isinstance(match.uid, ExpertUID) or match.uid.count(UID_DELIMITER) != ndim:
                    logger.warning(f"Found incompatible expert UID: {match.uid}")
                    continue
                coords = match.uid.split(UID_DELIMITER)[1:]
                if all(c.isdigit() and 0 <= int(c) < len(grid_scores[i]) for i, c in enumerate(coords)):
                    yield sum(dim_scores[int(c)] for dim_scores, c in zip(grid_scores, coords)), match
                else:
                    logger.warning(f"Found incompatible expert coordinates: {coords}")

    @classmethod
    async def _batch_find_best_experts(cls, dht: DHT, node: DHTNode, prefix: str,
                                       batch_grid_scores: Sequence[Sequence[Sequence[float]]], beam_size: int,
                                       negative_caching: bool, cache_expiration: DHTExpiration,
                                       num_workers: Optional[int]) -> Sequence[Sequence[ExpertInfo]]:
        batch_size = len(batch_grid_scores[0])
        per_sample = [[tuple(map(float, dim_scores[i])) for dim_scores in batch_grid_scores] for i in range(batch_size)]
        return await asyncio.gather(*(
            cls._find_best_experts(dht, node, prefix, scores, beam_size, negative_caching, cache_expiration, num_workers)
            for scores in per_sample))

"""Forming all-reduce groups without a coordinator.

Wire protocol and ordering rule (hivemind/averaging/matchmaking.py:24-550): every averager that wants a group
*declares* itself under the current group key in the DHT, with an expiration equal to the time at which it wants to
start. A peer only asks peers that come *before* it in (expiration, peer id) order to lead it, so the peer with the
earliest expiration ends up leading. A leader answers ``ACCEPTED`` or a rejection code; it assembles the group at once
when ``target_group_size`` is reached, or at its own expiration if at least ``min_group_size`` peers are present, and
otherwise disbands. A leader that is itself accepted by an earlier peer lets its followers go and names that peer as
``suggested_leader``. ``BEGIN_ALLREDUCE`` carries the shuffled peer order, a random group id and every member's
``gather`` blob. Two peers that ask each other at the same moment are untangled by ``request_timeout``.

How this implementation is organised: one ``_Search`` object holds everything that belongs to a single
``look_for_group`` call (the result future, the followers, the current leader, the declared expiration, the
candidates already tried). The *courting loop* declares this peer, asks better-placed candidates one by one, and
leads when its own time is up; ``rpc_join_group`` handlers of would-be followers read and update the same
``_Search``. A single lock orders "I accept a follower" against "I am accepted as a follower".
"""
from __future__ import annotations

import asyncio
import contextlib
import random
from math import isfinite
from typing import AsyncIterator, Dict, List, Optional, Set, Tuple, Type

from hivemind_b200.averaging.control import StepControl
from hivemind_b200.averaging.group_info import GroupInfo
from hivemind_b200.averaging.key_manager import GroupKey, GroupKeyManager
from hivemind_b200.dht import DHT, DHTID
from hivemind_b200.p2p import P2P, P2PContext, P2PDaemonError, P2PHandlerError, PeerID, ServicerBase
from hivemind_b200.proto import averaging_pb2
from hivemind_b200.utils import DHTExpiration, get_dht_time, get_logger
from hivemind_b200.utils.asyncio import anext, cancel_and_wait

logger = get_logger(__name__)
_Reply = averaging_pb2.MessageFromLeader
_CANDIDATE_POLL_SECONDS = 0.05  # pause between two looks at the DHT while nobody suitable is declared


class MatchmakingException(Exception):
    """Group formation failed in a way that the caller may retry."""


class _Search:
    """State of one ``look_for_group`` call."""

    def __init__(self, step: StepControl):
        self.step = step
        self.outcome: asyncio.Future = asyncio.get_event_loop().create_future()  # GroupInfo
        self.followers: Dict[PeerID, averaging_pb2.JoinRequest] = {}
        self.leader: Optional[PeerID] = None            # set while somebody has accepted us
        self.expiration: DHTExpiration = float("inf")   # what we declared; inf = nothing declared right now
        self.declared_key: Optional[GroupKey] = None
        self.end_time: DHTExpiration = step.deadline if step.deadline is not None else float("inf")
        self.tried: Set[Tuple[PeerID, DHTExpiration]] = set()
        self.changed = asyncio.Event()                   # pulsed when outcome, leader or followers change
        self.saw_candidates = False

    def pulse(self) -> None:
        self.changed.set()

    def desired_expiration(self, min_matchmaking_time: float) -> DHTExpiration:
        return float(min(max(self.step.scheduled_time, get_dht_time() + min_matchmaking_time), self.end_time))


class Matchmaking:
    def __init__(self, p2p: P2P, schema_hash: bytes, dht: DHT, *, servicer_type: Type[ServicerBase], prefix: str,
                 target_group_size: Optional[int], min_group_size: int, min_matchmaking_time: float,
                 request_timeout: float, client_mode: bool, initial_group_bits: str = ""):
        if "." in prefix:
            raise ValueError("the averager prefix must not contain '.'")
        if not issubclass(servicer_type, ServicerBase):
            raise TypeError("servicer_type must derive from ServicerBase")
        if request_timeout is None or request_timeout >= min_matchmaking_time:
            logger.warning("request_timeout should be shorter than min_matchmaking_time: two peers that ask each other "
                           "at the same moment only come apart when a request times out")
        self._p2p, self._servicer_type, self._prefix = p2p, servicer_type, prefix
        self.peer_id = p2p.peer_id
        self.schema_hash = schema_hash
        self.group_key_manager = GroupKeyManager(dht, prefix, initial_group_bits, target_group_size)
        self.target_group_size, self.min_group_size = target_group_size, min_group_size
        self.min_matchmaking_time, self.request_timeout = min_matchmaking_time, request_timeout
        self.client_mode = client_mode
        self._one_search_at_a_time = asyncio.Lock()
        self._membership = asyncio.Lock()   # accepting a follower vs. being accepted as one
        self._search: Optional[_Search] = None

    # ------------------------------------------------------------------------------------------ status
    @property
    def is_looking_for_group(self) -> bool:
        return self._search is not None

    @property
    def current_leader(self) -> Optional[PeerID]:
        return self._search.leader if self._search is not None else None

    @property
    def current_followers(self) -> Dict[PeerID, averaging_pb2.JoinRequest]:
        return self._search.followers if self._search is not None else {}

    def __repr__(self) -> str:
        if self._search is None:
            role = "idle"
        elif self._search.leader is not None:
            role = f"following {self._search.leader}"
        else:
            role = f"leading {len(self._search.followers)} followers"
        return (f"{type(self).__name__}(peer_id={self.peer_id}, {role}, key={self.group_key_manager.current_key}, "
                f"client_mode={self.client_mode})")

    def _full(self, search: _Search) -> bool:
        return self.target_group_size is not None and len(search.followers) + 1 >= self.target_group_size

    def _viable(self, search: _Search) -> bool:
        return len(search.followers) + 1 >= self.min_group_size

    # ------------------------------------------------------------------------------------------ entry point
    async def look_for_group(self, step: StepControl) -> Optional[GroupInfo]:
        """Find or lead a group before the step's deadline. Returns None if no group could be formed in time."""
        if self._one_search_at_a_time.locked():
            logger.info("look_for_group is already running; this call waits for that search to end")
        async with self._one_search_at_a_time:
            search = self._search = _Search(step)
            courting = asyncio.create_task(self._court(search))
            try:
                return await asyncio.wait_for(asyncio.shield(search.outcome), timeout=step.get_timeout())
            except asyncio.TimeoutError:
                return None
            finally:
                await cancel_and_wait(courting)
                if not search.outcome.done():
                    search.outcome.cancel()
                search.pulse()
                # followers' handlers notice that the search is over, answer them and remove themselves
                while search.followers:
                    search.changed.clear()
                    with contextlib.suppress(asyncio.TimeoutError):
                        await asyncio.wait_for(search.changed.wait(), timeout=1.0)
                await self._retract_declaration(search)
                self._search = None

    async def _court(self, search: _Search) -> None:
        """Declare this peer, ask better-placed candidates to lead it, lead when its own time is up; repeat."""
        try:
            while not search.outcome.done():
                if not self.client_mode:
                    await self._declare(search)
                else:
                    search.expiration = search.desired_expiration(self.min_matchmaking_time)
                search.saw_candidates = False
                while get_dht_time() < search.expiration and not search.outcome.done():
                    candidate = await self._next_candidate(search)
                    if candidate is None:
                        pause = min(_CANDIDATE_POLL_SECONDS, max(0.0, search.expiration - get_dht_time()))
                        search.changed.clear()
                        with contextlib.suppress(asyncio.TimeoutError):
                            await asyncio.wait_for(search.changed.wait(), timeout=pause)
                        continue
                    await self._propose(search, candidate)
                if search.outcome.done():
                    return
                # our own moment has come: go ahead with whoever joined, or start over
                async with self._membership:
                    if search.outcome.done():
                        return
                    if not self.client_mode and self._viable(search):
                        await self._assemble_as_leader(search)
                        return
                    self._release_followers(search)
                if not search.saw_candidates and not self.client_mode:
                    await self.group_key_manager.update_key_on_not_enough_peers()
                if get_dht_time() >= search.end_time:
                    return
        except asyncio.CancelledError:
            raise
        except Exception as e:
            if not search.outcome.done():
                search.outcome.set_exception(e)
                search.pulse()

    async def _declare(self, search: _Search) -> None:
        search.declared_key = self.group_key_manager.current_key
        search.expiration = search.desired_expiration(self.min_matchmaking_time)
        await self.group_key_manager.declare_averager(search.declared_key, self.peer_id, expiration_time=search.expiration)

    async def _retract_declaration(self, search: _Search) -> None:
        key, expiration = search.declared_key, search.expiration
        search.declared_key, search.expiration = None, float("inf")
        if key is not None and expiration > get_dht_time():
            with contextlib.suppress(Exception):
                await asyncio.shield(self.group_key_manager.declare_averager(key, self.peer_id, expiration,
                                                                             looking_for_group=False))

    async def _next_candidate(self, search: _Search) -> Optional[PeerID]:
        """The declared peer that precedes us most clearly in (expiration, id) order and was not asked yet."""
        listing = await self.group_key_manager.get_averagers(self.group_key_manager.current_key, only_active=True)
        # a client-mode peer never leads, so nobody is "behind" it: it may ask any declared peer, whereas a regular peer
        # only asks those whose turn to lead comes before its own (hivemind/averaging/matchmaking.py:477-480, where a
        # client's own expiration stays infinite because it never declares itself, and :254-260 for the promise)
        mine = (float("inf"), b"") if self.client_mode else (search.expiration, self.peer_id.to_bytes())
        best: Optional[Tuple[DHTExpiration, bytes, PeerID]] = None
        for peer, expiration in listing:
            if peer == self.peer_id:
                continue
            search.saw_candidates = True
            if (peer, expiration) in search.tried or expiration > search.end_time:
                continue
            rank = (expiration, peer.to_bytes())
            if rank < mine and (best is None or rank < best[:2]):
                best = (expiration, peer.to_bytes(), peer)
        if best is None:
            return None
        search.tried.add((best[2], best[0]))
        return best[2]

    # ------------------------------------------------------------------------------------------ follower side
    def _promised_start(self, search: _Search) -> DHTExpiration:
        """The latest moment by which we promise a leader to begin the all-reduce."""
        if isfinite(search.expiration) and not self.client_mode:
            return search.expiration
        # nothing was declared (client mode): promise afresh, so that a leader that declared after our search began
        # does not take us for a peer that ought to be leading it
        return search.desired_expiration(self.min_matchmaking_time)

    async def _propose(self, search: _Search, leader: PeerID) -> Optional[GroupInfo]:
        """Ask ``leader`` to take us in. Returns the group if one was assembled with us in it."""
        stream: Optional[AsyncIterator[averaging_pb2.MessageFromLeader]] = None
        try:
            async with self._membership:
                if search.outcome.done():
                    return None
                stub = self._servicer_type.get_stub(self._p2p, leader, namespace=self._prefix)
                stream = await stub.rpc_join_group(averaging_pb2.JoinRequest(
                    schema_hash=self.schema_hash, expiration=self._promised_start(search), client_mode=self.client_mode,
                    gather=search.step.data_for_gather, group_key=self.group_key_manager.current_key))
                verdict = await asyncio.wait_for(anext(stream), timeout=self.request_timeout)
                if verdict.code == averaging_pb2.ACCEPTED:
                    search.leader = leader
                    self._release_followers(search)  # they are told to try our new leader
            if verdict.code != averaging_pb2.ACCEPTED:
                logger.debug(f"{self.peer_id}: {leader} declined to lead us "
                             f"({averaging_pb2.MessageCode.Name(verdict.code)})")
                return None
            logger.debug(f"{self.peer_id}: accepted by {leader}, waiting for the group to fill")
            patience = max(0.0, search.expiration - get_dht_time()) + self.request_timeout
            verdict = await asyncio.wait_for(anext(stream), timeout=patience)
            if verdict.code == averaging_pb2.BEGIN_ALLREDUCE:
                async with self._membership:
                    return await self._adopt_group(search, leader, verdict)
            if verdict.code in (averaging_pb2.GROUP_DISBANDED, averaging_pb2.CANCELLED) and verdict.suggested_leader:
                elsewhere = PeerID(verdict.suggested_leader)
                if elsewhere != self.peer_id:
                    logger.debug(f"{self.peer_id}: {leader} let its group go and points to {elsewhere}")
                    search.leader = None
                    await _close_stream(stream)
                    stream = None
                    return await self._propose(search, elsewhere)
            logger.debug(f"{self.peer_id}: {leader} ended the group ({averaging_pb2.MessageCode.Name(verdict.code)})")
            return None
        except asyncio.TimeoutError:
            logger.debug(f"{self.peer_id}: no answer from {leader} within {self.request_timeout} s")
            return None
        except (P2PDaemonError, P2PHandlerError, StopAsyncIteration) as e:
            logger.debug(f"{self.peer_id}: asking {leader} failed: {e!r}")
            return None
        finally:
            if search.leader is not None:
                search.leader = None
                search.pulse()
            if stream is not None:
                await _close_stream(stream)

    async def _adopt_group(self, search: _Search, leader: PeerID, msg: averaging_pb2.MessageFromLeader) -> GroupInfo:
        if search.outcome.done():
            raise MatchmakingException("a group was announced to us after our search had ended")
        if search.leader != leader:
            raise MatchmakingException(f"{leader} announced a group but we follow {search.leader}")
        members = tuple(PeerID(raw) for raw in msg.ordered_peer_ids)
        if self.peer_id not in members or len(members) != len(msg.gathered):
            raise MatchmakingException("the leader announced a malformed group")
        group = GroupInfo(msg.group_id, members, tuple(msg.gathered))
        await self.group_key_manager.update_key_on_group_assembled(group)
        search.outcome.set_result(group)
        search.pulse()
        return group

    # ------------------------------------------------------------------------------------------ leader side
    async def rpc_join_group(self, request: averaging_pb2.JoinRequest, context: P2PContext
                             ) -> AsyncIterator[averaging_pb2.MessageFromLeader]:
        """Serve a peer that asks us to lead it: reject, or accept and later tell it how the group turned out."""
        suitor, search = context.remote_id, None
        try:
            async with self._membership:
                search = self._search
                refusal = self._reason_to_refuse(search, request, suitor)
                if refusal is not None:
                    search = None
                    yield refusal
                    return
                search.followers[suitor] = request
                yield _Reply(code=averaging_pb2.ACCEPTED)
                if self._full(search):
                    await self._assemble_as_leader(search)  # complete: begin right away

            # until the group is settled, we are taken in elsewhere, or our declared time has come
            while not search.outcome.done() and search.leader is None and suitor in search.followers:
                remaining = search.expiration - get_dht_time()
                if remaining <= 0:
                    break
                search.changed.clear()
                with contextlib.suppress(asyncio.TimeoutError):
                    await asyncio.wait_for(search.changed.wait(), timeout=remaining if isfinite(remaining) else None)
            if not search.outcome.done() and search.leader is None and suitor in search.followers:
                async with self._membership:
                    if search.outcome.done():
                        pass  # settled while we were waiting for the lock
                    elif self._viable(search) and self._search is search:
                        await self._assemble_as_leader(search)  # time is up: a smaller group will do
                    else:
                        self._release_followers(search)

            group = search.outcome.result() if (search.outcome.done() and not search.outcome.cancelled()
                                                and search.outcome.exception() is None) else None
            if search.leader is not None or group is None or suitor not in group:
                elsewhere = search.leader.to_bytes() if search.leader is not None else b""
                yield _Reply(code=averaging_pb2.GROUP_DISBANDED, suggested_leader=elsewhere)
                return
            yield _Reply(code=averaging_pb2.BEGIN_ALLREDUCE, group_id=group.group_id, gathered=group.gathered,
                         ordered_peer_ids=[member.to_bytes() for member in group.peer_ids])
        except asyncio.CancelledError:
            return  # the suitor hung up
        except Exception as e:
            logger.exception(e)
            yield _Reply(code=averaging_pb2.INTERNAL_ERROR)
        finally:
            if search is not None:
                search.followers.pop(suitor, None)
                search.pulse()

    def _reason_to_refuse(self, search: Optional[_Search], request: averaging_pb2.JoinRequest, suitor: PeerID
                          ) -> Optional[_Reply]:
        if search is None or search.outcome.done():
            return _Reply(code=averaging_pb2.NOT_LOOKING_FOR_GROUP)
        well_formed = (isinstance(request.schema_hash, bytes) and len(request.schema_hash) > 0
                       and isinstance(request.expiration, DHTExpiration) and isfinite(request.expiration)
                       and isinstance(request.group_key, GroupKey))
        if not well_formed or self.client_mode:
            return _Reply(code=averaging_pb2.PROTOCOL_VIOLATION)
        if request.schema_hash != self.schema_hash:
            return _Reply(code=averaging_pb2.BAD_SCHEMA_HASH)
        if request.group_key != self.group_key_manager.current_key:
            return _Reply(code=averaging_pb2.BAD_GROUP_KEY)
        if search.declared_key is None:
            return _Reply(code=averaging_pb2.NOT_DECLARED)
        if search.expiration > (request.expiration or float("inf")):
            return _Reply(code=averaging_pb2.BAD_EXPIRATION_TIME)  # it should be leading us, not the other way round
        if search.leader is not None:
            return _Reply(code=averaging_pb2.NOT_A_LEADER, suggested_leader=search.leader.to_bytes())
        if suitor == self.peer_id or suitor in search.followers:
            return _Reply(code=averaging_pb2.DUPLICATE_PEER_ID)
        if self._full(search):
            return _Reply(code=averaging_pb2.GROUP_IS_FULL)
        return None

    async def _assemble_as_leader(self, search: _Search) -> GroupInfo:
        """Close the group: shuffle the member order, draw a group id, let everybody who waits know."""
        if self.client_mode or search.outcome.done():
            raise MatchmakingException("cannot assemble a group now")
        members: List[PeerID] = [*search.followers, self.peer_id]
        random.shuffle(members)
        blobs = tuple(search.step.data_for_gather if m == self.peer_id else search.followers[m].gather for m in members)
        group = GroupInfo(DHTID.generate().to_bytes(), tuple(members), blobs)
        logger.debug(f"{self.peer_id}: leading a group of {len(members)}")
        await self.group_key_manager.update_key_on_group_assembled(group)
        search.outcome.set_result(group)
        search.pulse()
        return group

    def _release_followers(self, search: _Search) -> None:
        """Let the accepted followers go: their handlers see that they are no longer listed and answer them."""
        if search.followers:
            search.followers.clear()
        search.pulse()


async def _close_stream(stream) -> None:
    try:
        await stream.aclose()
    except RuntimeError as e:  # the generator is running in another task that is being cancelled
        logger.debug(e, exc_info=True)

"""Forming all-reduce groups without a coordinator.

Protocol (same messages and ordering rule as hivemind/averaging/matchmaking.py:24-550):
every averager that wants a group *declares* itself under the current group key in the DHT with an expiration = the
time it wants to start. A peer asks only peers that come *before* it in (expiration, peer id) order to lead it, so
the earliest-expiring peer ends up as leader. A leader accepts followers (``ACCEPTED``), and either assembles the
group at once when ``target_group_size`` is reached, or at its own expiration if at least ``min_group_size`` peers
are present, else disbands. A leader that gets accepted by a better leader disbands and redirects its followers
(``GROUP_DISBANDED`` + ``suggested_leader``). ``BEGIN_ALLREDUCE`` carries the shuffled peer order, a random group id
and everybody's ``gather`` blob.

Two-way waiting between peers that ask each other at the same moment is broken by ``request_timeout``.
"""
from __future__ import annotations

import asyncio
import concurrent.futures
import contextlib
import random
from math import isfinite
from typing import AsyncIterator, Dict, Optional, Set, Tuple, Type

from hivemind_b200.averaging.control import StepControl
from hivemind_b200.averaging.group_info import GroupInfo
from hivemind_b200.averaging.key_manager import GroupKey, GroupKeyManager
from hivemind_b200.dht import DHT, DHTID
from hivemind_b200.p2p import P2P, P2PContext, P2PDaemonError, P2PHandlerError, PeerID, ServicerBase
from hivemind_b200.proto import averaging_pb2
from hivemind_b200.utils import DHTExpiration, TimedStorage, get_dht_time, get_logger
from hivemind_b200.utils.asyncio import anext, cancel_and_wait
from hivemind_b200.utils.timed_storage import MAX_DHT_TIME_DISCREPANCY_SECONDS

logger = get_logger(__name__)
_Reply = averaging_pb2.MessageFromLeader


class MatchmakingException(Exception):
    """Group formation failed in a way that the caller may retry."""


class Matchmaking:
    def __init__(self, p2p: P2P, schema_hash: bytes, dht: DHT, *, servicer_type: Type[ServicerBase], prefix: str,
                 target_group_size: Optional[int], min_group_size: int, min_matchmaking_time: float,
                 request_timeout: float, client_mode: bool, initial_group_bits: str = ""):
        assert "." not in prefix, "group prefix must be a string without ."
        if request_timeout is None or request_timeout >= min_matchmaking_time:
            logger.warning("request_timeout should be smaller than min_matchmaking_time; otherwise two peers that "
                           "request each other simultaneously may block until matchmaking times out")
        if not issubclass(servicer_type, ServicerBase):
            raise TypeError("`servicer_type` is expected to be a ServicerBase subclass")
        self._p2p, self._servicer_type, self._prefix = p2p, servicer_type, prefix
        self.peer_id = p2p.peer_id
        self.schema_hash = schema_hash
        self.group_key_manager = GroupKeyManager(dht, prefix, initial_group_bits, target_group_size)
        self.target_group_size, self.min_group_size = target_group_size, min_group_size
        self.min_matchmaking_time, self.request_timeout = min_matchmaking_time, request_timeout
        self.client_mode = client_mode

        self.lock_looking_for_group = asyncio.Lock()
        self.lock_request_join_group = asyncio.Lock()
        self.follower_was_discarded = asyncio.Event()
        self.was_accepted_to_group = asyncio.Event()
        self.assembled_group: asyncio.Future = asyncio.Future()

        self.current_leader: Optional[PeerID] = None  # set while we follow somebody
        self.current_followers: Dict[PeerID, averaging_pb2.JoinRequest] = {}  # peers that we accepted
        self.potential_leaders = PotentialLeaders(self.peer_id, min_matchmaking_time, target_group_size)
        self.step_control: Optional[StepControl] = None

    # ------------------------------------------------------------------------------------------ status
    @property
    def is_looking_for_group(self) -> bool:
        return self.lock_looking_for_group.locked()

    def __repr__(self) -> str:
        state = "idle"
        if self.is_looking_for_group:
            state = f"following {self.current_leader}" if self.current_leader else f"leading {len(self.current_followers)} followers"
        return (f"{type(self).__name__}(peer_id={self.peer_id}, {state}, key={self.group_key_manager.current_key}, "
                f"client_mode={self.client_mode})")

    @contextlib.asynccontextmanager
    async def looking_for_group(self, step_control: StepControl):
        async with self.lock_looking_for_group:
            assert self.step_control is None
            self.step_control = step_control
            try:
                yield
            finally:
                self.step_control = None

    # ------------------------------------------------------------------------------------------ entry point
    async def look_for_group(self, step: StepControl) -> Optional[GroupInfo]:
        """Find or lead a group before the step's deadline. Returns None if no group could be formed in time."""
        if self.is_looking_for_group:
            logger.info("Another look_for_group is already in progress. The current run will be scheduled after"
                        " the existing group is either assembled or disbanded.")
        async with self.looking_for_group(step):
            search_task = asyncio.create_task(self._request_join_potential_leaders(step))
            try:
                return await asyncio.wait_for(self.assembled_group, timeout=step.get_timeout())
            except asyncio.TimeoutError:
                return None
            except BaseException as e:
                if len(self.current_followers) > 0:
                    async with self.lock_request_join_group:
                        await self.leader_disband_group()
                if not self.assembled_group.done():
                    self.assembled_group.set_exception(e)
                raise
            finally:
                await cancel_and_wait(search_task)
                self.assembled_group.cancel()
                while len(self.current_followers) > 0:
                    await self.follower_was_discarded.wait()
                    self.follower_was_discarded.clear()
                # a new future for the next call of look_for_group
                self.assembled_group = asyncio.Future()
                self.was_accepted_to_group.clear()

    async def _request_join_potential_leaders(self, step: StepControl) -> GroupInfo:
        """Ask better-placed peers to lead us, one at a time; lead ourselves when our own time runs out."""
        assert self.is_looking_for_group
        async with self.potential_leaders.begin_search(step, self.group_key_manager, declare=not self.client_mode):
            while True:
                try:
                    next_leader = await self.potential_leaders.pop_next_leader()  # TimeoutError = our declaration expired
                    group = await self._request_join_group(next_leader)
                    if group is not None:
                        return group
                except asyncio.TimeoutError:
                    async with self.lock_request_join_group:
                        if self.assembled_group.done():
                            return self.assembled_group.result()
                        if len(self.current_followers) + 1 >= self.min_group_size:
                            return await self.leader_assemble_group()  # good enough: run with whoever joined
                        if len(self.current_followers) > 0:
                            await self.leader_disband_group()
                        continue  # nobody came: declare again and keep looking
                except (concurrent.futures.CancelledError, asyncio.CancelledError):
                    break
                except Exception as e:
                    if not self.assembled_group.done():
                        self.assembled_group.set_exception(e)
                    raise e

    # ------------------------------------------------------------------------------------------ follower side
    async def _request_join_group(self, leader: PeerID) -> Optional[GroupInfo]:
        """Ask ``leader`` to take us in; returns the assembled group, or None if rejected / disbanded."""
        assert self.is_looking_for_group and self.current_leader is None
        stream: Optional[AsyncIterator[averaging_pb2.MessageFromLeader]] = None
        try:
            async with self.lock_request_join_group:
                leader_stub = self._servicer_type.get_stub(self._p2p, leader, namespace=self._prefix)
                request_expiration_time = self.get_request_expiration_time()
                stream = await leader_stub.rpc_join_group(averaging_pb2.JoinRequest(
                    schema_hash=self.schema_hash, expiration=request_expiration_time, client_mode=self.client_mode,
                    gather=self.step_control.data_for_gather, group_key=self.group_key_manager.current_key))
                message = await asyncio.wait_for(anext(stream), timeout=self.request_timeout)
                if message.code == averaging_pb2.ACCEPTED:
                    logger.debug(f"{self.peer_id} - joining the group of {leader}, waiting for peers")
                    self.current_leader = leader
                    self.was_accepted_to_group.set()
                    if len(self.current_followers) > 0:
                        await self.leader_disband_group()

            if message.code != averaging_pb2.ACCEPTED:
                code = averaging_pb2.MessageCode.Name(message.code)
                logger.debug(f"{self.peer_id} - requested {leader} to be my leader, but got rejected with {code}")
                return None

            async with self.potential_leaders.pause_search():
                time_to_expiration = max(0.0, self.potential_leaders.declared_expiration_time - get_dht_time())
                message = await asyncio.wait_for(anext(stream), time_to_expiration + self.request_timeout)
                if message.code == averaging_pb2.BEGIN_ALLREDUCE:
                    async with self.lock_request_join_group:
                        return await self.follower_assemble_group(leader, message)

            if message.code in (averaging_pb2.GROUP_DISBANDED, averaging_pb2.CANCELLED):
                if message.suggested_leader:
                    suggested_leader = PeerID(message.suggested_leader)
                    if suggested_leader != self.peer_id:
                        logger.debug(f"{self} - leader disbanded group and redirected us to {suggested_leader}")
                        self.current_leader = None
                        try:
                            await stream.aclose()
                        except RuntimeError as e:
                            logger.debug(e, exc_info=True)
                        return await self._request_join_group(suggested_leader)
                logger.debug(f"{self} - leader disbanded group")
                return None

            logger.debug(f"{self} - unexpected message from leader: {averaging_pb2.MessageCode.Name(message.code)}")
            return None
        except asyncio.TimeoutError:
            logger.debug(f"{self} - potential leader {leader} did not respond within {self.request_timeout}")
            return None
        except (P2PDaemonError, P2PHandlerError, StopAsyncIteration) as e:
            logger.debug(f"{self} - failed to request potential leader {leader}: {e!r}")
            return None
        finally:
            self.was_accepted_to_group.clear()
            self.current_leader = None
            if stream is not None:
                try:
                    await stream.aclose()
                except RuntimeError as e:
                    logger.debug(e, exc_info=True)

    def get_request_expiration_time(self) -> float:
        """The latest moment by which we promise to begin all-reduce with a leader."""
        if isfinite(self.potential_leaders.declared_expiration_time):
            return self.potential_leaders.declared_expiration_time
        scheduled_time = max(self.step_control.scheduled_time, get_dht_time() + self.min_matchmaking_time)
        return min(scheduled_time, self.potential_leaders.search_end_time)

    # ------------------------------------------------------------------------------------------ leader side
    async def rpc_join_group(self, request: averaging_pb2.JoinRequest, context: P2PContext
                             ) -> AsyncIterator[averaging_pb2.MessageFromLeader]:
        """Serve a peer that asks us to lead it: reject, or accept and later tell it how the group turned out."""
        try:
            async with self.lock_request_join_group:
                reason_to_reject = self._check_reasons_to_reject(request, context)
                if reason_to_reject is not None:
                    yield reason_to_reject
                    return
                self.current_followers[context.remote_id] = request
                yield _Reply(code=averaging_pb2.ACCEPTED)
                if self.target_group_size is not None and len(self.current_followers) + 1 >= self.target_group_size:
                    await self.leader_assemble_group()  # the group is full: begin right away

            # wait until the group is assembled, disbanded, or we are taken in by another leader
            timeout = max(0.0, self.potential_leaders.declared_expiration_time - get_dht_time())
            accepted_elsewhere = asyncio.create_task(self.was_accepted_to_group.wait())
            try:
                await asyncio.wait({self.assembled_group, accepted_elsewhere}, return_when=asyncio.FIRST_COMPLETED,
                                   timeout=timeout)
            finally:
                accepted_elsewhere.cancel()
            if not self.assembled_group.done() and not self.was_accepted_to_group.is_set():
                async with self.lock_request_join_group:
                    if self.assembled_group.done():
                        pass  # assembled while we were waiting for the lock
                    elif len(self.current_followers) + 1 >= self.min_group_size and self.is_looking_for_group:
                        await self.leader_assemble_group()  # time is up, proceed with a smaller group
                    else:
                        await self.leader_disband_group()

            if (self.was_accepted_to_group.is_set() or not self.assembled_group.done() or self.assembled_group.cancelled()
                    or context.remote_id not in self.assembled_group.result()):
                if self.current_leader is not None:
                    yield _Reply(code=averaging_pb2.GROUP_DISBANDED, suggested_leader=self.current_leader.to_bytes())
                else:
                    yield _Reply(code=averaging_pb2.GROUP_DISBANDED)
                return

            group_info = self.assembled_group.result()
            yield _Reply(code=averaging_pb2.BEGIN_ALLREDUCE, group_id=group_info.group_id,
                         ordered_peer_ids=[item.to_bytes() for item in group_info.peer_ids], gathered=group_info.gathered)
        except (concurrent.futures.CancelledError, asyncio.CancelledError):
            return  # the follower hung up
        except Exception as e:
            logger.exception(e)
            yield _Reply(code=averaging_pb2.INTERNAL_ERROR)
        finally:
            self.current_followers.pop(context.remote_id, None)
            self.follower_was_discarded.set()

    def _check_reasons_to_reject(self, request: averaging_pb2.JoinRequest, context: P2PContext) -> Optional[_Reply]:
        if not self.is_looking_for_group or self.assembled_group.done():
            return _Reply(code=averaging_pb2.NOT_LOOKING_FOR_GROUP)
        if not isinstance(request.schema_hash, bytes) or len(request.schema_hash) == 0 \
                or not isinstance(request.expiration, DHTExpiration) or not isfinite(request.expiration) \
                or self.client_mode or not isinstance(request.group_key, GroupKey):
            return _Reply(code=averaging_pb2.PROTOCOL_VIOLATION)
        if request.schema_hash != self.schema_hash:
            return _Reply(code=averaging_pb2.BAD_SCHEMA_HASH)
        if request.group_key != self.group_key_manager.current_key:
            return _Reply(code=averaging_pb2.BAD_GROUP_KEY)
        if self.potential_leaders.declared_group_key is None:
            return _Reply(code=averaging_pb2.NOT_DECLARED)
        if self.potential_leaders.declared_expiration_time > (request.expiration or float("inf")):
            return _Reply(code=averaging_pb2.BAD_EXPIRATION_TIME)
        if self.current_leader is not None:
            return _Reply(code=averaging_pb2.NOT_A_LEADER, suggested_leader=self.current_leader.to_bytes())
        if context.remote_id == self.peer_id or context.remote_id in self.current_followers:
            return _Reply(code=averaging_pb2.DUPLICATE_PEER_ID)
        if self.target_group_size is not None and len(self.current_followers) + 1 >= self.target_group_size:
            return _Reply(code=averaging_pb2.GROUP_IS_FULL)
        return None

    async def leader_assemble_group(self) -> GroupInfo:
        """Close the group: fix the (shuffled) peer order, draw a group id, publish the result to the waiters."""
        assert self.lock_looking_for_group.locked() and self.lock_request_join_group.locked() and not self.client_mode
        assert not self.assembled_group.done()
        group_id = DHTID.generate().to_bytes()
        ordered_peer_ids = list(self.current_followers)
        ordered_peer_ids.append(self.peer_id)
        random.shuffle(ordered_peer_ids)
        gathered = tuple(self.step_control.data_for_gather if peer_id == self.peer_id else self.current_followers[peer_id].gather
                         for peer_id in ordered_peer_ids)
        logger.debug(f"{self.peer_id} - assembled group of {len(ordered_peer_ids)} peers")
        group_info = GroupInfo(group_id, tuple(ordered_peer_ids), gathered)
        await self.group_key_manager.update_key_on_group_assembled(group_info)
        self.assembled_group.set_result(group_info)
        return group_info

    async def follower_assemble_group(self, leader: PeerID, msg: averaging_pb2.MessageFromLeader) -> GroupInfo:
        """Adopt the group announced by our leader."""
        assert self.lock_looking_for_group.locked() and self.lock_request_join_group.locked()
        assert not self.assembled_group.done()
        assert self.current_leader == leader, f"averager does not follow {leader} (actual: {self.current_leader})"
        group_id = msg.group_id
        ordered_peer_ids = [PeerID(item) for item in msg.ordered_peer_ids]
        assert self.peer_id in ordered_peer_ids, "Leader sent us group_peer_ids that does not contain us!"
        assert len(ordered_peer_ids) == len(msg.gathered)
        logger.debug(f"{self.peer_id} - follower assembled group with leader {leader}")
        group_info = GroupInfo(group_id, tuple(ordered_peer_ids), tuple(msg.gathered))
        await self.group_key_manager.update_key_on_group_assembled(group_info)
        self.assembled_group.set_result(group_info)
        return group_info

    async def leader_disband_group(self) -> None:
        """Let all accepted followers go (their handlers notice that they are no longer in ``current_followers``)."""
        assert self.lock_request_join_group.locked() and not self.client_mode
        self.current_followers.clear()


class PotentialLeaders:
    """Keeps our own declaration fresh in the DHT and maintains a queue of peers that could lead us."""

    def __init__(self, peer_id: PeerID, min_matchmaking_time: DHTExpiration, target_group_size: Optional[int]):
        self.peer_id, self.min_matchmaking_time = peer_id, min_matchmaking_time
        self.target_group_size = target_group_size
        self.running, self.update_triggered, self.update_finished = asyncio.Event(), asyncio.Event(), asyncio.Event()
        self.declared_expiration, self.lock_search, self.lock_declare = asyncio.Event(), asyncio.Lock(), asyncio.Lock()
        self.leader_queue = TimedStorage[PeerID, DHTExpiration]()
        self.past_attempts: Set[Tuple[PeerID, DHTExpiration]] = set()
        self.declared_expiration_time = float("inf")
        self.declared_group_key: Optional[GroupKey] = None
        self.max_assured_time = float("-inf")
        self.search_end_time = float("inf")

    @contextlib.asynccontextmanager
    async def begin_search(self, step: StepControl, key_manager: GroupKeyManager, declare: bool = True):
        async with self.lock_search:
            self.running.set()
            self.search_end_time = step.deadline if step.deadline is not None else float("inf")
            update_queue_task = asyncio.create_task(self._update_queue_periodically(key_manager))
            declare_averager_task = None
            if declare:
                declare_averager_task = asyncio.create_task(self._declare_averager_periodically(step, key_manager))
            try:
                yield self
            finally:
                await cancel_and_wait(update_queue_task)
                if declare_averager_task is not None:
                    await cancel_and_wait(declare_averager_task)
                for field in (self.past_attempts, self.leader_queue, self.running, self.update_finished,
                              self.update_triggered, self.declared_expiration):
                    field.clear()
                self.max_assured_time = float("-inf")
                self.search_end_time = float("inf")

    @contextlib.asynccontextmanager
    async def pause_search(self):
        was_running = self.running.is_set()
        try:
            self.running.clear()
            yield
        finally:
            if was_running:
                self.running.set()
            else:
                self.running.clear()

    async def pop_next_leader(self) -> PeerID:
        """The next peer to ask, i.e. one that precedes us in (expiration, id) order. Raises ``TimeoutError`` when
        our own declaration was renewed in the meantime (the caller then decides whether to lead)."""
        assert self.running.is_set(), "Not running search at the moment"
        while True:
            maybe_next_leader, entry = self.leader_queue.top() or (None, None)
            if maybe_next_leader is None or self.max_assured_time <= entry.expiration_time <= self.search_end_time:
                self.update_triggered.set()
            if maybe_next_leader is None or ((entry.expiration_time, maybe_next_leader.to_bytes())
                                             > (self.declared_expiration_time, self.peer_id.to_bytes())):
                update_wait = asyncio.create_task(self.update_finished.wait())
                declare_wait = asyncio.create_task(self.declared_expiration.wait())
                try:
                    await asyncio.wait({update_wait, declare_wait}, return_when=asyncio.FIRST_COMPLETED)
                finally:
                    update_wait.cancel()
                    declare_wait.cancel()
                self.declared_expiration.clear()
                if self.update_finished.is_set():
                    self.update_finished.clear()
                    continue
                raise asyncio.TimeoutError("pop_next_leader was invalidated: re-declared averager in background")
            del self.leader_queue[maybe_next_leader]
            self.past_attempts.add((maybe_next_leader, entry.expiration_time))
            return maybe_next_leader

    async def _update_queue_periodically(self, key_manager: GroupKeyManager) -> None:
        DISCREPANCY = MAX_DHT_TIME_DISCREPANCY_SECONDS
        while get_dht_time() < self.search_end_time:
            new_peers = await key_manager.get_averagers(key_manager.current_key, only_active=True)
            self.max_assured_time = max(self.max_assured_time, get_dht_time() + self.min_matchmaking_time - DISCREPANCY)
            self.leader_queue.clear()
            for peer, peer_expiration_time in new_peers:
                if peer == self.peer_id or (peer, peer_expiration_time) in self.past_attempts:
                    continue
                self.leader_queue.store(peer, peer_expiration_time, peer_expiration_time)
                self.max_assured_time = max(self.max_assured_time, peer_expiration_time - DISCREPANCY)
            self.update_finished.set()
            running_wait = asyncio.create_task(self.running.wait())
            trigger_wait = asyncio.create_task(self.update_triggered.wait())
            try:
                await asyncio.wait({running_wait, trigger_wait}, return_when=asyncio.ALL_COMPLETED,
                                   timeout=self.search_end_time - get_dht_time() if isfinite(self.search_end_time) else None)
            finally:
                running_wait.cancel()
                trigger_wait.cancel()
            self.update_triggered.clear()
            await asyncio.sleep(0.005)  # the DHT shares this process: do not starve it while polling

    async def _declare_averager_periodically(self, step: StepControl, key_manager: GroupKeyManager) -> None:
        async with self.lock_declare:
            try:
                while True:
                    await self.running.wait()
                    new_expiration_time = float(min(max(step.scheduled_time, get_dht_time() + self.min_matchmaking_time),
                                                    self.search_end_time))
                    self.declared_group_key = group_key = key_manager.current_key
                    self.declared_expiration_time = new_expiration_time
                    self.declared_expiration.set()
                    await key_manager.declare_averager(group_key, self.peer_id, expiration_time=new_expiration_time)
                    await asyncio.sleep(max(0.0, self.declared_expiration_time - get_dht_time()))
                    if self.running.is_set() and len(self.leader_queue) == 0:
                        await key_manager.update_key_on_not_enough_peers()
            finally:
                if self.declared_group_key is not None:
                    prev_declared_key, prev_expiration_time = self.declared_group_key, self.declared_expiration_time
                    self.declared_group_key, self.declared_expiration_time = None, float("inf")
                    self.leader_queue, self.max_assured_time = TimedStorage[PeerID, DHTExpiration](), float("-inf")
                    if prev_expiration_time > get_dht_time():
                        await asyncio.shield(key_manager.declare_averager(prev_declared_key, self.peer_id,
                                                                          prev_expiration_time, looking_for_group=False))

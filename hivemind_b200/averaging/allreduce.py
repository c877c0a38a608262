"""Butterfly all-reduce over RPC streams (the host data path; works for CPU tensors and across machines).

Each peer reduces one span of the flattened tensors. Every sender streams its compressed parts of that span to the
reducer through ``rpc_aggregate_part`` and receives, for every part, the compressed difference between the group
average and what it sent. Roles: NODE sends and reduces, CLIENT only sends (it reduces an empty span), AUX only
reduces (it sends nothing and has zero weight). A sender that does not start within ``sender_timeout`` or stalls
between parts is banned and left out of the remaining averages; a reducer that stalls for ``reducer_timeout`` makes
its senders keep their own values for that span. Semantics: hivemind/averaging/allreduce.py:26-377.

On a single box with all peers on GPUs the same round is executed by the device butterfly
(``hivemind_b200.parallel.device_butterfly``) instead; both paths share this file's modes and error types.
"""
from __future__ import annotations

import asyncio
from enum import Enum
from typing import AsyncIterator, Optional, Sequence, Set, Tuple, Type

import torch

from hivemind_b200.averaging.partition import AllreduceException, BannedException, TensorPartContainer, TensorPartReducer
from hivemind_b200.compression import deserialize_torch_tensor, serialize_torch_tensor
from hivemind_b200.p2p import P2P, P2PContext, PeerID, ServicerBase, StubBase
from hivemind_b200.proto import averaging_pb2
from hivemind_b200.utils import get_logger
from hivemind_b200.utils.asyncio import (achain, aiter_with_timeout, amap_in_executor, anext, as_aiter,
                                         attach_event_on_finished)

GroupID = bytes
logger = get_logger(__name__)


class AveragingMode(Enum):
    NODE = 0
    CLIENT = 1
    AUX = 2


class AllReduceRunner(ServicerBase):
    """
    :param p2p: endpoint used for calling groupmates
    :param servicer_type: the class whose ``rpc_aggregate_part`` groupmates serve (normally the averager class)
    :param prefix: RPC namespace (the averager prefix)
    :param group_id: id of this round, checked on every incoming part
    :param tensors: local tensors; ``run()`` yields one delta per tensor
    :param weight: this peer's weight (default 1.0 for senders, 0.0 for AUX)
    :param ordered_peer_ids: group members in span order
    :param peer_fractions: share of elements that each member reduces
    :param modes: ``AveragingMode`` of each member (default: CLIENT where fraction is 0, NODE elsewhere)
    :param sender_timeout: a sender must deliver its first/next part within this many seconds
    :param reducer_timeout: a reducer must answer a part within this many seconds (should exceed sender_timeout)
    :param kwargs: passed to ``TensorPartContainer`` (compression, part_size_bytes, tensor_infos, ...)
    """

    def __init__(self, *, p2p: P2P, servicer_type: Type[ServicerBase], prefix: Optional[str], group_id: GroupID,
                 tensors: Sequence[torch.Tensor], weight: Optional[float] = None, ordered_peer_ids: Sequence[PeerID],
                 peer_fractions: Tuple[float, ...], modes: Optional[Sequence[AveragingMode]] = None,
                 sender_timeout: Optional[float] = None, reducer_timeout: Optional[float] = None, **kwargs):
        self._p2p = p2p
        self.peer_id = p2p.peer_id
        assert self.peer_id in ordered_peer_ids, "peer_id is not a part of the group"
        if reducer_timeout is not None and (sender_timeout is None or reducer_timeout <= sender_timeout):
            raise ValueError("If reducer_timeout is enabled, sender_timeout must be shorter than reducer_timeout. "
                             "Otherwise, there is a chance that reducers will be banned while they await senders.")
        if not issubclass(servicer_type, ServicerBase):
            raise TypeError("`servicer_type` is expected to be a ServicerBase subclass")
        self._servicer_type, self._prefix = servicer_type, prefix

        modes = modes or tuple(AveragingMode.CLIENT if frac == 0 else AveragingMode.NODE for frac in peer_fractions)
        assert len(modes) == len(ordered_peer_ids), "lists have inconsistent length"
        assert any(mode != AveragingMode.CLIENT for mode in modes), "cannot run allreduce without reducers"
        for mode, frac in zip(modes, peer_fractions):
            assert mode != AveragingMode.CLIENT or frac == 0, "client-mode peer should have zero all-reduce fraction"
        self.modes = modes
        my_mode = modes[ordered_peer_ids.index(self.peer_id)]
        if weight is None:
            weight = float(my_mode != AveragingMode.AUX)
        self.weight = weight

        self.group_id, self.ordered_peer_ids = group_id, ordered_peer_ids
        self.peer_fractions = peer_fractions
        self.sender_timeout, self.reducer_timeout = sender_timeout, reducer_timeout
        self._future: asyncio.Future = asyncio.Future()
        self.all_senders_started = asyncio.Event()
        self.banned_senders: Set[PeerID] = set()
        self.banlock = asyncio.Lock()
        self.active_senders: Set[PeerID] = set()
        if my_mode != AveragingMode.AUX:
            self.active_senders.add(self.peer_id)
        if len(self.active_senders) == self._count_senders():
            self.all_senders_started.set()

        self.sender_peer_ids = [peer_id for peer_id, mode in zip(ordered_peer_ids, modes) if mode != AveragingMode.AUX]
        peer_id_index = self.ordered_peer_ids.index(self.peer_id)
        self.tensor_part_container = TensorPartContainer(tensors, peer_fractions, return_deltas=True, **kwargs)
        self.parts_for_local_averaging = self.tensor_part_container.get_raw_input_parts(peer_id_index)
        self.tensor_part_reducer = TensorPartReducer(tuple(part.shape for part in self.parts_for_local_averaging),
                                                     len(self.sender_peer_ids))

    def _count_senders(self) -> int:
        return sum(mode != AveragingMode.AUX for mode in self.modes)

    def __repr__(self) -> str:
        return f"{type(self).__name__}({self.peer_id}, group_size={self.group_size})"

    def __aiter__(self):
        return self.run()

    def __contains__(self, peer_id: PeerID) -> bool:
        return peer_id in self.ordered_peer_ids

    @property
    def group_size(self) -> int:
        return len(self.ordered_peer_ids)

    def _get_peer_stub(self, peer: PeerID) -> StubBase:
        return self._servicer_type.get_stub(self._p2p, peer, namespace=self._prefix)

    def should_delay_results(self, peer_id: PeerID) -> bool:
        return self.peer_fractions[self.ordered_peer_ids.index(peer_id)] == 0

    # ------------------------------------------------------------------------------------------ driver
    async def run(self) -> AsyncIterator[torch.Tensor]:
        """Run the round; yields ``average - local`` for every local tensor, in order."""
        pending_tasks = set()
        if self.tensor_part_container.num_parts_by_peer[self.ordered_peer_ids.index(self.peer_id)] != 0:
            pending_tasks.add(asyncio.create_task(self._handle_missing_senders()))
        try:
            if len(self.sender_peer_ids) == 0:
                logger.debug(f"{self} - finished all-reduce early: all peers are auxiliaries ({self.modes})")
                self.finalize()
            elif self.peer_id in self.sender_peer_ids:
                for peer_id, parts in zip(self.ordered_peer_ids, self.tensor_part_container.num_parts_by_peer):
                    if parts != 0:
                        pending_tasks.add(asyncio.create_task(self._communicate_with_peer(peer_id)))
                async for averaged_tensor_delta in self.tensor_part_container.iterate_output_tensors():
                    yield averaged_tensor_delta
                self.finalize()
            else:  # auxiliary peer: only reduce
                await self.tensor_part_reducer.finished.wait()
                self.finalize()
        except BaseException as e:
            self.finalize(exception=e)
            for task in pending_tasks:
                task.cancel()
            raise

    async def _handle_missing_senders(self) -> None:
        """Ban senders that have not opened their stream to us within ``sender_timeout``."""
        try:
            await asyncio.wait_for(self.all_senders_started.wait(), self.sender_timeout)
        except asyncio.TimeoutError:
            for peer_id in self.sender_peer_ids:
                if peer_id not in self.active_senders and peer_id not in self.banned_senders:
                    await self._ban_sender(peer_id)

    async def _communicate_with_peer(self, peer_id: PeerID) -> None:
        """Send our parts of ``peer_id``'s span and collect the averaged deltas."""
        peer_index = self.ordered_peer_ids.index(peer_id)
        if peer_id == self.peer_id:
            sender_index = self.sender_peer_ids.index(peer_id)
            for part_index, tensor_part in enumerate(self.parts_for_local_averaging):
                averaged_part = await self.tensor_part_reducer.accumulate_part(sender_index, part_index, tensor_part,
                                                                               weight=self.weight)
                self.tensor_part_container.register_processed_part(peer_index, part_index, averaged_part - tensor_part)
            return
        try:
            done_sending = asyncio.Event()
            inputs_aiter = attach_event_on_finished(self._generate_input_for_peer(peer_index), done_sending)
            stream = await self._get_peer_stub(peer_id).rpc_aggregate_part(inputs_aiter)

            if self.should_delay_results(self.peer_id):
                await done_sending.wait()  # client-mode peers receive results only after they finished sending

            part_index = 0

            def _try_deserialize(msg):
                if msg.code != averaging_pb2.AVERAGED_PART:
                    raise AllreduceException(f"{peer_id} sent {averaging_pb2.MessageCode.Name(msg.code)}")
                return deserialize_torch_tensor(msg.tensor_part), msg

            async for delta, msg in amap_in_executor(_try_deserialize, aiter_with_timeout(stream, self.reducer_timeout),
                                                     max_prefetch=self.tensor_part_container.prefetch):
                self.tensor_part_container.register_processed_part(peer_index, part_index, delta)
                part_index += 1
            if part_index != self.tensor_part_container.num_parts_by_peer[peer_index]:
                raise AllreduceException(f"peer {peer_id} sent {part_index} parts, but we expected "
                                         f"{self.tensor_part_container.num_parts_by_peer[peer_index]}")
        except BaseException as e:
            if isinstance(e, Exception):
                logger.debug(f"Caught {e!r} when communicating to {peer_id}", exc_info=True)
            self.tensor_part_container.register_failed_reducer(peer_index)
            if not isinstance(e, Exception):
                raise

    async def _generate_input_for_peer(self, peer_index: int) -> AsyncIterator[averaging_pb2.AveragingData]:
        parts_aiter = self.tensor_part_container.iterate_input_parts_for(peer_index)
        first_part = await anext(parts_aiter)
        yield averaging_pb2.AveragingData(code=averaging_pb2.PART_FOR_AVERAGING, group_id=self.group_id,
                                          tensor_part=first_part, weight=self.weight)
        async for part in parts_aiter:
            yield averaging_pb2.AveragingData(tensor_part=part, weight=self.weight)

    # ------------------------------------------------------------------------------------------ reducer side
    async def rpc_aggregate_part(self, stream: AsyncIterator[averaging_pb2.AveragingData], context: P2PContext
                                 ) -> AsyncIterator[averaging_pb2.AveragingData]:
        """A groupmate streams its parts of our span; answer each part with the averaged delta."""
        sender_peer_id = context.remote_id
        if sender_peer_id not in self.sender_peer_ids:
            yield averaging_pb2.AveragingData(code=averaging_pb2.PROTOCOL_VIOLATION)
            return
        self.active_senders.add(sender_peer_id)
        if len(self.active_senders) == len(self.sender_peer_ids):
            self.all_senders_started.set()
        try:
            request: averaging_pb2.AveragingData = await asyncio.wait_for(anext(stream), self.sender_timeout)
            reason_to_reject = self._check_reasons_to_reject(request, context)
            if reason_to_reject:
                yield reason_to_reject
                return
            if request.code == averaging_pb2.PART_FOR_AVERAGING:
                sender_index = self.sender_peer_ids.index(sender_peer_id)
                async for msg in self._accumulate_parts_streaming(achain(as_aiter(request), stream), sender_index):
                    yield msg
            else:
                code = averaging_pb2.MessageCode.Name(request.code)
                raise AllreduceException(f"{sender_peer_id} sent {code}, but we expected PART_FOR_AVERAGING")
        except BaseException as e:
            if isinstance(e, Exception):
                await self._ban_sender(sender_peer_id)
                if isinstance(e, (asyncio.TimeoutError, BannedException)):
                    logger.debug(f"sender {sender_peer_id} was banned: {e!r}")
                    yield averaging_pb2.AveragingData(code=averaging_pb2.CANCELLED)
                else:
                    logger.debug(f"caught {e!r} while reducing parts from {sender_peer_id}", exc_info=True)
                    yield averaging_pb2.AveragingData(code=averaging_pb2.INTERNAL_ERROR)
            else:
                raise

    def _check_reasons_to_reject(self, request: averaging_pb2.AveragingData, context: P2PContext
                                 ) -> Optional[averaging_pb2.AveragingData]:
        if request.group_id != self.group_id:
            return averaging_pb2.AveragingData(code=averaging_pb2.BAD_GROUP_ID)
        if self._future.cancelled():
            return averaging_pb2.AveragingData(code=averaging_pb2.CANCELLED)
        if self._future.done():
            return averaging_pb2.AveragingData(code=averaging_pb2.INTERNAL_ERROR)
        return None

    async def _accumulate_parts_streaming(self, stream: AsyncIterator[averaging_pb2.AveragingData], sender_index: int):
        part_index = 0
        try:
            loop = asyncio.get_event_loop()
            async for tensor_part, weight, part_compression in amap_in_executor(
                    lambda msg: (deserialize_torch_tensor(msg.tensor_part), msg.weight, msg.tensor_part.compression),
                    aiter_with_timeout(stream, self.sender_timeout), max_prefetch=self.tensor_part_container.prefetch):
                try:
                    averaged_part = await self.tensor_part_reducer.accumulate_part(sender_index, part_index,
                                                                                   tensor_part, weight=weight)
                    part_index += 1
                except BannedException:
                    logger.debug(f"Sender {sender_index} is already banned")
                    break
                serialized_delta = await loop.run_in_executor(
                    None, lambda: serialize_torch_tensor(averaged_part - tensor_part, part_compression))
                yield averaging_pb2.AveragingData(code=averaging_pb2.AVERAGED_PART, tensor_part=serialized_delta)
        finally:
            if part_index != self.tensor_part_reducer.num_parts:
                await self._ban_sender(self.sender_peer_ids[sender_index])

    async def _ban_sender(self, peer_id: PeerID) -> None:
        async with self.banlock:
            if peer_id not in self.banned_senders:
                self.banned_senders.add(peer_id)
                self.tensor_part_reducer.on_sender_failed(self.sender_peer_ids.index(peer_id))

    def finalize(self, *, cancel: bool = False, exception: Optional[BaseException] = None) -> bool:
        """Finish the round, release buffers; returns True if this call changed the state."""
        assert not cancel or not exception, "finalize accepts either exception or cancel, but not both"
        pending_tasks = set()
        if cancel or exception:
            # tell peers that are still streaming to us that we are out
            for peer_id, mode in zip(self.ordered_peer_ids, self.modes):
                if peer_id != self.peer_id and mode != AveragingMode.CLIENT:
                    pass  # their streams end when our handlers exit; nothing to send explicitly
        if not self._future.done():
            if cancel:
                logger.debug(f"{self} - cancelled")
                self._future.cancel()
            elif exception:
                logger.debug(f"{self} - caught {exception!r}")
                self._future.set_exception(exception)
            else:
                logger.debug(f"{self} - finished")
                self._future.set_result(None)
            self.tensor_part_container.finalize()
            self.tensor_part_reducer.finalize()
            return True
        logger.debug(f"{self} - attempted to finalize allreduce that is already finished: {self._future}")
        return False

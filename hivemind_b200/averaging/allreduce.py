"""Butterfly all-reduce over RPC streams (the host data path; works for CPU tensors and across machines).

Each peer reduces one span of the flattened tensors. Every sender streams its compressed parts of that span to the
reducer through ``rpc_aggregate_part`` and receives, for every part, the compressed difference between the group
average and what it sent. Roles: NODE sends and reduces, CLIENT only sends (it reduces an empty span), AUX only
reduces (it sends nothing and has zero weight). A sender that does not start within ``sender_timeout`` or stalls
between parts is banned and left out of the remaining averages; a reducer that stalls for ``reducer_timeout`` makes
its senders keep their own values for that span. Semantics: hivemind/averaging/allreduce.py:26-377.

On a single box with all peers on GPUs the same round is executed by the device butterfly
(``hivemind_b200.parallel.device_butterfly``) instead; both paths share this file's modes and error types.

The runner has two faces. As a *sender* (``run``) it opens one stream per reducer, feeds it from the part container
and files the deltas that come back; its own span goes straight into the local reducer. As a *reducer*
(``rpc_aggregate_part``) it takes one sender's stream, adds every part into the accumulator of that part and answers
with the delta once all live senders have contributed.
"""
from __future__ import annotations

import asyncio
from enum import Enum
from typing import AsyncIterator, List, Optional, Sequence, Set, Tuple, Type

import torch

from hivemind_b200.averaging.partition import AllreduceException, BannedException, TensorPartContainer, TensorPartReducer
from hivemind_b200.compression import deserialize_torch_tensor, serialize_torch_tensor
from hivemind_b200.compression.serialization import (RawMessage, TensorView, _varint, is_light_to_decode,
                                                     is_light_to_encode, split_length_delimited_field)
from hivemind_b200.p2p import P2P, P2PContext, PeerID, ServicerBase, StubBase
from hivemind_b200.proto import averaging_pb2
from hivemind_b200.utils import get_logger
from hivemind_b200.utils.asyncio import (achain, aiter_with_timeout, amap_in_executor, anext, as_aiter,
                                         attach_event_on_finished)

GroupID = bytes
logger = get_logger(__name__)
_Msg = averaging_pb2.AveragingData
_TENSOR_PART_TAG = bytes([(4 << 3) | 2])  # AveragingData.tensor_part: field 4, length-delimited


class PartMessage:
    """A received ``AveragingData`` whose tensor part is not parsed: the half-megabyte payload stays a view of the
    received bytes until a codec reads it (``FromString`` is what the RPC layer calls on arrival). Attribute access
    is that of the generated message for the fields this protocol uses."""

    __slots__ = ("code", "group_id", "peer_id", "weight", "tensor_part")
    _NO_TENSOR = averaging_pb2.AveragingData().tensor_part

    @classmethod
    def FromString(cls, payload: bytes) -> "PartMessage":
        part, rest = split_length_delimited_field(memoryview(payload), 4)
        small = _Msg.FromString(rest)
        self = cls()
        self.code, self.group_id, self.peer_id, self.weight = small.code, small.group_id, small.peer_id, small.weight
        self.tensor_part = TensorView(part) if part is not None else cls._NO_TENSOR
        return self


def _part_message(tensor_part, **small_fields) -> RawMessage:
    """An ``AveragingData`` message around a serialized tensor part, as wire bytes: the small fields are encoded by
    protobuf, the part is serialized once and appended as it is. Building the outer message as an object would copy
    the part into it and once more when serializing; for parts of half a megabyte those copies are most of the cost.
    Any protobuf parser reads the result as an ordinary ``AveragingData``."""
    inner = tensor_part.SerializeToString()
    return RawMessage(_Msg(**small_fields).SerializeToString() + _TENSOR_PART_TAG + _varint(len(inner)), inner)


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
        self._p2p, self.peer_id = p2p, p2p.peer_id
        if self.peer_id not in ordered_peer_ids:
            raise ValueError("this peer is not a member of the group")
        if not issubclass(servicer_type, ServicerBase):
            raise TypeError("servicer_type must derive from ServicerBase")
        if reducer_timeout is not None and (sender_timeout is None or reducer_timeout <= sender_timeout):
            raise ValueError("reducer_timeout must be longer than sender_timeout: a reducer that is still waiting for a "
                             "slow sender must not be written off by the other senders")
        self._servicer_type, self._prefix = servicer_type, prefix
        if not modes:
            modes = tuple(AveragingMode.CLIENT if fraction == 0 else AveragingMode.NODE for fraction in peer_fractions)
        if len(modes) != len(ordered_peer_ids) or len(peer_fractions) != len(ordered_peer_ids):
            raise ValueError("modes, fractions and peer ids must describe the same members")
        if all(mode == AveragingMode.CLIENT for mode in modes):
            raise ValueError("a group of client-mode peers has nobody to reduce")
        if any(mode == AveragingMode.CLIENT and fraction != 0 for mode, fraction in zip(modes, peer_fractions)):
            raise ValueError("client-mode peers reduce nothing: their fraction must be 0")
        self.modes, self.peer_fractions = modes, peer_fractions
        self.group_id, self.ordered_peer_ids = group_id, ordered_peer_ids
        self.sender_timeout, self.reducer_timeout = sender_timeout, reducer_timeout
        self._my_index = list(ordered_peer_ids).index(self.peer_id)
        self._i_send = modes[self._my_index] != AveragingMode.AUX
        self.weight = float(self._i_send) if weight is None else weight
        self.sender_peer_ids: List[PeerID] = [p for p, mode in zip(ordered_peer_ids, modes) if mode != AveragingMode.AUX]

        self._future: asyncio.Future = asyncio.Future()
        self.banned_senders: Set[PeerID] = set()
        self.banlock = asyncio.Lock()
        self.active_senders: Set[PeerID] = {self.peer_id} if self._i_send else set()
        self.all_senders_started = asyncio.Event()
        self._note_sender_progress()

        self.tensor_part_container = TensorPartContainer(tensors, peer_fractions, return_deltas=True, **kwargs)
        self.parts_for_local_averaging = self.tensor_part_container.get_raw_input_parts(self._my_index)
        self.tensor_part_reducer = TensorPartReducer(tuple(part.shape for part in self.parts_for_local_averaging),
                                                     len(self.sender_peer_ids))

    def _note_sender_progress(self) -> None:
        if len(self.active_senders) >= len(self.sender_peer_ids):
            self.all_senders_started.set()

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
        """Peers that reduce nothing (clients) read results only after they have sent everything."""
        return self.peer_fractions[list(self.ordered_peer_ids).index(peer_id)] == 0

    # ------------------------------------------------------------------------------------------ sender side
    async def run(self) -> AsyncIterator[torch.Tensor]:
        """Run the round; yields ``average - local`` for every local tensor, in order."""
        parts_per_reducer = self.tensor_part_container.num_parts_by_peer
        helpers = set()
        if parts_per_reducer[self._my_index] != 0:
            helpers.add(asyncio.create_task(self._watch_for_absent_senders()))
        try:
            if not self.sender_peer_ids:
                logger.debug(f"{self}: nothing to average, every member is an auxiliary ({self.modes})")
            elif self._i_send:
                for reducer, count in zip(self.ordered_peer_ids, parts_per_reducer):
                    if count != 0:
                        helpers.add(asyncio.create_task(self._exchange_with(reducer)))
                async for delta in self.tensor_part_container.iterate_output_tensors():
                    yield delta
            else:  # an auxiliary only reduces
                await self.tensor_part_reducer.finished.wait()
            self.finalize()
        except BaseException as e:
            self.finalize(exception=e)
            for task in helpers:
                task.cancel()
            raise

    async def _watch_for_absent_senders(self) -> None:
        """Senders that have not opened their stream to us within ``sender_timeout`` are written off."""
        try:
            await asyncio.wait_for(self.all_senders_started.wait(), self.sender_timeout)
        except asyncio.TimeoutError:
            for peer in self.sender_peer_ids:
                if peer not in self.active_senders and peer not in self.banned_senders:
                    await self._ban_sender(peer)

    async def _exchange_with(self, reducer: PeerID) -> None:
        """Deliver our parts of ``reducer``'s span and file the averaged deltas that come back."""
        reducer_index = list(self.ordered_peer_ids).index(reducer)
        container = self.tensor_part_container
        if reducer == self.peer_id:
            me_as_sender = self.sender_peer_ids.index(self.peer_id)
            for part_index, part in enumerate(self.parts_for_local_averaging):
                average = await self.tensor_part_reducer.accumulate_part(me_as_sender, part_index, part, weight=self.weight)
                container.register_processed_part(reducer_index, part_index, average - part)
            return
        try:
            everything_sent = asyncio.Event()
            outgoing = attach_event_on_finished(self._generate_input_for_peer(reducer_index), everything_sent)
            incoming = await self._get_peer_stub(reducer).rpc_aggregate_part(outgoing)
            if self.should_delay_results(self.peer_id):
                await everything_sent.wait()

            def decode(message: _Msg) -> torch.Tensor:
                if message.code != averaging_pb2.AVERAGED_PART:
                    raise AllreduceException(f"{reducer} answered {averaging_pb2.MessageCode.Name(message.code)}")
                return deserialize_torch_tensor(message.tensor_part)

            received = 0
            async for delta in amap_in_executor(decode, aiter_with_timeout(incoming, self.reducer_timeout),
                                                max_prefetch=container.prefetch,
                                                inline=lambda message: is_light_to_decode(message.tensor_part)):
                container.register_processed_part(reducer_index, received, delta)
                received += 1
            expected = container.num_parts_by_peer[reducer_index]
            if received != expected:
                raise AllreduceException(f"{reducer} returned {received} of {expected} parts")
        except BaseException as e:
            container.register_failed_reducer(reducer_index)  # we keep our own values for that span
            if not isinstance(e, Exception):
                raise
            logger.debug(f"exchange with reducer {reducer} failed: {e!r}", exc_info=True)

    async def _generate_input_for_peer(self, peer_index: int) -> AsyncIterator[averaging_pb2.AveragingData]:
        """The messages we stream to the reducer with this index; only the first carries the group id."""
        parts = self.tensor_part_container.iterate_input_parts_for(peer_index)
        yield _part_message(await anext(parts), code=averaging_pb2.PART_FOR_AVERAGING, group_id=self.group_id,
                            weight=self.weight)
        async for part in parts:
            yield _part_message(part, weight=self.weight)

    # ------------------------------------------------------------------------------------------ reducer side
    async def rpc_aggregate_part(self, stream: AsyncIterator[averaging_pb2.AveragingData], context: P2PContext
                                 ) -> AsyncIterator[averaging_pb2.AveragingData]:
        """A groupmate streams its parts of our span; answer each part with the averaged delta."""
        sender = context.remote_id
        if sender not in self.sender_peer_ids:
            yield _Msg(code=averaging_pb2.PROTOCOL_VIOLATION)
            return
        self.active_senders.add(sender)
        self._note_sender_progress()
        try:
            opening: _Msg = await asyncio.wait_for(anext(stream), self.sender_timeout)
            refusal = self._refusal_for(opening)
            if refusal is not None:
                yield refusal
                return
            if opening.code != averaging_pb2.PART_FOR_AVERAGING:
                raise AllreduceException(f"{sender} opened with {averaging_pb2.MessageCode.Name(opening.code)}")
            async for reply in self._reduce_stream(achain(as_aiter(opening), stream), self.sender_peer_ids.index(sender)):
                yield reply
        except BaseException as e:
            if not isinstance(e, Exception):
                raise
            await self._ban_sender(sender)
            if isinstance(e, (asyncio.TimeoutError, BannedException)):
                logger.debug(f"sender {sender} is out of this round: {e!r}")
                yield _Msg(code=averaging_pb2.CANCELLED)
            else:
                logger.debug(f"reducing parts of {sender} failed: {e!r}", exc_info=True)
                yield _Msg(code=averaging_pb2.INTERNAL_ERROR)

    def _refusal_for(self, opening: _Msg) -> Optional[_Msg]:
        if opening.group_id != self.group_id:
            return _Msg(code=averaging_pb2.BAD_GROUP_ID)
        if self._future.cancelled():
            return _Msg(code=averaging_pb2.CANCELLED)
        if self._future.done():
            return _Msg(code=averaging_pb2.INTERNAL_ERROR)
        return None

    async def _reduce_stream(self, stream: AsyncIterator[_Msg], sender_index: int) -> AsyncIterator[_Msg]:
        loop = asyncio.get_event_loop()
        reduced = 0

        def decode(message: _Msg):
            return deserialize_torch_tensor(message.tensor_part), message.weight, message.tensor_part.compression

        try:
            async for part, weight, codec in amap_in_executor(decode, aiter_with_timeout(stream, self.sender_timeout),
                                                              max_prefetch=self.tensor_part_container.prefetch,
                                                              inline=lambda message: is_light_to_decode(message.tensor_part)):
                try:
                    average = await self.tensor_part_reducer.accumulate_part(sender_index, reduced, part, weight=weight)
                except BannedException:
                    logger.debug(f"sender {sender_index} was banned while its part was waiting")
                    break
                reduced += 1
                if is_light_to_encode(part, codec):
                    delta = serialize_torch_tensor(average - part, codec)
                else:
                    delta = await loop.run_in_executor(None, lambda: serialize_torch_tensor(average - part, codec))
                yield _part_message(delta, code=averaging_pb2.AVERAGED_PART)
        finally:
            if reduced != self.tensor_part_reducer.num_parts:
                await self._ban_sender(self.sender_peer_ids[sender_index])

    async def _ban_sender(self, peer_id: PeerID) -> None:
        async with self.banlock:
            if peer_id in self.banned_senders:
                return
            self.banned_senders.add(peer_id)
            self.tensor_part_reducer.on_sender_failed(self.sender_peer_ids.index(peer_id))

    def finalize(self, *, cancel: bool = False, exception: Optional[BaseException] = None) -> bool:
        """Finish the round and release its buffers; returns True if this call changed the state. Streams to and
        from groupmates end when their handlers see the released containers."""
        if cancel and exception is not None:
            raise ValueError("finalize takes cancel or an exception, not both")
        if self._future.done():
            logger.debug(f"{self}: already finalized ({self._future})")
            return False
        if cancel or isinstance(exception, asyncio.CancelledError):
            self._future.cancel()
        elif exception is not None:
            self._future.set_exception(exception)
            self._future.exception()  # the future only records how the round ended; nobody awaits it
        else:
            self._future.set_result(None)
        logger.debug(f"{self}: finalized ({'cancelled' if cancel else repr(exception) if exception else 'ok'})")
        self.tensor_part_container.finalize()
        self.tensor_part_reducer.finalize()
        return True

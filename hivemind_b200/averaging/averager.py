"""``DecentralizedAverager``: background service that averages a set of tensors with peers found through the DHT.

Public behaviour follows the reference (hivemind/averaging/averager.py:50-821): ``step()`` looks for a group
(matchmaking), runs a butterfly all-reduce inside it and applies ``tensor += averaging_alpha * (average - tensor)``;
failed attempts are retried until the deadline; peers can download each other's state.

Execution model: the reference forks a process per averager and keeps tensors in host shared memory. Here the
averager is a thread with its own event loop inside the (one per GPU) training process, the averaged tensors stay
where they are (CPU or CUDA), and two data paths exist:
 * the RPC path (``AllReduceRunner``) — CPU tensors, mixed or remote groups;
 * the device path (``hivemind_b200.parallel.device_butterfly``) — when every group member advertises a
   peer-mappable device arena on the same machine, the round runs as sm_100a kernels over NVLink peer memory.
"""
from __future__ import annotations

import asyncio
import contextlib
import os
import random
import threading
from typing import Any, AsyncIterator, Dict, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from hivemind_b200.utils.asyncio import spawn
from hivemind_b200.averaging.allreduce import AllreduceException, AllReduceRunner, AveragingMode, GroupID, PartMessage
from hivemind_b200.averaging.control import AveragingStage, StepControl
from hivemind_b200.averaging.group_info import GroupInfo
from hivemind_b200.averaging.load_balancing import load_balance_peers
from hivemind_b200.averaging.matchmaking import Matchmaking, MatchmakingException
from hivemind_b200.averaging.partition import DEFAULT_PART_SIZE_BYTES
from hivemind_b200.compression import (CompressionBase, CompressionInfo, NoCompression, deserialize_torch_tensor,
                                       split_for_streaming, combine_from_streaming)
from hivemind_b200.dht import DHT, DHTID
from hivemind_b200.p2p import P2P, P2PContext, P2PDaemonError, P2PHandlerError, PeerID, ServicerBase
from hivemind_b200.p2p.control import DispatchFailure
from hivemind_b200.proto import averaging_pb2
from hivemind_b200.utils import MPFuture, MSGPackSerializer, get_logger
from hivemind_b200.utils.asyncio import (LoopThread, achain, aiter_with_timeout, anext, as_aiter, azip,
                                         enter_asynchronously)
from hivemind_b200.utils.timed_storage import DHTExpiration, ValueWithExpiration, get_dht_time

GatheredData = Any
logger = get_logger(__name__)


def compute_schema_hash(tensors: Sequence[torch.Tensor]) -> bytes:
    """Fingerprint of shapes and dtypes: peers with different tensor schemas never end up in one group."""
    schema_dicts = [{field_name: str(field_value) for field_name, field_value in
                     (("size", tuple(t.shape)), ("dtype", t.dtype), ("layout", t.layout))} for t in tensors]
    return DHTID.generate(source=schema_dicts).to_bytes()


_REHOMING_ANNOUNCED = False


class DecentralizedAverager(ServicerBase):
    """
    :param averaged_tensors: tensors to average; the averager keeps references (CUDA tensors may be re-homed into a
      peer-mappable arena, in which case ``get_tensors()`` returns the arena views)
    :param dht: a running DHT used to find groupmates
    :param start: start the background thread right away
    :param prefix: namespace of this averager; all peers that average together use the same prefix
    :param target_group_size: a leader begins all-reduce as soon as this many peers have joined
    :param min_group_size: with fewer peers than this at the deadline the group is disbanded
    :param initial_group_bits: starting group key suffix (string of 0/1)
    :param min_matchmaking_time: a peer waits at least this long for groupmates before leading a partial group
    :param request_timeout: how long to wait for a potential leader's first answer
    :param averaging_alpha: step towards the average (1.0 = replace by the average)
    :param part_size_bytes: size of one compressed part in the all-reduce stream
    :param allreduce_timeout: abort a round that takes longer
    :param next_chunk_timeout / sender_timeout / reducer_timeout: per-part deadlines (see ``AllReduceRunner``)
    :param compression: codec for parts sent to peers; ``state_compression``: codec for state downloads
    :param tensor_infos: per-tensor CompressionInfo (roles, keys) for adaptive codecs
    :param bandwidth: this peer's bandwidth hint for load balancing (None = average)
    :param min_vector_size: peers whose share would be smaller reduce nothing
    :param auxiliary: this peer only helps to reduce (weight 0, sends nothing)
    :param allow_state_sharing: let other peers download our state (default: unless client/auxiliary)
    :param declare_state_period: how often to re-announce that we can share state
    :param client_mode: never accept incoming requests (send only)
    :param shutdown_timeout: seconds to wait for a clean stop
    :param use_device_path: average CUDA fp32 tensors with the device butterfly when the whole group shares an NVLink
      box (default: yes, unless ``HIVEMIND_DEVICE_BUTTERFLY=0``). The tensors are then COPIED into a peer-mappable arena
      and ``get_tensors()`` yields the arena views: the tensors passed in are no longer the averaged ones. Pass
      False to keep averaging the caller's own tensors in place (through the RPC butterfly)
    :param device_endpoint: an existing ``DeviceEndpoint`` whose ``tensor_views`` are ``averaged_tensors``
    """

    _matchmaking: Matchmaking
    _pending_groups_registered: asyncio.Event
    _state_updated: asyncio.Event
    _p2p: P2P
    serializer = MSGPackSerializer

    def __init__(self, averaged_tensors: Sequence[torch.Tensor], dht: DHT, *, start: bool, prefix: str,
                 target_group_size: Optional[int] = None, min_group_size: int = 2, initial_group_bits: str = "",
                 min_matchmaking_time: float = 5.0, request_timeout: float = 3.0, averaging_alpha: float = 1.0,
                 part_size_bytes: int = DEFAULT_PART_SIZE_BYTES, allreduce_timeout: Optional[float] = None,
                 next_chunk_timeout: Optional[float] = None, sender_timeout: Optional[float] = None,
                 reducer_timeout: Optional[float] = None, compression: CompressionBase = NoCompression(),
                 state_compression: CompressionBase = NoCompression(),
                 tensor_infos: Optional[Sequence[CompressionInfo]] = None, bandwidth: Optional[float] = None,
                 min_vector_size: int = 0, auxiliary: bool = False, allow_state_sharing: Optional[bool] = None,
                 declare_state_period: float = 30, client_mode: Optional[bool] = None, daemon: bool = True,
                 shutdown_timeout: float = 5, use_device_path: Optional[bool] = None, device_endpoint=None):
        assert "." not in prefix, "group prefix must be a string without trailing '.'"
        assert bandwidth is None or (bandwidth >= 0 and np.isfinite(np.float32(bandwidth))), \
            "bandwidth must be a non-negative float32"
        assert all(bit in "01" for bit in initial_group_bits)
        assert not client_mode or not auxiliary, "auxiliary peers must accept incoming connections"
        super().__init__()
        self.dht = dht
        self.prefix = prefix
        if client_mode is None:
            client_mode = dht.client_mode
        if sender_timeout is None:
            sender_timeout = next_chunk_timeout
        if reducer_timeout is None:
            reducer_timeout = 2 * sender_timeout if sender_timeout is not None else None
        self.client_mode = client_mode
        self.mode = AveragingMode.CLIENT if client_mode else (AveragingMode.AUX if auxiliary else AveragingMode.NODE)
        self.daemon = daemon

        for tensor in averaged_tensors:
            assert tensor.grad_fn is None, "averaged_tensors must be either parameters or leaf tensors"
        self._averaged_tensors = tuple(averaged_tensors)
        self.lock_averaged_tensors = threading.Lock()
        self.total_size = sum(map(torch.Tensor.numel, self._averaged_tensors))
        self.schema_hash = compute_schema_hash(self._averaged_tensors)
        self.shutdown_timeout = shutdown_timeout
        self.next_chunk_timeout = next_chunk_timeout
        self.bandwidth = bandwidth
        self.matchmaking_kwargs = dict(servicer_type=type(self), prefix=prefix, initial_group_bits=initial_group_bits,
                                       target_group_size=target_group_size, min_group_size=min_group_size,
                                       request_timeout=request_timeout, min_matchmaking_time=min_matchmaking_time)
        self.allreduce_kwargs = dict(compression=compression, part_size_bytes=part_size_bytes,
                                     min_vector_size=min_vector_size, sender_timeout=sender_timeout,
                                     reducer_timeout=reducer_timeout)
        self._averaging_alpha, self._allreduce_timeout = averaging_alpha, allreduce_timeout
        self._running_groups: Dict[GroupID, asyncio.Future] = {}
        self._allow_state_sharing = False
        self._state_sharing_priority = 0.0
        if allow_state_sharing is None:
            allow_state_sharing = not client_mode and not auxiliary
        self.declare_state_period = declare_state_period
        self.state_compression = state_compression
        self.tensor_infos = tensor_infos

        # device data path: CUDA tensors live in one peer-mappable arena. A subclass that needs the arena before this
        # constructor runs (its optimizer works on the arena views) passes the endpoint whose views it handed in
        self._device_endpoint = device_endpoint
        all_cuda_fp32 = len(self._averaged_tensors) > 0 and all(
            t.is_cuda and t.dtype == torch.float32 for t in self._averaged_tensors)
        if use_device_path is None:
            use_device_path = all_cuda_fp32 and os.environ.get("HIVEMIND_DEVICE_BUTTERFLY", "1") != "0"
        if device_endpoint is None and use_device_path and all_cuda_fp32:
            from hivemind_b200.parallel.device_butterfly import DeviceEndpoint

            infos = tensor_infos or tuple(CompressionInfo.from_tensor(t, key=i) for i, t in enumerate(self._averaged_tensors))
            self._device_endpoint = DeviceEndpoint(self._averaged_tensors, compression, infos, part_size_bytes)
            self._averaged_tensors = tuple(self._device_endpoint.tensor_views)
            global _REHOMING_ANNOUNCED
            if not _REHOMING_ANNOUNCED:  # once per process: the tensors passed in are no longer the averaged ones
                _REHOMING_ANNOUNCED = True
                logger.info("CUDA tensors given to an averager were copied into a peer-mappable device arena; "
                            "get_tensors() returns the live (arena) tensors, use_device_path=False keeps them in place")

        self._ready = MPFuture()
        self._thread: Optional[LoopThread] = None
        self._p2p = None
        self._alive = False
        self._allow_state_sharing_requested = allow_state_sharing
        if start:
            self.run_in_background(await_ready=True)

    # ---------------------------------------------------------------------------------------------- properties
    @property
    def allow_state_sharing(self) -> bool:
        """If True, other peers may download this peer's state through ``load_state_from_peers``."""
        return bool(self._allow_state_sharing)

    @allow_state_sharing.setter
    def allow_state_sharing(self, value: bool) -> None:
        if value and self.client_mode:
            raise ValueError("Cannot allow state sharing: averager in client mode cannot share its state")
        old, self._allow_state_sharing = self._allow_state_sharing, value
        if value != old and self._thread is not None and self._thread.loop is not None:
            self._thread.loop.call_soon_threadsafe(self._state_updated.set)

    @property
    def state_sharing_priority(self) -> float:
        """Peers with a higher priority are asked for their state first."""
        return float(self._state_sharing_priority)

    @state_sharing_priority.setter
    def state_sharing_priority(self, value: float) -> None:
        if value != self._state_sharing_priority:
            self._state_sharing_priority = value
            if self._thread is not None and self._thread.loop is not None and self._alive:
                self._thread.loop.call_soon_threadsafe(self._state_updated.set)

    @property
    def peer_id(self) -> PeerID:
        return self.dht.peer_id

    @property
    def request_timeout(self) -> float:
        return self._matchmaking.request_timeout

    def is_alive(self) -> bool:
        return self._alive and self._thread is not None and self._thread.is_alive

    def __repr__(self) -> str:
        return f"{type(self).__name__}({self.prefix}, peer_id={self.peer_id if self._alive else '?'})"

    # ---------------------------------------------------------------------------------------------- lifecycle
    def run_in_background(self, await_ready: bool = True, timeout: Optional[float] = None) -> None:
        """Start the averager's thread and event loop; optionally wait until its RPC handlers are registered."""
        if self._thread is not None:
            return
        self._thread = LoopThread(name=f"Averager-{self.prefix}-{id(self):x}").start()
        self._thread.submit(self._setup())
        if await_ready:
            self.wait_until_ready(timeout)

    def wait_until_ready(self, timeout: Optional[float] = None) -> None:
        self._ready.result(timeout=timeout)

    async def _setup(self) -> None:
        try:
            self._p2p = await self.dht.replicate_p2p()
            if not self.client_mode:
                await self.add_p2p_handlers(self._p2p, namespace=self.prefix)
            else:
                logger.debug("The averager is running in client mode")
            self._matchmaking = Matchmaking(self._p2p, self.schema_hash, self.dht, client_mode=self.client_mode,
                                            **self.matchmaking_kwargs)
            self._pending_groups_registered = asyncio.Event()
            self._pending_groups_registered.set()
            self._state_updated = asyncio.Event()
            self._alive = True
            if self._allow_state_sharing_requested:
                self._allow_state_sharing = True
            if not self.client_mode:
                self._declare_task = asyncio.create_task(self._declare_for_download_periodically())
            self._ready.set_result(None)
        except BaseException as e:  # a cancellation must not leave the constructor waiting forever either
            logger.exception(e)
            if not self._ready.done():
                self._ready.set_exception(e if isinstance(e, Exception) else RuntimeError(f"averager setup failed: {e!r}"))
            if not isinstance(e, Exception):
                raise

    def shutdown(self) -> None:
        """Stop the background thread; pending steps fail with an exception."""
        thread, self._thread = self._thread, None
        if thread is None:
            return
        self._alive = False

        async def _stop():
            for task in [getattr(self, "_declare_task", None)]:
                if task is not None:
                    task.cancel()
            if self._p2p is not None:
                with contextlib.suppress(Exception):
                    if not self.client_mode:
                        await self.remove_p2p_handlers(self._p2p, namespace=self.prefix)
                with contextlib.suppress(Exception):
                    await self._p2p.shutdown()

        try:
            thread.run(_stop(), timeout=self.shutdown_timeout)
        except Exception as e:
            logger.debug(f"averager did not shut down cleanly: {e!r}")
        thread.stop()
        if self._device_endpoint is not None:
            self._device_endpoint.close()

    def __del__(self):
        with contextlib.suppress(Exception):
            self.shutdown()

    # ---------------------------------------------------------------------------------------------- step
    def step(self, gather: Optional[GatheredData] = None, scheduled_time: Optional[DHTExpiration] = None,
             weight: Optional[float] = None, timeout: Optional[float] = None, allow_retries: bool = True,
             require_trigger: bool = False, wait: bool = True) -> Union[Optional[Dict[PeerID, GatheredData]], StepControl]:
        """Find a group and average tensors with it.

        :param gather: small picklable-by-msgpack object sent to all groupmates (returned as ``{peer: gather}``)
        :param scheduled_time: when averaging should begin (default: after ``min_matchmaking_time``)
        :param weight: this peer's weight in the average (default 1, or 0 for auxiliaries)
        :param timeout: give up after this many seconds
        :param allow_retries: retry failed matchmaking / all-reduce until the timeout
        :param require_trigger: hold the assembled group until ``StepControl.allow_allreduce()`` is called
        :param wait: block until done and return the gathered dict; otherwise return the ``StepControl``
        """
        if self.mode == AveragingMode.AUX and weight is not None:
            logger.warning("Averager is running in auxiliary mode, weight is unused")
        if scheduled_time is None:
            scheduled_time = get_dht_time() + self.matchmaking_kwargs["min_matchmaking_time"]
        if weight is None:
            weight = float(self.mode != AveragingMode.AUX)
        deadline = get_dht_time() + timeout if timeout is not None else float("inf")
        assert isinstance(weight, (int, float)) and weight >= 0, f"Expected a positive int/float, got {type(weight)}"
        assert not (wait and require_trigger), "Non-asynchronous step cannot wait for trigger (use wait=False)"
        assert scheduled_time < deadline, "Scheduled start time does not fit within timeout"

        user_data_for_gather = self.serializer.dumps(gather)
        device_info = self._describe_device()
        data_for_gather = self.serializer.dumps([self.bandwidth, self.mode.value, user_data_for_gather, device_info])
        step = StepControl(scheduled_time=scheduled_time, deadline=deadline, allow_retries=allow_retries, weight=weight,
                           data_for_gather=data_for_gather)
        step.attach(MPFuture(), MPFuture())
        if not require_trigger:
            step.allow_allreduce()
        assert self._thread is not None, "the averager is not running"
        self._thread.submit(self._step(step=step))
        return step.result() if wait else step

    def _describe_device(self) -> Optional[dict]:
        """What groupmates need to map this averager's device arena(s); None if it averages through RPC only."""
        return self._device_endpoint.describe() if self._device_endpoint is not None else None

    async def _step(self, *, step: StepControl) -> None:
        try:
            while not step.done():
                try:
                    self._pending_groups_registered.clear()
                    step.stage = AveragingStage.LOOKING_FOR_GROUP
                    matchmaking_task = asyncio.create_task(self._matchmaking.look_for_group(step))
                    check_cancel_task = asyncio.create_task(step.wait_for_cancel())
                    await asyncio.wait({matchmaking_task, check_cancel_task}, return_when=asyncio.FIRST_COMPLETED)
                    if step.cancelled():
                        matchmaking_task.cancel()
                        raise asyncio.CancelledError()
                    check_cancel_task.cancel()
                    group_info = await matchmaking_task
                    if group_info is None:
                        raise AllreduceException("Averaging step failed: could not find a group")

                    with self._register_allreduce_group(group_info):
                        step.stage = AveragingStage.AWAITING_TRIGGER
                        await step.wait_for_trigger()
                        step.stage = AveragingStage.RUNNING_ALLREDUCE
                        result = await asyncio.wait_for(
                            self._aggregate_with_group(group_info, tensor_infos=self.tensor_infos, weight=step.weight,
                                                       **self.allreduce_kwargs),
                            timeout=self._allreduce_timeout)
                        if not step.done():
                            step.set_result(result)
                except (AllreduceException, MatchmakingException, AssertionError, StopAsyncIteration,
                        asyncio.CancelledError, asyncio.InvalidStateError, asyncio.TimeoutError, P2PHandlerError,
                        P2PDaemonError, DispatchFailure) as e:
                    if step.done() or not step.allow_retries or get_dht_time() >= step.deadline:
                        if not step.cancelled():
                            logger.debug(f"averaging step failed: {e!r}", exc_info=True)
                        if not step.done():
                            step.set_exception(e if not isinstance(e, asyncio.CancelledError) else AllreduceException("cancelled"))
                    else:
                        logger.warning(f"{self.__class__.__name__} caught {e!r}, retrying")
        except BaseException as e:
            if not step.done():
                step.set_exception(e if isinstance(e, Exception) else RuntimeError(repr(e)))
            if not isinstance(e, Exception):
                raise
        finally:
            step.stage = AveragingStage.FINISHED
            if not step.done():
                step.set_exception(RuntimeError("Internal sanity check failed: averager.step left future pending."))

    @contextlib.contextmanager
    def _register_allreduce_group(self, group_info: GroupInfo):
        """Make the round addressable by incoming ``rpc_aggregate_part`` calls before the runner exists."""
        try:
            self._running_groups[group_info.group_id] = asyncio.Future()
            self._pending_groups_registered.set()
            yield
        finally:
            maybe_future = self._running_groups.pop(group_info.group_id, None)
            if maybe_future is not None and not maybe_future.done():
                logger.warning(f"All-reduce group {group_info.group_id} did not finish.")
            self._pending_groups_registered.set()

    async def _aggregate_with_group(self, group_info: GroupInfo, min_vector_size: int, **kwargs) -> GatheredData:
        """Run one all-reduce round in an assembled group; returns what the peers gathered."""
        try:
            unpacked = [self.serializer.loads(blob) for blob in group_info.gathered]
            bandwidths = [item[0] for item in unpacked]
            modes = tuple(AveragingMode(item[1]) for item in unpacked)
            user_gathered = dict(zip(group_info.peer_ids, (self.serializer.loads(item[2]) for item in unpacked)))
            device_infos = [item[3] if len(item) > 3 else None for item in unpacked]

            # peers that cannot reduce get no span; the rest share the vector according to their bandwidth
            download_bandwidths = [thr if mode != AveragingMode.CLIENT else 0.0 for thr, mode in zip(bandwidths, modes)]
            peer_fractions = await asyncio.get_event_loop().run_in_executor(
                None, load_balance_peers, self.total_size, download_bandwidths, min_vector_size)

            if self._device_endpoint is not None and self._device_endpoint.can_run_with(device_infos, modes):
                await self._run_device_allreduce_(group_info, peer_fractions, modes, device_infos, **kwargs)
                return user_gathered

            async with enter_asynchronously(self.get_tensors()) as local_tensors:
                await self._run_allreduce_inplace_(local_tensors, group_info, peer_fractions=peer_fractions,
                                                   modes=modes, **kwargs)
                return user_gathered
        except BaseException as e:
            if isinstance(e, Exception):
                logger.debug(e, exc_info=True)
                raise MatchmakingException(f"Unable to run All-Reduce: {e!r}")
            raise

    def _make_allreduce_runner(self, **kwargs) -> AllReduceRunner:
        """Factory of the RPC round's runner (a seam for subclasses, e.g. tests that inject host-side faults)."""
        return AllReduceRunner(**kwargs)

    async def _run_allreduce_inplace_(self, tensors: Sequence[torch.Tensor], group_info: GroupInfo,
                                      group_id: Optional[bytes] = None, **kwargs) -> None:
        """RPC data path: stream parts to groupmates and add the averaged deltas to ``tensors`` in place."""
        group_id = group_info.group_id if group_id is None else group_id
        host_tensors = [t if not t.is_cuda else t.detach().to("cpu", torch.float32) for t in tensors]
        runner = self._make_allreduce_runner(p2p=self._p2p, servicer_type=type(self), prefix=self.prefix, tensors=host_tensors,
                                 group_id=group_id, ordered_peer_ids=group_info.peer_ids, **kwargs)
        assert group_id in self._running_groups, f"Group id {group_id} was not registered in _register_allreduce_group"
        self._running_groups[group_id].set_result(runner)
        if runner.modes[group_info.peer_ids.index(self.peer_id)] != AveragingMode.AUX:
            async for tensor, update in azip(as_aiter(*tensors), runner):
                tensor.add_(update.to(tensor.device, tensor.dtype), alpha=self._averaging_alpha)
                self._state_updated.set()
        else:
            async for _ in runner:
                raise ValueError("aux peers should not receive averaged tensors")

    async def _run_device_allreduce_(self, group_info: GroupInfo, peer_fractions, modes, device_infos, *, weight: float,
                                     sender_timeout=None, reducer_timeout=None, endpoint=None, group_id=None,
                                     lock: bool = True, **_unused) -> None:
        """Device data path: launch the round's kernels over peer-mapped arenas and wait for the stream.

        Every member's weight travels inside the flags that its kernel publishes, so nothing is exchanged up front.
        """
        endpoint = endpoint if endpoint is not None else self._device_endpoint
        group_id = group_id if group_id is not None else group_info.group_id
        my_index = group_info.peer_ids.index(self.peer_id)
        pending = self._running_groups.get(group_id)
        if pending is not None and not pending.done():
            pending.set_result(None)  # no RPC runner in this round: the data moves through peer-mapped memory
        loop = asyncio.get_event_loop()
        async with (enter_asynchronously(self.lock_averaged_tensors) if lock else contextlib.AsyncExitStack()):
            status = await loop.run_in_executor(None, lambda: endpoint.run_round(
                group_id=group_id, my_index=my_index, device_infos=device_infos, modes=modes,
                peer_fractions=peer_fractions, weight=weight, alpha=self._averaging_alpha,
                sender_timeout=sender_timeout, reducer_timeout=reducer_timeout))
        self._state_updated.set()
        if status.failed_fraction > 0 or status.banned_senders:
            logger.warning(f"Averaging: received {(1 - status.failed_fraction) * 100:.1f}% results "
                           f"(banned senders: {status.banned_senders}, failed reducers: {status.failed_reducers})")

    @contextlib.contextmanager
    def get_tensors(self) -> Sequence[torch.Tensor]:
        """Context manager: exclusive access to the averaged tensors (no round touches them meanwhile)."""
        with self.lock_averaged_tensors:
            yield self._averaged_tensors

    # ---------------------------------------------------------------------------------------------- RPC handlers
    async def rpc_join_group(self, request: averaging_pb2.JoinRequest, context: P2PContext
                             ) -> AsyncIterator[averaging_pb2.MessageFromLeader]:
        """A peer asks us to lead it (see ``Matchmaking.rpc_join_group``)."""
        async for response in self._matchmaking.rpc_join_group(request, context):
            yield response

    async def rpc_aggregate_part(self, stream: AsyncIterator[PartMessage], context: P2PContext
                                 ) -> AsyncIterator[PartMessage]:
        """A groupmate sends us parts of the span that we reduce; forwarded to the round's ``AllReduceRunner``."""
        request = await anext(stream)
        if request.group_id not in self._running_groups:
            # the sender may have learned about the group a moment before we did
            await self._pending_groups_registered.wait()
        future = self._running_groups.get(request.group_id)
        if future is None:
            yield averaging_pb2.AveragingData(code=averaging_pb2.BAD_GROUP_ID)
            return
        group = await future
        if group is None:  # this round runs on the device path; nobody should stream parts to us
            yield averaging_pb2.AveragingData(code=averaging_pb2.PROTOCOL_VIOLATION)
            return
        async for message in group.rpc_aggregate_part(achain(as_aiter(request), stream), context):
            yield message

    # ---------------------------------------------------------------------------------------------- state sharing
    async def _declare_for_download_periodically(self) -> None:
        """While sharing is allowed, keep a record under ``{prefix}.all_averagers`` so that newcomers can find us."""
        download_key = f"{self.prefix}.all_averagers"
        sharing_was_allowed = self.allow_state_sharing
        while True:
            expiration_time = get_dht_time() + self.declare_state_period
            if self.allow_state_sharing or sharing_was_allowed:
                # a record with the value None retracts an earlier offer
                spawn(asyncio.wait_for(self.dht.store(
                    download_key, subkey=self.peer_id.to_bytes(),
                    value=self.state_sharing_priority if self.allow_state_sharing else None,
                    expiration_time=expiration_time, return_future=True), timeout=expiration_time - get_dht_time()))
                sharing_was_allowed = self.allow_state_sharing
            # re-declare when the state or priority changes, or when the record is about to expire
            try:
                await asyncio.wait_for(self._state_updated.wait(), timeout=max(0.0, expiration_time - get_dht_time()) * 0.5)
                self._state_updated.clear()
                await asyncio.sleep(0.05)  # coalesce bursts of updates
            except asyncio.TimeoutError:
                pass

    async def rpc_download_state(self, _request: averaging_pb2.DownloadRequest, _context: P2PContext
                                 ) -> AsyncIterator[averaging_pb2.DownloadData]:
        """Stream our current state: metadata first, then every tensor cut into chunks.

        A chunk whose ``tensor_part.dtype`` is set begins a new tensor (wire contract of the reference,
        hivemind/averaging/averager.py:628-651).
        """
        if not self.allow_state_sharing:
            return
        loop = asyncio.get_event_loop()
        metadata, tensors, infos = await loop.run_in_executor(None, self.get_current_state)
        if infos is None:
            infos = [CompressionInfo.from_tensor(tensor, key=i) for i, tensor in enumerate(tensors)]
        assert len(tensors) == len(infos)
        metadata = self.serializer.dumps(metadata)
        for tensor, info in zip(tensors, infos):
            message = await loop.run_in_executor(None, self.state_compression.compress, tensor, info)
            for part in split_for_streaming(message):
                if metadata is not None:
                    yield averaging_pb2.DownloadData(tensor_part=part, metadata=metadata)
                    metadata = None
                else:
                    yield averaging_pb2.DownloadData(tensor_part=part)

    def get_current_state(self) -> Tuple[Any, Sequence[torch.Tensor], Optional[Sequence[CompressionInfo]]]:
        """What this averager shares with peers that ask for its state: (metadata, tensors, tensor infos).

        Subclasses override this to add optimizer statistics and the like.
        """
        with self.get_tensors() as tensors:
            return dict(group_key=self.get_group_bits()), [t.detach().clone() for t in tensors], self.tensor_infos

    def load_state_from_peers(self, wait: bool = True, timeout: Optional[float] = None
                              ) -> Optional[Tuple[Any, Sequence[torch.Tensor]]]:
        """Download the freshest state offered by other peers: ``(metadata, tensors)`` or None if nobody answered.

        Donors are tried in order of decreasing ``state_sharing_priority``.
        """
        future = MPFuture()
        assert self._thread is not None, "the averager is not running"

        async def _runner():
            try:
                future.set_result(await self._load_state_from_peers(timeout))
            except BaseException as e:
                if not future.done():
                    future.set_exception(e if isinstance(e, Exception) else RuntimeError(repr(e)))

        self._thread.submit(_runner())
        return future.result(timeout=timeout) if wait else future

    async def _load_state_from_peers(self, timeout: Optional[float] = None):
        if timeout is None:  # per-chunk deadline of the download stream
            timeout = self.next_chunk_timeout if self.next_chunk_timeout is not None else self.request_timeout
        key_manager = self._matchmaking.group_key_manager
        peer_priority, _ = (await self.dht.get(f"{key_manager.prefix}.all_averagers", latest=True, return_future=True)) or ({}, None)
        peer_priority = {PeerID(peer_id): (float(info.value), random.random())  # random tie-breaker
                         for peer_id, info in peer_priority.items()
                         if isinstance(info, ValueWithExpiration) and isinstance(info.value, (float, int))}
        if not isinstance(peer_priority, dict) or len(peer_priority) == 0:
            logger.info(f"Averager could not load state from peers: peer dict empty or corrupted {peer_priority}")
            return None
        metadata = None
        for peer in sorted(peer_priority.keys(), key=peer_priority.get, reverse=True):
            if peer == self.peer_id:
                continue
            logger.info(f"Downloading parameters from peer {peer}")
            try:
                stub = type(self).get_stub(self._p2p, peer, namespace=self.prefix)
                stream = await stub.rpc_download_state(averaging_pb2.DownloadRequest())
                current_tensor_parts, tensors = [], []
                async for message in aiter_with_timeout(stream, timeout=timeout):
                    if message.metadata:
                        metadata = self.serializer.loads(message.metadata)
                    if message.tensor_part.dtype and current_tensor_parts:
                        tensors.append(deserialize_torch_tensor(combine_from_streaming(current_tensor_parts)))
                        current_tensor_parts = []
                    current_tensor_parts.append(message.tensor_part)
                if current_tensor_parts:
                    tensors.append(deserialize_torch_tensor(combine_from_streaming(current_tensor_parts)))
                if not metadata:
                    logger.debug(f"Peer {peer} did not send its state")
                    continue
                logger.info(f"Finished downloading state from {peer}")
                return metadata, tensors
            except Exception as e:
                logger.exception(f"Failed to download state from {peer} - {e!r}")
        return None

    # ---------------------------------------------------------------------------------------------- group bits
    def get_group_bits(self, wait: bool = True):
        """The current suffix of this averager's group key (see ``GroupKeyManager``)."""
        bits = self._matchmaking.group_key_manager.group_bits
        if wait:
            return bits
        future = MPFuture()
        future.set_result(bits)
        return future

    def set_group_bits(self, group_bits: str, wait: bool = True):
        assert all(bit in "01" for bit in group_bits)
        future = MPFuture()

        def _set():
            self._matchmaking.group_key_manager.group_bits = group_bits
            future.set_result(None)

        self._thread.loop.call_soon_threadsafe(_set)
        return future.result() if wait else future

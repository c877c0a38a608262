"""Splitting tensors into parts for the butterfly all-reduce, and reducing parts from several senders (host path).

Contract (hivemind/averaging/partition.py:17-285): tensors are flattened and cut into parts whose *compressed* size is
about ``part_size_bytes``; consecutive parts are assigned to peers so that peer i receives ``peer_fractions[i]`` of all
elements; parts never span two tensors. The reducer accumulates ``weight * part`` from every sender of a part index
and releases ``sum / total weight`` once all live senders have delivered; a failed sender shrinks the quorum.
The same assignment arithmetic (``compute_part_layout``) drives the device butterfly, which works on a flat arena.
"""
from __future__ import annotations

import asyncio
from collections import deque
from dataclasses import dataclass
from typing import AsyncIterable, AsyncIterator, Deque, List, Optional, Sequence, Tuple, TypeVar

import numpy as np
import torch

from hivemind_b200.compression import (CompressionBase, CompressionInfo, Float16Compression, NoCompression,
                                       ScaledFloat16Compression)
from hivemind_b200.compression.serialization import is_light_to_encode
from hivemind_b200.proto import runtime_pb2
from hivemind_b200.utils import amap_in_executor, as_aiter, get_logger

T = TypeVar("T")
DEFAULT_PART_SIZE_BYTES = 2 ** 19
logger = get_logger(__name__)


@dataclass(frozen=True)
class PartSpec:
    tensor_index: int
    start: int  # first element inside the flattened tensor
    length: int
    owner: int  # index of the peer that reduces this part


def compute_part_layout(numels: Sequence[int], element_sizes: Sequence[int], compression_ratios: Sequence[float],
                        peer_fractions: Sequence[float], part_size_bytes: int, align: int = 1) -> List[PartSpec]:
    """Cut every tensor into parts and give each part to a peer.

    A part goes to the current peer until that peer's cumulative share (``pivot``) of all elements is used up;
    a part that straddles the boundary is split there, so that peer shares are exact (up to ``align`` elements).
    """
    total = int(sum(numels))
    fractions = np.asarray(peer_fractions, dtype=np.float64)
    pivots = (np.cumsum(fractions) / max(fractions.sum(), 1e-30) * total).astype(np.int64)
    pivots[-1] = total
    specs: List[PartSpec] = []
    peer, consumed = 0, 0
    for t, n in enumerate(numels):
        part_elems = max(1, int(part_size_bytes / (element_sizes[t] * compression_ratios[t])))
        if align > 1:  # device path: keep every part boundary inside a tensor on an aligned element
            part_elems = max(align, part_elems // align * align)
        offset = 0
        while offset < n:
            length = min(part_elems, n - offset)
            while peer < len(pivots) - 1 and consumed >= pivots[peer]:
                peer += 1
            if consumed + length > pivots[peer] and peer < len(pivots) - 1:
                cut = int(pivots[peer] - consumed)  # finish this peer's share exactly
                if align > 1:
                    cut = cut // align * align
                if cut > 0:
                    length = cut
                else:  # the aligned cut would be empty: the whole part goes to the next peer
                    peer += 1
                    continue
            specs.append(PartSpec(t, offset, length, peer))
            offset += length
            consumed += length
    return specs


class TensorPartContainer:
    """Holds local tensors split into parts, serves compressed input parts and collects output deltas.

    :param tensors: local tensors; averaged values are returned as deltas with the same shapes
    :param peer_fractions: share of all elements that each peer reduces (zeros for client-mode peers)
    :param compression: codec for parts sent to other peers
    :param part_size_bytes: target size of one compressed part
    :param tensor_infos: per-tensor ``CompressionInfo`` (role, key) for adaptive codecs
    :param return_deltas: if True, outputs are ``average - local``; otherwise the averages themselves
    :param prefetch: how many parts may be compressed ahead of the consumer
    """

    def __init__(self, tensors: Sequence[torch.Tensor], peer_fractions: Sequence[float],
                 compression: CompressionBase = NoCompression(), part_size_bytes: int = DEFAULT_PART_SIZE_BYTES,
                 tensor_infos: Optional[Sequence[CompressionInfo]] = None, return_deltas: bool = True, prefetch: int = 1):
        if tensor_infos is None:
            tensor_infos = tuple(CompressionInfo.from_tensor(x, key=i) for i, x in enumerate(tensors))
        assert len(tensor_infos) == len(tensors), "compression types do not match the number of tensors"
        self.local_tensors, self.peer_fractions, self.group_size = tensors, peer_fractions, len(peer_fractions)
        self.compression, self.part_size_bytes, self.tensor_infos = compression, part_size_bytes, tensor_infos
        self.total_size = sum(tensor.numel() for tensor in tensors)
        self.failed_size = 0
        self.return_deltas = return_deltas
        self.prefetch = prefetch

        ratios = [compression.estimate_compression_ratio(info) for info in tensor_infos]
        layout = compute_part_layout([t.numel() for t in tensors], [t.element_size() for t in tensors], ratios,
                                     peer_fractions, part_size_bytes)
        self._input_parts_by_peer: List[Deque[Tuple[torch.Tensor, CompressionInfo]]] = [deque() for _ in range(self.group_size)]
        self._output_parts_by_peer: List[Deque[torch.Tensor]] = [deque() for _ in range(self.group_size)]
        self._inputs_consumed_by_peer = [False] * self.group_size
        self._output_part_available = [asyncio.Event() for _ in range(self.group_size)]
        self._outputs_registered_by_peer = [0] * self.group_size
        self._outputs_consumed = False
        self.finished = asyncio.Event()
        self.num_parts_by_tensor = [0] * len(tensors)
        self.num_parts_by_peer = [0] * self.group_size
        flats = [t.detach().reshape(-1) for t in tensors]
        part_index_in_tensor = [0] * len(tensors)
        for spec in layout:
            part = flats[spec.tensor_index][spec.start:spec.start + spec.length]
            info = tensor_infos[spec.tensor_index].get_part(part_index_in_tensor[spec.tensor_index],
                                                            max(1, int(part_size_bytes / (part.element_size() * ratios[spec.tensor_index]))))
            part_index_in_tensor[spec.tensor_index] += 1
            self.num_parts_by_tensor[spec.tensor_index] += 1
            self.num_parts_by_peer[spec.owner] += 1
            self._input_parts_by_peer[spec.owner].append((part, info))
        self._part_owner_order = [spec.owner for spec in layout]
        self._specs_by_peer: List[List[PartSpec]] = [[] for _ in range(self.group_size)]
        for spec in layout:
            self._specs_by_peer[spec.owner].append(spec)

    @torch.no_grad()
    def get_raw_input_parts(self, peer_index: int) -> Tuple[torch.Tensor, ...]:
        """Uncompressed parts that peer ``peer_index`` is responsible for (used for the local span)."""
        assert not self._inputs_consumed_by_peer[peer_index], "input parts of a given peer are already deallocated."
        self._inputs_consumed_by_peer[peer_index] = True
        input_parts = tuple(part for part, compression in self._input_parts_by_peer[peer_index])
        self._input_parts_by_peer[peer_index].clear()
        return input_parts

    @torch.no_grad()
    async def iterate_input_parts_for(self, peer_index: int) -> AsyncIterator[runtime_pb2.Tensor]:
        """Compressed parts for peer ``peer_index``, produced in a background thread with a bounded look-ahead."""
        assert not self._inputs_consumed_by_peer[peer_index], "input parts of a given peer are already deallocated."
        self._inputs_consumed_by_peer[peer_index] = True
        parts_aiter = as_aiter(*self._input_parts_by_peer[peer_index])
        light = isinstance(self.compression, (NoCompression, Float16Compression, ScaledFloat16Compression))
        async for serialized_part in amap_in_executor(
                lambda x_and_info: self.compression.compress(*x_and_info), parts_aiter, max_prefetch=self.prefetch,
                inline=lambda x_and_info: light and is_light_to_encode(x_and_info[0], runtime_pb2.CompressionType.NONE)):
            yield serialized_part
        self._input_parts_by_peer[peer_index].clear()

    def register_processed_part(self, peer_index: int, part_index: int, part: torch.Tensor) -> None:
        """Record the averaged delta for the ``part_index``-th part handled by ``peer_index`` (in order)."""
        if part_index != self._outputs_registered_by_peer[peer_index]:
            raise ValueError(f"Could not register part #{part_index} from peer #{peer_index}, "
                             f" expected part index: {self._outputs_registered_by_peer[peer_index]}")
        self._output_parts_by_peer[peer_index].append(part)
        self._outputs_registered_by_peer[peer_index] += 1
        self._output_part_available[peer_index].set()

    def register_failed_reducer(self, peer_index: int) -> None:
        """Peer ``peer_index`` will not deliver its remaining parts: keep our own values there (zero delta)."""
        for part_index in range(self._outputs_registered_by_peer[peer_index], self.num_parts_by_peer[peer_index]):
            spec = self._specs_by_peer[peer_index][part_index]
            self.failed_size += spec.length
            if self.return_deltas:
                self.register_processed_part(peer_index, part_index, torch.zeros(spec.length))
            else:
                local = self.local_tensors[spec.tensor_index].detach().reshape(-1)
                self.register_processed_part(peer_index, part_index, local[spec.start:spec.start + spec.length].clone())

    async def iterate_output_tensors(self) -> AsyncIterable[torch.Tensor]:
        """Yield averaged deltas (or averages), one per local tensor, as soon as all of a tensor's parts are in."""
        assert not self._outputs_consumed, "output tensors are already iterated and no longer available."
        self._outputs_consumed = True
        part_cursor = 0
        for tensor_index in range(len(self.local_tensors)):
            tensor_parts = []
            while len(tensor_parts) < self.num_parts_by_tensor[tensor_index]:
                owner = self._part_owner_order[part_cursor]
                while not self._output_parts_by_peer[owner]:
                    self._output_part_available[owner].clear()
                    await self._output_part_available[owner].wait()
                    if self.finished.is_set():
                        raise AllreduceException("All-reduce was terminated during iteration")
                tensor_parts.append(self._output_parts_by_peer[owner].popleft())
                part_cursor += 1
            local = self.local_tensors[tensor_index]
            if tensor_parts:
                flat = tensor_parts[0].reshape(-1) if len(tensor_parts) == 1 else torch.cat([p.reshape(-1) for p in tensor_parts])
                yield flat.view(local.shape).to(local.dtype)
            else:
                yield torch.zeros_like(local)

    def __del__(self):
        self.finalize()

    def finalize(self) -> None:
        """Release buffers and wake up anybody still waiting for outputs."""
        if not self.finished.is_set():
            for peer_index in range(self.group_size):
                self._inputs_consumed_by_peer[peer_index] = True
                self._output_part_available[peer_index].set()
                self._input_parts_by_peer[peer_index].clear()
                self._output_parts_by_peer[peer_index].clear()
            if self.failed_size != 0:
                logger.warning(f"Averaging: received {(1. - self.failed_size / max(self.total_size, 1)) * 100:.1f}% results")
            self._outputs_consumed = True
            self.finished.set()


class TensorPartReducer:
    """Accumulates the parts that several senders submit for this peer's span, one part index at a time.

    :param part_shapes: shapes of the parts this peer reduces, in order
    :param num_senders: how many peers send parts (the local peer included, if it sends)
    """

    def __init__(self, part_shapes: Sequence[torch.Size], num_senders: int):
        self.part_shapes, self.num_senders, self.num_parts = part_shapes, num_senders, len(part_shapes)
        self.current_part_index = -1  # index in local_parts of the part being accumulated
        self.current_part_accumulated_from = 0  # number of senders that delivered the current part
        self.accumulator = None
        self.denominator = 0.0
        self.current_part_future = asyncio.Future()
        self.finished = asyncio.Event()
        self.num_parts_received = [0 for _ in range(self.num_senders)]
        self.sender_failed_after = [float("inf") for _ in range(self.num_senders)]
        self.num_current_senders = self.num_senders
        self.reset_accumulators()

    def reset_accumulators(self) -> None:
        """Start the next part (or finish if there is none)."""
        assert self.current_part_accumulated_from == self.num_current_senders or self.current_part_index == -1
        if self.current_part_index >= self.num_parts - 1:
            self.finalize()
            return
        self.current_part_index += 1
        self.current_part_accumulated_from = 0
        self.current_part_future = asyncio.Future()
        self.num_current_senders = sum(self.current_part_index < failed_index for failed_index in self.sender_failed_after)
        self.accumulator = torch.zeros(self.part_shapes[self.current_part_index])
        self.denominator = 0.0

    async def accumulate_part(self, sender_index: int, part_index: int, tensor_part: torch.Tensor,
                              weight: float = 1.0) -> torch.Tensor:
        """Add a sender's part; resolves to the average of that part once every live sender has contributed."""
        assert 0 <= sender_index < self.num_senders, "invalid sender index"
        assert 0 <= part_index < self.num_parts, "invalid part index"
        if self.finished.is_set():  # a straggler after the last part (or after a shutdown) gets a clean error
            raise AllreduceException(f"attempted to aggregate part in a finalized {self.__class__.__name__}")
        self.num_parts_received[sender_index] += 1
        while part_index > self.current_part_index:
            # wait for previous parts to finish; a sender may run ahead of the others
            finished = asyncio.create_task(self.finished.wait())
            try:
                await asyncio.wait({self.current_part_future, finished}, return_when=asyncio.FIRST_COMPLETED)
            finally:
                finished.cancel()  # otherwise one pending task per wait outlives the round
            if self.finished.is_set():
                raise AllreduceException(f"attempted to aggregate part in a finalized {self.__class__.__name__}")
        if self.sender_failed_after[sender_index] != float("inf"):
            raise BannedException(f"sender {sender_index} was banned in background")
        assert part_index == self.current_part_index
        current_part_future = self.current_part_future
        if part_index < self.sender_failed_after[sender_index]:
            self.accumulator.add_(tensor_part.to(self.accumulator.dtype), alpha=weight)
            self.current_part_accumulated_from += 1
            self.denominator += weight
            self.check_current_part_finished()
        return await current_part_future

    def on_sender_failed(self, sender_index: int) -> None:
        """Exclude the sender from all parts it has not submitted yet."""
        self.sender_failed_after[sender_index] = self.num_parts_received[sender_index]
        if self.finished.is_set():
            return
        if self.current_part_index == self.num_parts_received[sender_index]:
            self.num_current_senders -= 1
            self.check_current_part_finished()

    def check_current_part_finished(self) -> None:
        assert self.current_part_accumulated_from <= self.num_current_senders
        if self.current_part_accumulated_from == self.num_current_senders:
            self.current_part_future.set_result(self.accumulator.div_(max(self.denominator, 1e-30))
                                                if self.denominator > 0 else self.accumulator)
            self.reset_accumulators()

    def finalize(self) -> None:
        if not self.finished.is_set():
            if hasattr(self, "current_part_future"):
                self.current_part_future.cancel()
                del self.accumulator
            self.finished.set()
            if self.num_parts != 0 and self.num_senders != 0:
                parts_expected = self.num_parts * self.num_senders
                parts_received = sum(self.num_parts_received)
                if parts_expected != parts_received:
                    logger.warning(f"Reducer: received {parts_received / parts_expected * 100:.1f}% of input tensors")

    def __del__(self):
        self.finalize()


class AllreduceException(Exception):
    """An error during all-reduce that may be retried."""


class BannedException(AllreduceException):
    """A sender (or reducer) was excluded from the round for being late or faulty."""

"""RPC butterfly all-reduce under host-side faults: peers that raise before the round, senders that fail or stall
mid-stream, reducers that fail or stall, a cancelled peer. The healthy peers must finish within their timeouts and
end up with either the average over the peers that delivered or their own values, element by element (modelled on
the reference's tests/test_allreduce_fault_tolerance.py; all faults are exceptions, sleeps or error codes on the host).
"""
import asyncio
from enum import Enum, auto
from typing import AsyncIterator

import pytest
import torch

from hivemind_b200 import DHT, DecentralizedAverager
from hivemind_b200.averaging.allreduce import AllReduceRunner
from hivemind_b200.proto import averaging_pb2
from hivemind_b200.utils.asyncio import aenumerate, anext


class Fault(Enum):
    NONE = auto()
    FAIL_BEFORE = auto()
    FAIL_SENDING = auto()
    SLOW_SENDING = auto()
    FAIL_REDUCING = auto()
    SLOW_REDUCING = auto()
    CANCEL = auto()


class FaultyAllReduceRunner(AllReduceRunner):
    def __init__(self, *args, fault: Fault, **kwargs):
        self.fault = fault
        super().__init__(*args, **kwargs)

    async def rpc_aggregate_part(self, stream, context) -> AsyncIterator[averaging_pb2.AveragingData]:
        if self.fault in (Fault.FAIL_REDUCING, Fault.SLOW_REDUCING):
            async for i, message in aenumerate(super().rpc_aggregate_part(stream, context)):
                yield message
                if i == 2:
                    if self.fault == Fault.FAIL_REDUCING:
                        yield averaging_pb2.AveragingData(code=averaging_pb2.INTERNAL_ERROR)
                        break
                    await asyncio.sleep(10)
        elif self.fault == Fault.CANCEL:
            yield averaging_pb2.AveragingData(code=averaging_pb2.CANCELLED)
        else:
            async for message in super().rpc_aggregate_part(stream, context):
                yield message

    async def _generate_input_for_peer(self, peer_index: int) -> AsyncIterator[averaging_pb2.AveragingData]:
        parts = self.tensor_part_container.iterate_input_parts_for(peer_index)
        first = await anext(parts)
        yield averaging_pb2.AveragingData(code=averaging_pb2.PART_FOR_AVERAGING, group_id=self.group_id,
                                          tensor_part=first, weight=self.weight)
        if self.fault in (Fault.FAIL_SENDING, Fault.SLOW_SENDING):
            counts = self.tensor_part_container.num_parts_by_peer
            last_reducer = max(i for i, n in enumerate(counts) if n > 0)
            if peer_index == last_reducer:
                if self.fault == Fault.FAIL_SENDING:
                    raise RuntimeError("injected: sender fails after its first part")
                await asyncio.sleep(10)
        async for part in parts:
            yield averaging_pb2.AveragingData(tensor_part=part, weight=self.weight)


class FaultyAverager(DecentralizedAverager):
    def __init__(self, *args, fault: Fault = Fault.NONE, **kwargs):
        self.fault = fault
        super().__init__(*args, **kwargs)

    def _make_allreduce_runner(self, **kwargs):
        if self.fault == Fault.FAIL_BEFORE:
            raise RuntimeError("injected: peer fails before the round starts")
        return FaultyAllReduceRunner(fault=self.fault, **kwargs)


def _make_tensors():
    return [torch.rand(16, 1024), -torch.rand(3, 8192), 2 * torch.randn(4, 4, 4), torch.randn(1024, 1024)]


@pytest.mark.parametrize("fault0, fault1", [
    (Fault.NONE, Fault.FAIL_BEFORE),
    (Fault.FAIL_BEFORE, Fault.FAIL_BEFORE),
    (Fault.SLOW_SENDING, Fault.FAIL_SENDING),
    (Fault.FAIL_SENDING, Fault.FAIL_BEFORE),
    (Fault.SLOW_REDUCING, Fault.FAIL_SENDING),
    (Fault.FAIL_REDUCING, Fault.FAIL_REDUCING),
    (Fault.NONE, Fault.CANCEL),
])
def test_fault_tolerance(fault0: Fault, fault1: Fault):
    """Five peers in ONE group, two of them faulty. Whether all five find each other within the matchmaking window is
    not what this test is about (on a loaded machine a peer can come late and the others start without it, which
    changes every expected value), so an attempt whose group came out smaller is repeated."""
    for attempt in range(4):
        if _fault_tolerance_scenario(fault0, fault1):
            return
    pytest.fail("the five peers did not assemble into one group in four attempts")


def _fault_tolerance_scenario(fault0: Fault, fault1: Fault) -> bool:
    torch.manual_seed(0)
    dht = DHT(start=True)
    averagers = []
    for i in range(5):
        averagers.append(FaultyAverager(
            _make_tensors(), DHT(initial_peers=dht.get_visible_maddrs(), start=True), prefix="test",
            request_timeout=0.5, min_matchmaking_time=2.0, target_group_size=5, next_chunk_timeout=1.0,
            allreduce_timeout=6, part_size_bytes=2 ** 16, client_mode=(i == 1), start=True,
            fault=fault0 if i == 0 else fault1 if i == 1 else Fault.NONE))
    try:
        numerators, denominator = [0, 0, 0, 0], 0
        for averager in averagers:
            if averager.fault not in (Fault.FAIL_BEFORE, Fault.CANCEL):
                with averager.get_tensors() as tensors:
                    for i, tensor in enumerate(tensors):
                        numerators[i] = numerators[i] + tensor.clone()
                denominator += 1
        flat_ref = torch.cat([(n / denominator).flatten() for n in numerators])
        before = []
        for averager in averagers:
            with averager.get_tensors() as tensors:
                before.append(torch.cat([t.flatten() for t in tensors]))

        futures = [averager.step(timeout=10, wait=False, allow_retries=False) for averager in averagers]
        for averager, future in zip(averagers, futures):
            if averager.fault == Fault.CANCEL:
                future.cancel()
        group_sizes = []
        for future in futures[2:]:
            gathered = future.result(timeout=30)
            assert gathered is not None  # the healthy peers always finish
            group_sizes.append(len(gathered))
        if Fault.CANCEL not in (fault0, fault1) and any(size != len(averagers) for size in group_sizes):
            print(f"group sizes {group_sizes}: somebody missed the matchmaking window, repeating the attempt")
            return False  # not the scenario under test

        for averager, previous in zip(averagers[2:], before[2:]):
            with averager.get_tensors() as tensors:
                after = torch.cat([t.flatten() for t in tensors])
            to_reference, to_local = (flat_ref - after).abs(), (previous - after).abs()
            if Fault.CANCEL in (fault0, fault1):
                continue  # a late cancel may leave any mix of results with and without the cancelled peer
            if fault0 == Fault.NONE:  # only the client-mode peer 1 can have failed: nobody lost a reducer
                assert to_reference.max() < 1e-5
            elif all(f in (Fault.FAIL_REDUCING, Fault.SLOW_REDUCING) for f in (fault0, fault1)):
                assert (to_reference < 1e-5).float().mean() > 0.5
                assert torch.all(torch.minimum(to_reference, to_local) < 1e-5)  # the average, or the old value
            else:
                assert (to_reference < 1e-5).float().mean() > 0.5
        return True
    finally:
        for averager in averagers:
            averager.shutdown()
        dht.shutdown()

"""Unit tests of the RPC butterfly's building blocks: part container and reducer.

Modelled on the behaviours that the reference pins in tests/test_allreduce.py (partitioning round trips, edge cases,
asynchronous producers/consumers, reducer arithmetic), plus the partial-failure rules of
hivemind/averaging/partition.py:128-160,230-277 (zero delta for a failed reducer, shrinking denominators for failed
senders).
"""
import asyncio
import random

import pytest
import torch

from hivemind_b200.averaging.partition import (AllreduceException, BannedException, TensorPartContainer,
                                               TensorPartReducer)
from hivemind_b200.compression import Float16Compression, deserialize_torch_tensor


def _run(coro):
    return asyncio.new_event_loop().run_until_complete(coro)


@pytest.mark.parametrize("fractions", [(0.25, 0.25, 0.5), (0.0, 1.0), (0.6, 0.0, 0.4, 0.0), (1.0,)])
@pytest.mark.parametrize("part_size_bytes", [64, 1000, 2 ** 20])
def test_partitioning_is_an_identity_when_every_part_comes_back(fractions, part_size_bytes):
    async def scenario():
        torch.manual_seed(0)
        tensors = [torch.randn(30), torch.randn(7, 11), torch.randn(1), torch.zeros(0), torch.randn(128, 3)]
        container = TensorPartContainer(tensors, fractions, part_size_bytes=part_size_bytes, return_deltas=False)
        total = 0
        for peer, fraction in enumerate(fractions):
            parts = container.get_raw_input_parts(peer)
            assert len(parts) == container.num_parts_by_peer[peer]
            if fraction == 0.0:
                assert len(parts) == 0  # client-mode peers reduce nothing
            total += sum(p.numel() for p in parts)
            for index, part in enumerate(parts):
                assert part.numel() * part.element_size() <= max(part_size_bytes, part.element_size())
                container.register_processed_part(peer, index, part.clone())
        assert total == sum(t.numel() for t in tensors)
        outputs = [t async for t in container.iterate_output_tensors()]
        assert len(outputs) == len(tensors)
        for out, ref in zip(outputs, tensors):
            assert out.shape == ref.shape and torch.equal(out, ref)

    _run(scenario())


def test_parts_follow_fractions_and_travel_compressed():
    async def scenario():
        tensors = [torch.randn(1000), torch.randn(3000)]
        container = TensorPartContainer(tensors, (0.1, 0.6, 0.3), compression=Float16Compression(), part_size_bytes=512)
        sizes = []
        for peer in range(3):
            restored = [deserialize_torch_tensor(msg) async for msg in container.iterate_input_parts_for(peer)]
            sizes.append(sum(p.numel() for p in restored))
            with pytest.raises(AssertionError):
                container.get_raw_input_parts(peer)  # a peer's inputs are handed out once
        assert sum(sizes) == 4000
        for size, fraction in zip(sizes, (0.1, 0.6, 0.3)):
            assert abs(size - 4000 * fraction) <= 260  # spans end on part boundaries

    _run(scenario())


def test_out_of_order_registration_is_rejected_and_failed_reducers_leave_zero_deltas():
    async def scenario():
        tensors = [torch.arange(100, dtype=torch.float32)]
        container = TensorPartContainer(tensors, (0.5, 0.5), part_size_bytes=100)
        first = container.get_raw_input_parts(0)
        assert len(first) >= 2
        with pytest.raises(ValueError):
            container.register_processed_part(0, 1, torch.zeros_like(first[1]))
        container.register_processed_part(0, 0, torch.ones_like(first[0]))
        container.register_failed_reducer(0)  # the rest of peer 0's span
        container.register_failed_reducer(1)  # all of peer 1's span
        (delta,) = [t async for t in container.iterate_output_tensors()]
        assert torch.equal(delta[:first[0].numel()], torch.ones(first[0].numel()))
        assert torch.count_nonzero(delta[first[0].numel():]) == 0
        assert container.failed_size == 100 - first[0].numel()

    _run(scenario())


def test_consumer_waits_for_asynchronous_producers_and_finalize_unblocks_it():
    async def scenario():
        tensors = [torch.randn(64), torch.randn(64)]
        container = TensorPartContainer(tensors, (0.5, 0.5), part_size_bytes=64, return_deltas=False)
        inputs = [container.get_raw_input_parts(peer) for peer in range(2)]

        async def produce(peer):
            for index, part in enumerate(inputs[peer]):
                await asyncio.sleep(random.random() * 0.01)
                container.register_processed_part(peer, index, part * 2)

        producers = [asyncio.create_task(produce(peer)) for peer in (1, 0)]
        outputs = [t async for t in container.iterate_output_tensors()]
        await asyncio.gather(*producers)
        for out, ref in zip(outputs, tensors):
            assert torch.allclose(out, ref * 2)

        stuck = TensorPartContainer([torch.randn(10)], (1.0,), part_size_bytes=16)

        async def consume():
            return [t async for t in stuck.iterate_output_tensors()]

        consumer = asyncio.create_task(consume())
        await asyncio.sleep(0.02)
        assert not consumer.done()
        stuck.finalize()
        with pytest.raises(AllreduceException):
            await consumer

    _run(scenario())


def test_reducer_weighted_average_with_senders_running_ahead():
    async def scenario():
        torch.manual_seed(1)
        shapes = [torch.Size([8]), torch.Size([3]), torch.Size([5])]
        n = 4
        weights = [0.5, 1.0, 2.0, 1.5]
        data = [[torch.randn(shape) for shape in shapes] for _ in range(n)]
        reducer = TensorPartReducer(shapes, n)

        async def sender(index):
            results = []
            for part_index in range(len(shapes)):
                await asyncio.sleep(random.random() * 0.005)
                results.append(await reducer.accumulate_part(index, part_index, data[index][part_index], weights[index]))
            return results

        results = await asyncio.gather(*[sender(i) for i in range(n)])
        for part_index in range(len(shapes)):
            ref = sum(w * data[i][part_index] for i, w in enumerate(weights)) / sum(weights)
            for i in range(n):
                assert torch.allclose(results[i][part_index], ref, atol=1e-6)
        assert reducer.finished.is_set()
        with pytest.raises(AllreduceException):
            await reducer.accumulate_part(0, 0, data[0][0])

    _run(scenario())


def test_reducer_drops_failed_senders_from_later_parts():
    async def scenario():
        shapes = [torch.Size([4]), torch.Size([4])]
        reducer = TensorPartReducer(shapes, 3)
        ones = torch.ones(4)
        # part 0: everybody contributes; part 1: sender 2 fails before sending it
        first = await asyncio.gather(*[reducer.accumulate_part(i, 0, ones * (i + 1)) for i in range(3)])
        assert torch.allclose(first[0], ones * 2)
        pending = [asyncio.create_task(reducer.accumulate_part(i, 1, ones * (i + 1))) for i in range(2)]
        await asyncio.sleep(0.01)
        assert not any(task.done() for task in pending)  # still waiting for sender 2
        reducer.on_sender_failed(2)
        second = await asyncio.gather(*pending)
        assert torch.allclose(second[0], ones * 1.5)  # mean of senders 0 and 1 only
        assert reducer.finished.is_set()

        banned = TensorPartReducer(shapes, 2)
        banned.on_sender_failed(1)
        with pytest.raises(BannedException):
            await banned.accumulate_part(1, 0, ones)
        assert torch.allclose(await banned.accumulate_part(0, 0, ones * 7), ones * 7)

    _run(scenario())

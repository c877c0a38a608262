"""Codec accuracy and round trips on CPU (thresholds of the reference's tests/test_compression.py:33-119)."""
import asyncio
import struct

import pytest
import torch

from hivemind_b200.compression import (CompressionInfo, Float16Compression, NoCompression, PerTensorCompression,
                                       RoleAdaptiveCompression, SizeAdaptiveCompression, TensorRole,
                                       Uniform8BitQuantization, combine_from_streaming, deserialize_tensor_stream,
                                       deserialize_torch_tensor, serialize_torch_tensor, split_for_streaming)
from hivemind_b200.compression.quantization import dynamic_code_table
from hivemind_b200.proto.runtime_pb2 import CompressionType


def _mse(a, b):
    return (a - b).pow(2).mean().item()


def test_accuracy_thresholds():
    torch.manual_seed(0)
    x = torch.randn(128, 128, 64)
    for ctype, bound in [(CompressionType.NONE, 1e-12), (CompressionType.MEANSTD_16BIT, 5e-8), (CompressionType.FLOAT16, 5e-8),
                         (CompressionType.QUANTILE_8BIT, 8e-4), (CompressionType.UNIFORM_8BIT, 8e-4),
                         (CompressionType.BLOCKWISE_8BIT, 8e-4)]:
        restored = deserialize_torch_tensor(serialize_torch_tensor(x, ctype))
        assert restored.shape == x.shape and restored.dtype == x.dtype
        assert _mse(restored, x) < bound, CompressionType.Name(ctype)
    zeros = torch.zeros(5, 5)
    for ctype in CompressionType.values():
        assert deserialize_torch_tensor(serialize_torch_tensor(zeros, ctype)).isfinite().all()


def test_scaled_fp16_handles_large_scales_and_rows():
    torch.manual_seed(1)
    x = torch.randn(64, 256) * torch.logspace(-2, 6, 64).unsqueeze(1) + 100.0
    restored = deserialize_torch_tensor(serialize_torch_tensor(x, CompressionType.MEANSTD_16BIT))
    rel = ((restored - x).norm(dim=1) / (x - x.mean(1, keepdim=True)).norm(dim=1)).max().item()
    assert rel < 5e-3
    plain = deserialize_torch_tensor(serialize_torch_tensor(x, CompressionType.FLOAT16))
    assert plain.isfinite().all()  # clamped, not inf


def test_dtype_requires_grad_and_bf16_round_trips():
    for dtype in (torch.float32, torch.float16, torch.bfloat16, torch.float64):
        x = torch.randn(3, 7).to(dtype).requires_grad_(True)
        y = deserialize_torch_tensor(serialize_torch_tensor(x, CompressionType.NONE))
        assert y.dtype == dtype and y.requires_grad and torch.equal(y.detach().float(), x.detach().float())
    ints = torch.arange(12).reshape(3, 4)
    assert torch.equal(deserialize_torch_tensor(serialize_torch_tensor(ints)), ints)
    with pytest.raises(ValueError):
        serialize_torch_tensor(ints, CompressionType.FLOAT16)
    bf = torch.randn(50).to(torch.bfloat16)
    msg = serialize_torch_tensor(bf, CompressionType.NONE)
    assert len(msg.buffer) == 4 * 50  # legacy mode ships fp32


def test_chunking_and_stream_deserialization():
    x = torch.randn(1000, 100)
    msg = serialize_torch_tensor(x, CompressionType.FLOAT16)
    chunks = list(split_for_streaming(msg, 16384))
    assert chunks[0].chunks == len(chunks) == (len(msg.buffer) - 1) // 16384 + 1
    assert combine_from_streaming(chunks) == msg
    y = torch.randn(3)
    chunks2 = list(split_for_streaming(serialize_torch_tensor(y), 16384))

    async def stream():
        yield chunks[:3]
        yield chunks[3:] + chunks2

    out = asyncio.new_event_loop().run_until_complete(deserialize_tensor_stream(stream()))
    assert len(out) == 2 and torch.allclose(out[0], x, atol=1e-2) and torch.equal(out[1], y)


def test_adaptive_codecs_choose_by_size_role_and_key():
    class Counting(NoCompression):
        def __init__(self):
            self.calls = 0

        def compress(self, *args, **kwargs):
            self.calls += 1
            return super().compress(*args, **kwargs)

    small, big, grads = Counting(), Counting(), Counting()
    codec = SizeAdaptiveCompression(100, less=small, greater_equal=big)
    for n in (10, 99, 100, 5000):
        t = torch.randn(n)
        codec.compress(t, CompressionInfo.from_tensor(t))
    assert (small.calls, big.calls) == (2, 2)
    by_role = RoleAdaptiveCompression(gradient=grads, default=small)
    t = torch.randn(4)
    by_role.compress(t, CompressionInfo.from_tensor(t, role=TensorRole.GRADIENT))
    by_role.compress(t, CompressionInfo.from_tensor(t, role=TensorRole.PARAMETER))
    assert grads.calls == 1 and small.calls == 3
    per = PerTensorCompression({"a": Float16Compression(), "b": Uniform8BitQuantization()})
    assert per.compress(t, CompressionInfo.from_tensor(t, key="a")).compression == CompressionType.FLOAT16
    assert per.compress(t, CompressionInfo.from_tensor(t, key="b")).compression == CompressionType.UNIFORM_8BIT
    assert abs(per.estimate_compression_ratio(CompressionInfo.from_tensor(t, key="b")) - 0.25) < 1e-9
    assert torch.allclose(per.extract(per.compress(t, CompressionInfo.from_tensor(t, key="a"))), t, atol=1e-2)


def test_dynamic_code_table_shape():
    code = dynamic_code_table()
    assert code.numel() == 256 and float(code.max()) == 1.0 and (code == 0).any()
    assert torch.equal(code, code.sort().values) and float(code.min()) < -0.9
    assert len(set(code.tolist())) >= 255


def test_received_messages_can_be_read_without_parsing_the_payload():
    """``split_length_delimited_field`` / ``TensorView`` / ``PartMessage``: the big ``buffer`` field stays a view of the
    received bytes, everything else equals what protobuf parses, for every codec and for odd messages."""
    from hivemind_b200.averaging.allreduce import PartMessage, _part_message
    from hivemind_b200.compression.serialization import TensorView, split_length_delimited_field
    from hivemind_b200.proto import averaging_pb2, runtime_pb2

    torch.manual_seed(0)
    tensor = torch.randn(3, 777)
    for name in runtime_pb2.CompressionType.keys():
        codec = runtime_pb2.CompressionType.Value(name)
        serialized = serialize_torch_tensor(tensor, codec)
        wire = serialized.SerializeToString()
        view = TensorView(memoryview(wire))
        assert (list(view.size), view.dtype, view.compression, view.requires_grad, view.chunks) == (
            list(serialized.size), serialized.dtype, serialized.compression, serialized.requires_grad, serialized.chunks)
        assert bytes(view.buffer) == serialized.buffer and view.to_message() == serialized
        assert view.buffer.obj is wire, "the payload is a view of the received bytes, not a copy"
        assert torch.equal(deserialize_torch_tensor(view), deserialize_torch_tensor(serialized))

        outer = _part_message(serialized, code=averaging_pb2.PART_FOR_AVERAGING, group_id=b"g" * 20, weight=0.75)
        parsed = averaging_pb2.AveragingData.FromString(outer.SerializeToString())
        lazy = PartMessage.FromString(outer.SerializeToString())
        assert parsed.tensor_part == serialized and parsed.weight == 0.75, "any protobuf parser reads the raw form"
        assert (lazy.code, lazy.group_id, lazy.peer_id, lazy.weight) == (parsed.code, parsed.group_id, parsed.peer_id, 0.75)
        assert torch.equal(deserialize_torch_tensor(lazy.tensor_part), deserialize_torch_tensor(serialized))

    # messages without a tensor, with fields in another order, with unknown fields of every wire type
    bare = PartMessage.FromString(averaging_pb2.AveragingData(code=averaging_pb2.CANCELLED).SerializeToString())
    assert bare.code == averaging_pb2.CANCELLED and len(bare.tensor_part.buffer) == 0 and bare.weight == 0.0
    inner = runtime_pb2.Tensor(buffer=b"abc", dtype="uint8", size=[3]).SerializeToString()
    shuffled = (b"\x22" + bytes([len(inner)]) + inner      # tensor_part first
                + b"\x29" + struct.pack("<d", 2.5)           # weight (fixed64)
                + b"\x98\x06\x07"                          # unknown field 99, varint
                + b"\x9d\x06" + b"\x01\x02\x03\x04"       # unknown field 99, fixed32
                + b"\x08\x05")                             # code last
    lazy = PartMessage.FromString(shuffled)
    assert (lazy.code, lazy.weight, bytes(lazy.tensor_part.buffer), lazy.tensor_part.dtype) == (5, 2.5, b"abc", "uint8")
    wanted, rest = split_length_delimited_field(memoryview(shuffled), 4)
    assert bytes(wanted) == inner and averaging_pb2.AveragingData.FromString(rest).code == 5
    for broken in (b"\x22\x7f" + b"x", b"\x08", b"\x0b", b"\x29\x00"):
        with pytest.raises((ValueError, IndexError)):
            split_length_delimited_field(memoryview(broken), 4)


def test_sorted_quantiles_agree_with_numpy():
    """The quantile codec takes chunk quantiles from one sort; they must be numpy's linear-interpolation quantiles."""
    import numpy as np

    from hivemind_b200.compression.quantization import _linear_quantiles, quantile_qq_approximation

    rng = np.random.default_rng(0)
    points = np.linspace(0, 1, 257, dtype=np.float32)
    for n in (1, 2, 7, 1000, 100_003):
        for values in (rng.standard_normal(n), rng.integers(0, 5, n).astype(np.float64), -np.sort(rng.standard_normal(n))):
            values = values.astype(np.float32)
            out = np.empty(257, dtype=np.float32)
            _linear_quantiles(values, points, out)
            assert np.allclose(out, np.quantile(values, points), atol=5e-5, rtol=1e-5)
            assert out[0] == values.min() and out[-1] == values.max() and np.all(np.diff(out) >= 0)
    # the two-level approximation for large inputs stays close to the exact quantiles
    big = rng.standard_normal(700_000).astype(np.float32)
    approx, exact = quantile_qq_approximation(big, 257), np.quantile(big, points)
    assert np.abs(approx - exact)[8:-8].max() < 0.02

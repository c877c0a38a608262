"""``RemoteExpert``: a ``torch.nn.Module`` whose forward and backward run on another peer.

The call is an autograd function: forward serialises the inputs with the compression the expert's schema asks for,
sends them (one unary message, or a chunked stream above ``MAX_UNARY_PAYLOAD_SIZE``) and returns the outputs;
backward sends inputs and output gradients and returns input gradients — the server re-runs the forward pass and
also trains the expert (reference: hivemind/moe/client/expert.py:33-233).
"""
from __future__ import annotations

from concurrent.futures import Future
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

import torch
import torch.nn as nn
from torch.autograd.function import once_differentiable

from hivemind_b200.compression import deserialize_torch_tensor, serialize_torch_tensor
from hivemind_b200.compression.serialization import _varint, deserialize_tensor_stream_into, stream_tensor_messages
from hivemind_b200.dht import DHT
from hivemind_b200.moe.client.remote_expert_worker import RemoteExpertWorker
from hivemind_b200.moe.expert_uid import ExpertInfo
from hivemind_b200.p2p import P2P, PeerID, StubBase
from hivemind_b200.p2p.control import DEFAULT_MAX_MSG_SIZE, MAX_UNARY_PAYLOAD_SIZE
from hivemind_b200.proto import runtime_pb2
from hivemind_b200.utils import MPFuture, MSGPackSerializer, nested_compare, nested_flatten, nested_pack

DUMMY = torch.empty(0, requires_grad=True)  # keeps the remote call in the graph when no input requires grad


def get_server_stub(p2p: P2P, server_peer_id: PeerID) -> StubBase:
    """A stub for the ConnectionHandler of the peer that hosts the expert."""
    from hivemind_b200.moe.server.connection_handler import ConnectionHandler

    return ConnectionHandler.get_stub(p2p, server_peer_id)


class RemoteExpert(nn.Module):
    """
    :param expert_info: uid and peer id of the hosting server
    :param p2p: a transport endpoint that can reach that peer
    """

    def __init__(self, expert_info: ExpertInfo, p2p: P2P):
        super().__init__()
        self._info, self.p2p = expert_info, p2p
        self._rpc_info: Optional[Dict[str, Any]] = None

    @property
    def uid(self) -> str:
        return self._info.uid

    @property
    def peer_id(self) -> PeerID:
        return self._info.peer_id

    @property
    def stub(self) -> StubBase:
        return get_server_stub(self.p2p, self.peer_id)

    @property
    def info(self) -> Dict[str, Any]:
        """The expert's schemas, fetched from the server on first use."""
        if self._rpc_info is None:
            reply = RemoteExpertWorker.run_coroutine(self.stub.rpc_info(runtime_pb2.ExpertUID(uid=self.uid)))
            self._rpc_info = MSGPackSerializer.loads(reply.serialized_info)
        return self._rpc_info

    def forward(self, *args, **kwargs):
        info = self.info
        assert len(kwargs) == len(info["keyword_names"]), f"Keyword args should be {info['keyword_names']}"
        kwargs = {name: kwargs[name] for name in info["keyword_names"]}  # the server's keyword order
        forward_inputs = (args, kwargs)
        if not nested_compare(forward_inputs, info["forward_schema"]):
            raise TypeError("Inputs do not match expert input schema. Did you pass the right number of parameters?")
        flat_outputs = _RemoteModuleCall.apply(DUMMY, self.uid, self.stub, info, *nested_flatten(forward_inputs))
        return nested_pack(flat_outputs, structure=info["outputs_schema"])

    def extra_repr(self) -> str:
        return f"uid={self.uid}, server_peer_id={self.peer_id}"


def _wrap_infos(infos: Sequence[Optional[ExpertInfo]], p2p: P2P) -> List[Optional[RemoteExpert]]:
    return [RemoteExpert(info, p2p) if info is not None else None for info in infos]


def create_remote_experts(infos: Union[Sequence[Optional[ExpertInfo]], MPFuture], dht: DHT, return_future: bool = False
                          ) -> Union[List[Optional[RemoteExpert]], Future]:
    """Turn ``ExpertInfo`` records (or a future of them) into ``RemoteExpert`` modules sharing the DHT's transport."""
    if return_future:
        async def _later():
            p2p = await dht.replicate_p2p()
            return _wrap_infos(await infos, p2p)

        return RemoteExpertWorker.run_coroutine(_later(), return_future=True)
    p2p = RemoteExpertWorker.run_coroutine(dht.replicate_p2p())
    return _wrap_infos(infos, p2p)


def batch_create_remote_experts(infos: Union[Sequence[Sequence[Optional[ExpertInfo]]], MPFuture], dht: DHT,
                                return_future: bool = False):
    if return_future:
        async def _later():
            p2p = await dht.replicate_p2p()
            return [_wrap_infos(row, p2p) for row in await infos]

        return RemoteExpertWorker.run_coroutine(_later(), return_future=True)
    p2p = RemoteExpertWorker.run_coroutine(dht.replicate_p2p())
    return [_wrap_infos(row, p2p) for row in infos]


def _payload_bytes(tensors: Sequence[torch.Tensor]) -> int:
    return sum(t.element_size() * t.nelement() for t in tensors)


async def _call_expert(uid: str, method: str, tensors: Sequence[torch.Tensor], compressions: Sequence[int], stub
                       ) -> List[torch.Tensor]:
    """One forward or backward exchange; unary if the raw payload fits into one message, streamed otherwise.
    Streamed tensors are written chunk by chunk from their own memory (no intermediate protobuf objects)."""
    if _payload_bytes(tensors) <= MAX_UNARY_PAYLOAD_SIZE:
        serialized = [serialize_torch_tensor(t, c) for t, c in zip(tensors, compressions)]
        reply = await getattr(stub, f"rpc_{method}")(runtime_pb2.ExpertRequest(uid=uid, tensors=serialized))
        return [deserialize_torch_tensor(t) for t in reply.tensors]

    async def _requests():
        uid_bytes = uid.encode()
        uid_field = b"\x0a" + _varint(len(uid_bytes)) + uid_bytes  # ExpertRequest.uid is field 1
        for tensor, compression in zip(tensors, compressions):
            for message in stream_tensor_messages(tensor, compression, DEFAULT_MAX_MSG_SIZE, outer_field=2,
                                                  outer_prefix=uid_field):
                yield message

    async def _reply_parts(stream):
        async for message in stream:
            yield message.tensors

    stream = await _maybe_await(getattr(stub, f"rpc_{method}_stream")(_requests()))
    return await deserialize_tensor_stream_into(_reply_parts(stream))


async def _maybe_await(value):
    return await value if hasattr(value, "__await__") else value


def _compressions(schema) -> List[int]:
    return [descr.compression for descr in nested_flatten(schema)]


async def expert_forward(uid: str, inputs: Sequence[torch.Tensor], compressions: Sequence[int], stub
                         ) -> List[torch.Tensor]:
    """Forward pass of a remote expert; ``compressions[i]`` is the wire codec of ``inputs[i]``."""
    return await _call_expert(uid, "forward", inputs, compressions, stub)


async def expert_backward(uid: str, inputs_and_grads: Sequence[torch.Tensor], compressions: Sequence[int], stub
                          ) -> List[torch.Tensor]:
    return await _call_expert(uid, "backward", inputs_and_grads, compressions, stub)


class _RemoteModuleCall(torch.autograd.Function):
    """Autograd bridge of one remote expert call; applications use ``RemoteExpert``."""

    @staticmethod
    def forward(ctx, dummy: torch.Tensor, uid: str, stub, info: Dict[str, Any], *inputs: torch.Tensor
                ) -> Tuple[torch.Tensor, ...]:
        inputs = tuple(t.detach().cpu() for t in inputs)
        ctx.uid, ctx.stub, ctx.info = uid, stub, info
        ctx.save_for_backward(*inputs)
        outputs = RemoteExpertWorker.run_coroutine(
            expert_forward(uid, inputs, _compressions(info["forward_schema"]), stub))
        return tuple(outputs)

    @staticmethod
    @once_differentiable
    def backward(ctx, *grad_outputs) -> Tuple[Optional[torch.Tensor], ...]:
        grads_cpu = tuple(g.cpu() for g in grad_outputs)
        payload = tuple(nested_flatten((ctx.saved_tensors, grads_cpu)))
        compressions = _compressions((ctx.info["forward_schema"], ctx.info["outputs_schema"]))
        grad_inputs = RemoteExpertWorker.run_coroutine(expert_backward(ctx.uid, payload, compressions, ctx.stub))
        return (DUMMY, None, None, None, *grad_inputs)

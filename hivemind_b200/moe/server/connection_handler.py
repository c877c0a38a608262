"""``ConnectionHandler``: the RPC face of an expert server.

Serves ``rpc_info``, ``rpc_forward`` / ``rpc_backward`` and their streamed variants for large tensors
(reference: hivemind/moe/server/connection_handler.py:22-177). The reference forks several handler processes that
share one daemon; here a handler is an event-loop thread with its own replica of the DHT's transport endpoint, and
several handlers register the same handle names with ``balanced=True`` so the daemon spreads calls across them.
Tensors are deserialised on the handler's loop, queued into the expert's ``TaskPool`` and the future awaited; the
``Runtime`` thread does the compute.
"""
from __future__ import annotations

from typing import AsyncIterator, Dict, List, Optional, Sequence

import torch

from hivemind_b200.compression import deserialize_torch_tensor, serialize_torch_tensor
from hivemind_b200.compression.serialization import deserialize_tensor_stream_into, stream_tensor_messages
from hivemind_b200.dht import DHT
from hivemind_b200.moe.server.module_backend import ModuleBackend
from hivemind_b200.moe.server.task_pool import TaskPool
from hivemind_b200.p2p import P2P, P2PContext, ServicerBase
from hivemind_b200.p2p.control import DEFAULT_MAX_MSG_SIZE
from hivemind_b200.proto import runtime_pb2
from hivemind_b200.utils import MPFuture, MSGPackSerializer, get_logger, nested_flatten
from hivemind_b200.utils.asyncio import LoopThread

logger = get_logger(__name__)


class ConnectionHandler(ServicerBase):
    """
    :param dht: a running DHT whose transport daemon carries the expert traffic
    :param module_backends: uid -> ModuleBackend for every expert served here
    :param balanced: register handlers so that the daemon load-balances between several ConnectionHandlers
    """

    def __init__(self, dht: DHT, module_backends: Dict[str, ModuleBackend], *, balanced: bool = True,
                 shutdown_timeout: float = 3, start: bool = False):
        self.dht, self.module_backends = dht, module_backends
        self.balanced, self.shutdown_timeout = balanced, shutdown_timeout
        self._p2p: Optional[P2P] = None
        self._pin_inputs = torch.cuda.is_available()  # streamed inputs land in page-locked memory for the H2D copy
        self._thread = LoopThread("ConnectionHandler")
        self.ready = MPFuture()
        if start:
            self.run_in_background(await_ready=True)

    def start(self) -> None:
        self._thread.start()

        async def _serve():
            try:
                self._p2p = await self.dht.replicate_p2p()
                await self.add_p2p_handlers(self._p2p, balanced=self.balanced)
                self.ready.set_result(None)
            except Exception as e:
                logger.error("ConnectionHandler failed to start:", exc_info=True)
                self.ready.set_exception(e)

        self._thread.submit(_serve())

    def run_in_background(self, await_ready: bool = True, timeout: Optional[float] = None) -> None:
        self.start()
        if await_ready:
            self.wait_until_ready(timeout)

    def wait_until_ready(self, timeout: Optional[float] = None) -> None:
        self.ready.result(timeout=timeout)

    def is_alive(self) -> bool:
        return self._thread.is_alive

    def join(self, timeout: Optional[float] = None) -> None:
        thread = self._thread._thread
        if thread is not None:
            thread.join(timeout)

    def shutdown(self) -> None:
        if not self._thread.is_alive:
            logger.debug("ConnectionHandler shutdown had no effect: it is not running")
            return

        async def _close():
            if self._p2p is not None:
                try:
                    await self.remove_p2p_handlers(self._p2p)
                except Exception as e:
                    logger.debug(f"Could not remove handlers: {e!r}")
                await self._p2p.shutdown()

        try:
            self._thread.run(_close(), timeout=self.shutdown_timeout)
        except Exception as e:
            logger.debug(f"ConnectionHandler did not close cleanly: {e!r}")
        self._thread.stop()

    # ------------------------------------------------------------------ RPC methods

    async def rpc_info(self, request: runtime_pb2.ExpertUID, context: P2PContext) -> runtime_pb2.ExpertInfo:
        module_info = self.module_backends[request.uid].get_info()
        return runtime_pb2.ExpertInfo(serialized_info=MSGPackSerializer.dumps(module_info))

    async def _run_pool(self, pool: TaskPool, tensors: Sequence[torch.Tensor], schema) -> List[runtime_pb2.Tensor]:
        outputs = await pool.submit_task(*tensors)
        return [serialize_torch_tensor(result, descr.compression, allow_inplace=True)
                for result, descr in zip(outputs, nested_flatten(schema))]

    async def _run_pool_streamed(self, pool: TaskPool, tensors: Sequence[torch.Tensor], schema):
        """Like ``_run_pool`` for large results: yields response messages chunk by chunk from the tensors' memory."""
        outputs = await pool.submit_task(*tensors)
        for result, descr in zip(outputs, nested_flatten(schema)):
            for message in stream_tensor_messages(result, descr.compression, DEFAULT_MAX_MSG_SIZE, outer_field=2):
                yield message

    async def _gather_stream(self, requests: AsyncIterator[runtime_pb2.ExpertRequest]):
        """Reassemble the tensors of a chunked request; every message must name the same expert."""
        uid: Optional[str] = None

        async def _tensor_parts():
            nonlocal uid
            async for message in requests:
                if uid is None:
                    uid = message.uid
                elif message.uid != uid:
                    raise ValueError("Expert uids differ in one request")
                yield message.tensors

        tensors = await deserialize_tensor_stream_into(_tensor_parts(), pin_memory=self._pin_inputs)
        return uid, tensors

    async def rpc_forward(self, request: runtime_pb2.ExpertRequest, context: P2PContext) -> runtime_pb2.ExpertResponse:
        backend = self.module_backends[request.uid]
        inputs = [deserialize_torch_tensor(tensor) for tensor in request.tensors]
        return runtime_pb2.ExpertResponse(tensors=await self._run_pool(backend.forward_pool, inputs, backend.outputs_schema))

    async def rpc_forward_stream(self, requests: AsyncIterator[runtime_pb2.ExpertRequest], context: P2PContext
                                 ) -> AsyncIterator[runtime_pb2.ExpertResponse]:
        uid, inputs = await self._gather_stream(requests)
        backend = self.module_backends[uid]
        async for message in self._run_pool_streamed(backend.forward_pool, inputs, backend.outputs_schema):
            yield message

    async def rpc_backward(self, request: runtime_pb2.ExpertRequest, context: P2PContext) -> runtime_pb2.ExpertResponse:
        backend = self.module_backends[request.uid]
        inputs_and_grads = [deserialize_torch_tensor(tensor) for tensor in request.tensors]
        return runtime_pb2.ExpertResponse(
            tensors=await self._run_pool(backend.backward_pool, inputs_and_grads, backend.grad_inputs_schema))

    async def rpc_backward_stream(self, requests: AsyncIterator[runtime_pb2.ExpertRequest], context: P2PContext
                                  ) -> AsyncIterator[runtime_pb2.ExpertResponse]:
        uid, inputs_and_grads = await self._gather_stream(requests)
        backend = self.module_backends[uid]
        async for message in self._run_pool_streamed(backend.backward_pool, inputs_and_grads, backend.grad_inputs_schema):
            yield message

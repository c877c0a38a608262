"""RPC services by reflection: subclass ``ServicerBase``, write ``async def rpc_*`` methods with type hints.

For every ``rpc_*(self, request: ProtoIn, context: P2PContext) -> ProtoOut`` (either side may be an
``AsyncIterator[...]``) the class gets a handler registration (``add_p2p_handlers``) and an auto-generated stub
(``get_stub``) whose method of the same name performs the call; unary-output calls accept ``timeout=``.
Handle names are ``[{namespace}::]{ClassName}.{method}`` (reference: hivemind/p2p/servicer.py:33-158).
"""
from __future__ import annotations

import asyncio
import inspect
from dataclasses import dataclass
from typing import Any, AsyncIterator, Optional, Tuple, get_type_hints

from hivemind_b200.p2p.datastructures import PeerID
from hivemind_b200.p2p.p2p_daemon import P2P


@dataclass
class RPCHandler:
    method_name: str
    request_type: type
    response_type: type
    stream_input: bool
    stream_output: bool


class StubBase:
    """Base of the generated stubs: holds the endpoint, the target peer and the namespace."""

    def __init__(self, p2p: P2P, peer: PeerID, namespace: Optional[str]):
        self._p2p = p2p
        self._peer = peer
        self._namespace = namespace


def _split_iterator_hint(hint: Any) -> Tuple[type, bool]:
    origin = getattr(hint, "__origin__", None)
    if origin is not None and origin in (AsyncIterator, getattr(__import__("collections.abc").abc, "AsyncIterator")):
        return hint.__args__[0], True
    return hint, False


class ServicerBase:
    _rpc_handlers = None
    _stub_type = None

    @classmethod
    def _collect_rpc_handlers(cls) -> None:
        if cls._rpc_handlers is not None and cls.__dict__.get("_rpc_handlers") is not None:
            return
        handlers = []
        for method_name, method in inspect.getmembers(cls, predicate=inspect.isfunction):
            if not method_name.startswith("rpc_"):
                continue
            spec = inspect.getfullargspec(method)
            if len(spec.args) < 3:
                raise ValueError(f"{method_name} is expected to take (self, request, context)")
            hints = get_type_hints(method)
            try:
                request_type, stream_input = _split_iterator_hint(hints[spec.args[1]])
                response_type, stream_output = _split_iterator_hint(hints["return"])
            except KeyError:
                raise ValueError(f"{method_name} needs type hints for its request and its return value") from None
            handlers.append(RPCHandler(method_name, request_type, response_type, stream_input, stream_output))
        cls._rpc_handlers = handlers
        cls._stub_type = type(f"{cls.__name__}Stub", (StubBase,), {h.method_name: cls._make_rpc_caller(h) for h in handlers})

    @classmethod
    def _make_rpc_caller(cls, handler: RPCHandler):
        input_type = AsyncIterator[handler.request_type] if handler.stream_input else handler.request_type
        output_type = AsyncIterator[handler.response_type] if handler.stream_output else handler.response_type

        if handler.stream_output:
            def caller(self: StubBase, input: input_type, timeout: None = None) -> output_type:
                if timeout is not None:
                    raise ValueError("timeouts are not supported for calls with a streamed output")
                return self._p2p.iterate_protobuf_handler(self._peer, cls._get_handle_name(self._namespace, handler.method_name),
                                                          input, handler.response_type)
        else:
            async def caller(self: StubBase, input: input_type, timeout: Optional[float] = None) -> output_type:
                return await asyncio.wait_for(
                    self._p2p.call_protobuf_handler(self._peer, cls._get_handle_name(self._namespace, handler.method_name),
                                                    input, handler.response_type),
                    timeout=timeout)

        caller.__name__ = handler.method_name
        return caller

    async def add_p2p_handlers(self, p2p: P2P, wrapper: Any = None, *, namespace: Optional[str] = None,
                               balanced: bool = False) -> None:
        """Register every ``rpc_*`` method on ``p2p``; ``wrapper`` (e.g. an auth wrapper) intercepts the calls."""
        self._collect_rpc_handlers()
        servicer = self if wrapper is None else wrapper
        await asyncio.gather(*[
            p2p.add_protobuf_handler(self._get_handle_name(namespace, h.method_name), getattr(servicer, h.method_name),
                                     h.request_type, stream_input=h.stream_input, stream_output=h.stream_output,
                                     balanced=balanced)
            for h in self._rpc_handlers])

    async def remove_p2p_handlers(self, p2p: P2P, *, namespace: Optional[str] = None) -> None:
        self._collect_rpc_handlers()
        await asyncio.gather(*[
            p2p.remove_protobuf_handler(self._get_handle_name(namespace, h.method_name), stream_input=h.stream_input,
                                        stream_output=h.stream_output)
            for h in self._rpc_handlers])

    @classmethod
    def get_stub(cls, p2p: P2P, peer: PeerID, *, namespace: Optional[str] = None) -> StubBase:
        cls._collect_rpc_handlers()
        return cls._stub_type(p2p, peer, namespace)

    @classmethod
    def _get_handle_name(cls, namespace: Optional[str], method_name: str) -> str:
        handle_name = f"{cls.__name__}.{method_name}"
        if namespace is not None:
            handle_name = f"{namespace}::{handle_name}"
        return handle_name

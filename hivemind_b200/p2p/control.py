"""Client side of the hmp2pd control protocol (asyncio).

Plays the role of the reference's ``ControlClient`` (hivemind/p2p/p2p_daemon_bindings/control.py:89-427): one-shot
commands on short-lived connections to the daemon's control socket, a persistent multiplexed connection for unary
calls keyed by a 16-byte call id (with cancel propagation), and a unix listener that receives inbound streams.
Frames are ``u32 big-endian length, u8 type, body`` (see ``native/hmp2pd.cpp``).
"""
from __future__ import annotations

import asyncio
import os
import struct
from typing import Awaitable, Callable, Dict, Optional, Sequence, Tuple

from hivemind_b200.p2p.chunked_reader import open_unix_stream, start_unix_stream_server
from hivemind_b200.p2p.datastructures import PeerID, PeerInfo, StreamInfo
from hivemind_b200.utils.logging import get_logger
from hivemind_b200.utils.multiaddr import Multiaddr

logger = get_logger(__name__)

DEFAULT_MAX_MSG_SIZE = 4 * 1024 ** 2
MAX_UNARY_PAYLOAD_SIZE = DEFAULT_MAX_MSG_SIZE // 2

(C_IDENTIFY, C_CONNECT, C_LIST_PEERS, C_DISCONNECT, C_PERSISTENT, C_STREAM_OPEN, C_STREAM_HANDLER,
 C_REMOVE_STREAM_HANDLER) = range(1, 9)
R_OK, R_ERR = 20, 21
P_ADD_UNARY_HANDLER, P_REMOVE_UNARY_HANDLER, P_CALL_UNARY, P_UNARY_RESPONSE, P_CANCEL, P_REQUEST, P_RESPONSE, P_ACK = range(30, 38)
S_INFO = 62

StreamHandler = Callable[[StreamInfo, asyncio.StreamReader, asyncio.StreamWriter], Awaitable[None]]
UnaryHandler = Callable[[bytes, PeerID], Awaitable[bytes]]


class P2PDaemonError(Exception):
    """The daemon refused or failed a control request."""


class P2PHandlerError(Exception):
    """The remote handler raised an error (or the protocol is not served there)."""


class DispatchFailure(Exception):
    pass


class _Writer:
    def __init__(self, msg_type: int):
        self.parts = [bytes([msg_type])]

    def u8(self, v: int) -> "_Writer":
        self.parts.append(bytes([v]))
        return self

    def u32(self, v: int) -> "_Writer":
        self.parts.append(struct.pack(">I", v))
        return self

    def blob(self, b: bytes) -> "_Writer":
        self.parts.append(struct.pack(">I", len(b)))
        self.parts.append(b)
        return self

    def finish(self) -> bytes:
        body = b"".join(self.parts)
        return struct.pack(">I", len(body)) + body


class _Reader:
    def __init__(self, buf: bytes):
        self.buf, self.pos = buf, 0

    def u8(self) -> int:
        v = self.buf[self.pos]
        self.pos += 1
        return v

    def u32(self) -> int:
        (v,) = struct.unpack_from(">I", self.buf, self.pos)
        self.pos += 4
        return v

    def blob(self) -> bytes:
        n = self.u32()
        v = self.buf[self.pos:self.pos + n]
        if len(v) != n:
            raise P2PDaemonError("truncated frame from the daemon")
        self.pos += n
        return v


async def read_frame(reader: asyncio.StreamReader) -> Tuple[int, _Reader]:
    header = await reader.readexactly(4)
    (length,) = struct.unpack(">I", header)
    body = await reader.readexactly(length)
    return body[0], _Reader(body[1:])


def _peer_bytes(peer_id: PeerID) -> bytes:
    return peer_id.to_base58().encode("ascii")


def _new_call_id() -> bytes:
    """16 random bytes: call ids of different peers meet in one table inside the callee's daemon."""
    return os.urandom(16)


class DaemonClient:
    """One client of a running hmp2pd. Several clients (one per process or component) may share a daemon."""

    def __init__(self, control_path: str, listen_path: str, *, persistent_conn_max_msg_size: int = DEFAULT_MAX_MSG_SIZE):
        self.control_path = control_path
        self.listen_path = listen_path
        self.persistent_conn_max_msg_size = persistent_conn_max_msg_size
        self.stream_handlers: Dict[str, StreamHandler] = {}
        self.unary_handlers: Dict[str, UnaryHandler] = {}
        self._listener: Optional[asyncio.AbstractServer] = None
        self._pers_reader: Optional[asyncio.StreamReader] = None
        self._pers_writer: Optional[asyncio.StreamWriter] = None
        self._pers_task: Optional[asyncio.Task] = None
        self._pending: Dict[bytes, asyncio.Future] = {}
        self._caller_ids: Dict[bytes, PeerID] = {}
        self._serving: Dict[bytes, asyncio.Task] = {}
        self._write_lock = asyncio.Lock()
        self._closed = False

    # ------------------------------------------------------------------------------------------ lifecycle
    @classmethod
    async def create(cls, control_path: str, listen_path: str, **kwargs) -> "DaemonClient":
        self = cls(control_path, listen_path, **kwargs)
        if os.path.exists(listen_path):
            os.unlink(listen_path)
        self._listener = await start_unix_stream_server(self._on_inbound_stream, listen_path)
        await self._open_persistent()
        return self

    async def close(self) -> None:
        self._closed = True
        if self._pers_task is not None:
            self._pers_task.cancel()
        for task in list(self._serving.values()):
            task.cancel()
        if self._pers_writer is not None:
            self._pers_writer.close()
        if self._listener is not None:
            self._listener.close()
        for fut in self._pending.values():
            if not fut.done():
                fut.set_exception(P2PDaemonError("daemon client closed"))
        self._pending.clear()
        try:
            os.unlink(self.listen_path)
        except OSError:
            pass

    async def _command(self, frame: bytes) -> Tuple[asyncio.StreamReader, asyncio.StreamWriter, _Reader]:
        reader, writer = await open_unix_stream(self.control_path, limit=2 ** 20)
        try:
            writer.write(frame)
            await writer.drain()
            msg_type, body = await read_frame(reader)
        except BaseException:
            writer.close()
            raise
        if msg_type == R_ERR:
            writer.close()
            raise P2PDaemonError(body.blob().decode("utf-8", "replace"))
        if msg_type != R_OK:
            writer.close()
            raise P2PDaemonError(f"unexpected reply type {msg_type}")
        return reader, writer, body

    async def _simple(self, frame: bytes) -> _Reader:
        _, writer, body = await self._command(frame)
        writer.close()
        return body

    # ------------------------------------------------------------------------------------------ one-shot commands
    async def identify(self) -> Tuple[PeerID, Tuple[Multiaddr, ...]]:
        body = await self._simple(_Writer(C_IDENTIFY).finish())
        peer_id = PeerID.from_base58(body.blob().decode("ascii"))
        addrs = tuple(Multiaddr(body.blob().decode("utf-8")) for _ in range(body.u32()))
        return peer_id, addrs

    async def connect(self, peer_id: PeerID, maddrs: Sequence[Multiaddr]) -> None:
        w = _Writer(C_CONNECT).blob(_peer_bytes(peer_id)).u32(len(maddrs))
        for m in maddrs:
            w.blob(str(Multiaddr(m).decapsulate_code(0x01A5)).encode("utf-8"))
        await self._simple(w.finish())

    async def list_peers(self) -> Tuple[PeerInfo, ...]:
        body = await self._simple(_Writer(C_LIST_PEERS).finish())
        out = []
        for _ in range(body.u32()):
            pid, addr = body.blob(), body.blob()
            out.append(PeerInfo(PeerID.from_base58(pid.decode("ascii")), [Multiaddr(addr.decode())] if addr else []))
        return tuple(out)

    async def disconnect(self, peer_id: PeerID) -> None:
        await self._simple(_Writer(C_DISCONNECT).blob(_peer_bytes(peer_id)).finish())

    # ------------------------------------------------------------------------------------------ streams
    async def stream_open(self, peer_id: PeerID, protocols: Sequence[str]
                          ) -> Tuple[StreamInfo, asyncio.StreamReader, asyncio.StreamWriter]:
        w = _Writer(C_STREAM_OPEN).blob(_peer_bytes(peer_id)).u32(len(protocols))
        for p in protocols:
            w.blob(p.encode("utf-8"))
        reader, writer, body = await self._command(w.finish())
        proto = body.blob().decode("utf-8")
        return StreamInfo(peer_id, Multiaddr(), proto), reader, writer

    async def stream_handler(self, proto: str, handler: StreamHandler, balanced: bool = False) -> None:
        w = _Writer(C_STREAM_HANDLER).blob(self.listen_path.encode()).u8(int(balanced)).u32(1).blob(proto.encode("utf-8"))
        await self._simple(w.finish())
        self.stream_handlers[proto] = handler

    async def remove_stream_handler(self, proto: str) -> None:
        w = _Writer(C_REMOVE_STREAM_HANDLER).blob(self.listen_path.encode()).u32(1).blob(proto.encode("utf-8"))
        await self._simple(w.finish())
        self.stream_handlers.pop(proto, None)

    async def _on_inbound_stream(self, reader: asyncio.StreamReader, writer: asyncio.StreamWriter) -> None:
        try:
            msg_type, body = await read_frame(reader)
            if msg_type != S_INFO:
                raise DispatchFailure(f"expected stream info, got frame type {msg_type}")
            peer, addr, proto = body.blob(), body.blob(), body.blob().decode("utf-8")
            info = StreamInfo(PeerID.from_base58(peer.decode("ascii")), Multiaddr(addr.decode()) if addr else Multiaddr(), proto)
            handler = self.stream_handlers.get(proto)
            if handler is None:
                raise DispatchFailure(f"no handler for protocol {proto}")
            await handler(info, reader, writer)
        except (asyncio.IncompleteReadError, ConnectionError):
            pass
        except asyncio.CancelledError:
            raise
        except Exception as e:
            logger.debug(f"inbound stream failed: {e!r}")
        finally:
            try:
                writer.close()
            except Exception:
                pass

    # ------------------------------------------------------------------------------------------ unary calls
    async def _open_persistent(self) -> None:
        reader, writer, _ = await self._command(_Writer(C_PERSISTENT).finish())
        self._pers_reader, self._pers_writer = reader, writer
        self._pers_task = asyncio.create_task(self._read_persistent())

    async def _send_persistent(self, frame: bytes) -> None:
        async with self._write_lock:
            self._pers_writer.write(frame)
            await self._pers_writer.drain()

    async def _read_persistent(self) -> None:
        try:
            while True:
                msg_type, body = await read_frame(self._pers_reader)
                if msg_type in (P_RESPONSE, P_ACK):
                    call_id, is_err, data = body.blob(), body.u8(), body.blob()
                    fut = self._pending.pop(call_id, None)
                    if fut is not None and not fut.done():
                        if is_err:
                            fut.set_exception(P2PHandlerError(data.decode("utf-8", "replace")) if msg_type == P_RESPONSE
                                              else P2PDaemonError(data.decode("utf-8", "replace")))
                        else:
                            fut.set_result(data)
                elif msg_type == P_REQUEST:
                    call_id, peer, proto, data = body.blob(), body.blob(), body.blob().decode("utf-8"), body.blob()
                    task = asyncio.create_task(self._serve_unary(call_id, self._caller_id(peer), proto, data))
                    self._serving[call_id] = task
                    task.add_done_callback(lambda _t, cid=call_id: self._serving.pop(cid, None))
                elif msg_type == P_CANCEL:
                    task = self._serving.get(body.blob())
                    if task is not None:
                        task.cancel()
        except (asyncio.IncompleteReadError, ConnectionError):
            if not self._closed:
                logger.debug("persistent connection to the daemon was closed")
        except asyncio.CancelledError:
            pass
        finally:
            for fut in self._pending.values():
                if not fut.done():
                    fut.set_exception(P2PDaemonError("the connection to the daemon was lost"))
            self._pending.clear()

    async def _serve_unary(self, call_id: bytes, peer_id: PeerID, proto: str, data: bytes) -> None:
        handler = self.unary_handlers.get(proto)
        try:
            if handler is None:
                raise P2PHandlerError(f"protocol not supported: {proto}")
            result = await handler(data, peer_id)
            frame = _Writer(P_UNARY_RESPONSE).blob(call_id).u8(0).blob(result).finish()
        except asyncio.CancelledError:
            return
        except Exception as e:
            frame = _Writer(P_UNARY_RESPONSE).blob(call_id).u8(1).blob(repr(e).encode("utf-8")).finish()
        try:
            await self._send_persistent(frame)
        except Exception:
            pass

    def _caller_id(self, text: bytes) -> PeerID:
        """The ``PeerID`` for the base58 text that the daemon puts in front of an incoming call; the same few callers
        come back thousands of times, so the decoded ids are kept."""
        known = self._caller_ids.get(text)
        if known is None:
            if len(self._caller_ids) >= 4096:
                self._caller_ids.clear()
            known = self._caller_ids[text] = PeerID.from_base58(text.decode("ascii"))
        return known

    async def _request(self, frame: bytes, call_id: bytes) -> bytes:
        fut = asyncio.get_event_loop().create_future()
        self._pending[call_id] = fut
        await self._send_persistent(frame)
        return await fut

    async def add_unary_handler(self, proto: str, handler: UnaryHandler, balanced: bool = False) -> None:
        call_id = _new_call_id()
        await self._request(_Writer(P_ADD_UNARY_HANDLER).blob(call_id).blob(proto.encode()).u8(int(balanced)).finish(), call_id)
        self.unary_handlers[proto] = handler

    async def remove_unary_handler(self, proto: str) -> None:
        call_id = _new_call_id()
        await self._request(_Writer(P_REMOVE_UNARY_HANDLER).blob(call_id).blob(proto.encode()).finish(), call_id)
        self.unary_handlers.pop(proto, None)

    async def call_unary_handler(self, peer_id: PeerID, proto: str, data: bytes) -> bytes:
        call_id = _new_call_id()
        frame = _Writer(P_CALL_UNARY).blob(call_id).blob(_peer_bytes(peer_id)).blob(proto.encode()).blob(data).finish()
        try:
            return await self._request(frame, call_id)
        except asyncio.CancelledError:
            self._pending.pop(call_id, None)
            try:
                await asyncio.shield(self._send_persistent(_Writer(P_CANCEL).blob(call_id).finish()))
            except Exception:
                pass
            raise

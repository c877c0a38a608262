"""``P2P``: the peer-to-peer endpoint of one process, backed by the C++ ``hmp2pd`` transport daemon.

Interface parity with the reference's wrapper around the Go daemon (hivemind/p2p/p2p_daemon.py:42-749):
``create`` spawns a daemon and connects to it, ``replicate`` attaches to a running one, protobuf handlers are unary
(multiplexed over the daemon's persistent connection) or streaming (one spliced byte stream per call), and raw
binary stream handlers are available too. Streamed protobufs are framed as a 1-byte marker (message / error),
an 8-byte big-endian length and the payload (reference :58-62,367-407).

Differences by design: the daemon is a small epoll program (``native/hmp2pd.cpp``) rather than libp2p; it does not
encrypt, traverse NATs, relay or speak QUIC — options for those are accepted and ignored with a debug message.
"""
from __future__ import annotations

import asyncio
import os
import secrets
import subprocess
import tempfile
import threading
import time
from contextlib import closing, suppress
from dataclasses import dataclass
from typing import AsyncIterator, Awaitable, Callable, List, Optional, Sequence, Tuple, Type, TypeVar, Union

from cryptography.hazmat.primitives import serialization
from cryptography.hazmat.primitives.asymmetric import rsa
from google.protobuf.message import Message

from hivemind_b200.ops import _build
from hivemind_b200.p2p.control import DEFAULT_MAX_MSG_SIZE, DaemonClient, P2PDaemonError, P2PHandlerError
from hivemind_b200.p2p.datastructures import PeerID, PeerInfo, StreamInfo
from hivemind_b200.proto import crypto_pb2
from hivemind_b200.utils.asyncio import as_aiter, asingle
from hivemind_b200.utils.logging import get_logger
from hivemind_b200.utils.multiaddr import Multiaddr

logger = get_logger(__name__)
TInputProtobuf = TypeVar("TInputProtobuf")
TOutputProtobuf = TypeVar("TOutputProtobuf")


@dataclass(frozen=True)
class P2PContext:
    handle_name: str
    local_id: PeerID
    remote_id: PeerID = None


class RPCError(Exception):
    """Error record sent over a protobuf stream in place of a message."""

    def __init__(self, message: str = ""):
        super().__init__(message)
        self.message = message

    def SerializeToString(self) -> bytes:
        return self.message.encode("utf-8")


class P2P:
    HEADER_LEN = 8
    BYTEORDER = "big"
    MESSAGE_MARKER = b"\x00"
    ERROR_MARKER = b"\x01"
    END_OF_STREAM = RPCError()

    _UNSUPPORTED_OPTIONS = ("announce_maddrs", "auto_nat", "conn_manager", "dht_mode", "force_reachability", "idle_timeout",
                            "nat_port_map", "relay_hop_limit", "tls", "use_auto_relay", "use_ipfs", "use_relay", "quic",
                            "use_relay_hop", "use_relay_discovery", "trusted_relays")

    def __init__(self):
        self.peer_id: Optional[PeerID] = None
        self._client: Optional[DaemonClient] = None
        self._child: Optional[subprocess.Popen] = None
        self._alive = False
        self._control_path: Optional[str] = None
        self._visible_maddrs: Optional[List[Multiaddr]] = None
        self._reader_thread: Optional[threading.Thread] = None
        self._workdir: Optional[str] = None

    # ------------------------------------------------------------------------------------------ construction
    @classmethod
    async def create(cls, initial_peers: Optional[Sequence[Union[Multiaddr, str]]] = None, *,
                     host_maddrs: Optional[Sequence[Union[Multiaddr, str]]] = ("/ip4/127.0.0.1/tcp/0",),
                     identity_path: Optional[str] = None, startup_timeout: float = 15,
                     persistent_conn_max_msg_size: int = DEFAULT_MAX_MSG_SIZE, check_if_identity_free: bool = True,
                     no_listen: bool = False, **options) -> "P2P":
        """Start a new transport daemon and connect to it.

        :param initial_peers: multiaddrs (with ``/p2p/<id>``) of peers to connect to at start
        :param host_maddrs: addresses to listen on (``/ip4/<ip>/tcp/<port>`` or ``/unix/<path>``)
        :param identity_path: private key file; makes the peer id deterministic (created if missing)
        :param no_listen: do not accept connections from other peers (client mode)
        """
        for name in options:
            if name not in cls._UNSUPPORTED_OPTIONS:
                raise TypeError(f"P2P.create() got an unexpected keyword argument {name!r}")
        ignored = [k for k, v in options.items() if v not in (None, False, 0) and k not in ("idle_timeout", "tls", "dht_mode",
                   "auto_nat", "conn_manager", "nat_port_map", "use_relay")]
        if ignored:
            logger.debug(f"options without effect on a single-box transport: {ignored}")

        self = cls()
        private_key = cls._load_or_make_identity(identity_path)
        self.peer_id = PeerID.from_private_key(private_key)
        if identity_path is not None and check_if_identity_free and initial_peers:
            if await cls.is_identity_taken(self.peer_id, initial_peers):
                raise P2PDaemonError(f"identity {identity_path} is already in use by a peer on the network")

        self._workdir = tempfile.mkdtemp(prefix="hivemind-b200-")
        self._control_path = os.path.join(self._workdir, "ctl.sock")
        args = [str(_build.build_daemon()), "--control", self._control_path, "--peer-id", self.peer_id.to_base58()]
        tcp_set = False
        for maddr in ([] if no_listen else (host_maddrs or [])):
            maddr = Multiaddr(maddr)
            if "unix" in maddr:
                args += ["--peer-unix", maddr["unix"]]
            elif "ip4" in maddr and "tcp" in maddr and not tcp_set:
                args += ["--host", maddr["ip4"], "--port", maddr["tcp"]]
                tcp_set = True
            else:
                logger.debug(f"listen address {maddr} is not supported by the transport daemon; skipped")
        if not tcp_set:
            args.append("--no-tcp")
        # same switch as for the reference's Go daemon (hivemind/p2p/p2p_daemon.py:222): the daemon's own log
        if os.environ.get("GOLOG_LOG_LEVEL", "").strip().lower() == "debug":
            args.append("--verbose")
        spawned = time.monotonic()
        self._child = subprocess.Popen(args, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, bufsize=1)
        self._alive = True
        ready = asyncio.get_event_loop().create_future()
        loop = asyncio.get_event_loop()
        # the thread gets the child process, not this object: a bound method would keep the instance alive, and with it
        # the daemon that __del__ is there to stop
        self._reader_thread = threading.Thread(target=self._read_outputs, args=(self._child, loop, ready), daemon=True)
        self._reader_thread.start()
        try:
            await asyncio.wait_for(ready, startup_timeout)
            # the limit is on the daemon, not on how promptly this loop gets to look: a daemon that needed longer has
            # failed even if it is up by the time a busy loop checks
            if time.monotonic() - spawned > startup_timeout:
                raise asyncio.TimeoutError
        except asyncio.TimeoutError:
            await self.shutdown()
            raise P2PDaemonError(f"Daemon failed to start in {startup_timeout:.1f} seconds")
        self._client = await DaemonClient.create(self._control_path, os.path.join(self._workdir, f"h-{secrets.token_hex(4)}.sock"),
                                                 persistent_conn_max_msg_size=persistent_conn_max_msg_size)
        await self._ping_daemon()
        connected, problems = 0, []
        for peer in initial_peers or []:
            peer = Multiaddr(peer)
            try:
                remote = PeerID.from_base58(peer["p2p"])
                await self._client.connect(remote, [peer])
                if not await self._answers(remote):  # the daemon only notes the address; see whether anybody is there
                    raise P2PDaemonError("no answer")
                connected += 1
            except Exception as e:
                problems.append(f"{peer}: {e!r}")
                logger.warning(f"could not connect to initial peer {peer}: {e!r}")
        if initial_peers and connected == 0:
            # like the reference's daemon, which refuses to start when no bootstrap peer answers
            await self.shutdown()
            raise P2PDaemonError("failed to connect to bootstrap peers: " + "; ".join(problems))
        return self

    @staticmethod
    def _load_or_make_identity(identity_path: Optional[str]):
        if identity_path is not None and os.path.exists(identity_path):
            with open(identity_path, "rb") as f:
                data = crypto_pb2.PrivateKey.FromString(f.read()).data
            return serialization.load_der_private_key(data, password=None)
        key = rsa.generate_private_key(public_exponent=65537, key_size=2048)
        if identity_path is not None:
            P2P._write_identity(identity_path, key)
        return key

    @staticmethod
    def _write_identity(identity_path: str, key) -> None:
        der = key.private_bytes(encoding=serialization.Encoding.DER, format=serialization.PrivateFormat.TraditionalOpenSSL,
                                encryption_algorithm=serialization.NoEncryption())
        blob = crypto_pb2.PrivateKey(key_type=crypto_pb2.RSA, data=der).SerializeToString()
        fd = os.open(identity_path, os.O_WRONLY | os.O_CREAT | os.O_TRUNC, 0o400)
        with os.fdopen(fd, "wb") as f:
            f.write(blob)

    @staticmethod
    def generate_identity(identity_path: str) -> None:
        """Write a fresh RSA identity (protobuf ``crypto.pb.PrivateKey``) to ``identity_path``."""
        P2P._write_identity(identity_path, rsa.generate_private_key(public_exponent=65537, key_size=2048))

    async def _answers(self, peer_id: PeerID, timeout: float = 3.5) -> bool:
        """True if a daemon with this id answers a call to a handler that nobody registers ("not supported" is an
        answer; an unknown address, a refused connection or silence is not)."""
        try:
            await asyncio.wait_for(self._client.call_unary_handler(peer_id, "__identity_probe__", b""), timeout)
        except P2PHandlerError as e:
            text = str(e).lower()
            return not any(word in text for word in ("address unknown", "connect", "unreachable", "refused"))
        except (P2PDaemonError, asyncio.TimeoutError):
            return False
        return True

    @classmethod
    async def is_identity_taken(cls, peer_id: PeerID, initial_peers: Sequence[Union[Multiaddr, str]]) -> bool:
        """True if a peer with this id answers on the network reachable through ``initial_peers``."""
        probe = await cls.create(initial_peers, check_if_identity_free=False, no_listen=True)
        try:
            if any(info.peer_id == peer_id for info in await probe.list_peers()):
                return True
            return await probe._answers(peer_id)
        finally:
            await probe.shutdown()

    @classmethod
    async def replicate(cls, daemon_listen_maddr: Multiaddr) -> "P2P":
        """Attach another client (e.g. a second component or process) to a running daemon."""
        self = cls()
        self._control_path = Multiaddr(daemon_listen_maddr)["unix"]
        self._workdir = os.path.dirname(self._control_path)
        self._client = await DaemonClient.create(self._control_path, os.path.join(self._workdir, f"h-{secrets.token_hex(4)}.sock"))
        self._alive = True
        await self._ping_daemon()
        return self

    async def _ping_daemon(self) -> None:
        self.peer_id, maddrs = await self._client.identify()
        self._visible_maddrs = [m.encapsulate(f"/p2p/{self.peer_id.to_base58()}") for m in maddrs]
        logger.debug(f"launched transport daemon with peer id {self.peer_id} and host maddrs {maddrs}")

    # ------------------------------------------------------------------------------------------ info
    async def get_visible_maddrs(self, latest: bool = False) -> List[Multiaddr]:
        if latest or self._visible_maddrs is None:
            await self._ping_daemon()
        if not self._visible_maddrs:
            raise ValueError(f"no multiaddrs found for peer {self.peer_id}")
        return list(self._visible_maddrs)

    async def list_peers(self) -> List[PeerInfo]:
        return list(await self._client.list_peers())

    async def wait_for_at_least_n_peers(self, n_peers: int, attempts: int = 3, delay: float = 1) -> None:
        for _ in range(attempts):
            if len(await self._client.list_peers()) >= n_peers:
                return
            await asyncio.sleep(delay)
        raise RuntimeError("Not enough peers")

    @property
    def daemon_listen_maddr(self) -> Multiaddr:
        return Multiaddr(f"/unix{self._control_path}")

    # ------------------------------------------------------------------------------------------ framing
    @staticmethod
    async def send_raw_data(data: bytes, writer: asyncio.StreamWriter, *, chunk_size: int = 2 ** 20) -> None:
        writer.write(len(data).to_bytes(P2P.HEADER_LEN, P2P.BYTEORDER))
        view = memoryview(data)
        for offset in range(0, len(data), chunk_size):
            writer.write(view[offset:offset + chunk_size])
        await writer.drain()

    @staticmethod
    async def receive_raw_data(reader: asyncio.StreamReader) -> bytes:
        header = await reader.readexactly(P2P.HEADER_LEN)
        return await reader.readexactly(int.from_bytes(header, P2P.BYTEORDER))

    @staticmethod
    async def send_protobuf(protobuf: Union[Message, RPCError], writer: asyncio.StreamWriter) -> None:
        writer.write(P2P.ERROR_MARKER if isinstance(protobuf, RPCError) else P2P.MESSAGE_MARKER)
        pieces = getattr(protobuf, "raw_parts", None)
        if pieces is None:
            await P2P.send_raw_data(protobuf.SerializeToString(), writer)
            return
        # a message that is already serialized as several byte pieces (large tensor chunks): no joining, no copies
        writer.write(sum(len(piece) for piece in pieces).to_bytes(P2P.HEADER_LEN, P2P.BYTEORDER))
        for piece in pieces:
            writer.write(piece)
        await writer.drain()

    @staticmethod
    async def receive_protobuf(input_protobuf_type: Type[Message], reader: asyncio.StreamReader
                               ) -> Tuple[Optional[Message], Optional[RPCError]]:
        marker = await reader.readexactly(1)
        payload = await P2P.receive_raw_data(reader)
        if marker == P2P.MESSAGE_MARKER:
            return input_protobuf_type.FromString(payload), None
        if marker == P2P.ERROR_MARKER:
            return None, RPCError(payload.decode("utf-8", "replace"))
        raise TypeError("invalid protobuf marker on the stream")

    # ------------------------------------------------------------------------------------------ handlers
    async def add_protobuf_handler(self, name: str, handler: Callable, input_protobuf_type: Type[Message], *,
                                   stream_input: bool = False, stream_output: bool = False, balanced: bool = False) -> None:
        """Register ``handler(request_or_stream, context)`` under ``name``.

        Unary handlers (no streaming on either side) are multiplexed over the persistent connection; a handler
        with a streamed input or output gets one byte stream per call.
        """
        if not stream_input and not stream_output:
            await self._add_protobuf_unary_handler(name, handler, input_protobuf_type, balanced=balanced)
            return

        async def _stream_handler(requests: AsyncIterator[Message], context: P2PContext) -> AsyncIterator[Message]:
            arg = requests if stream_input else await asingle(requests)
            if stream_output:
                async for item in handler(arg, context):
                    yield item
            else:
                yield await handler(arg, context)

        await self._add_protobuf_stream_handler(name, _stream_handler, input_protobuf_type, balanced=balanced)

    async def remove_protobuf_handler(self, name: str, *, stream_input: bool = False, stream_output: bool = False) -> None:
        if not stream_input and not stream_output:
            await self._client.remove_unary_handler(name)
        else:
            await self._client.remove_stream_handler(name)

    async def _add_protobuf_unary_handler(self, name: str, handler: Callable, input_protobuf_type: Type[Message], *,
                                          balanced: bool = False) -> None:
        async def _unary_handler(request: bytes, remote_id: PeerID) -> bytes:
            parsed = input_protobuf_type.FromString(request)
            context = P2PContext(handle_name=name, local_id=self.peer_id, remote_id=remote_id)
            response = await handler(parsed, context)
            return response.SerializeToString()

        await self._client.add_unary_handler(name, _unary_handler, balanced=balanced)

    async def _add_protobuf_stream_handler(self, name: str, handler: Callable, input_protobuf_type: Type[Message], *,
                                           max_prefetch: int = 5, balanced: bool = False) -> None:
        """``handler(requests: AsyncIterator, context) -> AsyncIterator``; closing the stream cancels the handler."""

        async def _handle_stream(stream_info: StreamInfo, reader: asyncio.StreamReader, writer: asyncio.StreamWriter) -> None:
            context = P2PContext(handle_name=name, local_id=self.peer_id, remote_id=stream_info.peer_id)
            requests: asyncio.Queue = asyncio.Queue(max_prefetch)

            async def _read_stream() -> AsyncIterator[Message]:
                while True:
                    request = await requests.get()
                    if request is None:
                        break
                    yield request

            async def _process_stream() -> None:
                responses = handler(_read_stream(), context)
                try:
                    async for response in responses:
                        try:
                            await P2P.send_protobuf(response, writer)
                        except Exception:
                            logger.debug("could not send a response: the stream is closed", exc_info=True)
                            break
                except Exception as e:
                    logger.warning(f"handler {name} failed:", exc_info=True)
                    with suppress(Exception):
                        await P2P.send_protobuf(RPCError(str(e) or repr(e)), writer)
                finally:
                    # a caller that walked away must not leave the handler's generator suspended until it is
                    # garbage-collected: close it now, so that its ``finally`` blocks run
                    close = getattr(responses, "aclose", None)
                    if close is not None:
                        with suppress(Exception):
                            await close()

            with closing(writer):
                processing_task = asyncio.create_task(_process_stream())
                try:
                    while True:
                        receive_task = asyncio.create_task(P2P.receive_protobuf(input_protobuf_type, reader))
                        await asyncio.wait({processing_task, receive_task}, return_when=asyncio.FIRST_COMPLETED)
                        if processing_task.done():
                            receive_task.cancel()
                            return
                        if receive_task.done():
                            try:
                                request, _ = await receive_task
                            except asyncio.IncompleteReadError:  # the caller finished (or dropped) its side
                                await requests.put(None)
                                await processing_task
                                return
                            await requests.put(request)
                except Exception:
                    logger.debug("exception while receiving requests:", exc_info=True)
                finally:
                    processing_task.cancel()

        await self._client.stream_handler(name, _handle_stream, balanced)

    async def _iterate_protobuf_stream_handler(self, peer_id: PeerID, name: str, requests: AsyncIterator[Message],
                                               output_protobuf_type: Type[Message]) -> AsyncIterator[Message]:
        _, reader, writer = await self.call_binary_stream_handler(peer_id, name)

        async def _write_to_stream() -> None:
            async for request in requests:
                await P2P.send_protobuf(request, writer)
            if writer.can_write_eof():
                writer.write_eof()

        # requests start flowing right away, even if the caller reads the responses later
        writing_task = asyncio.create_task(_write_to_stream())
        # its outcome is collected below when the responses end normally; if the caller leaves earlier, a failure of
        # the writing side (typically: the connection went away) has nobody to report to
        writing_task.add_done_callback(lambda task: task.cancelled() or task.exception())

        async def _read_from_stream() -> AsyncIterator[Message]:
            with closing(writer):
                try:
                    while True:
                        try:
                            response, err = await P2P.receive_protobuf(output_protobuf_type, reader)
                        except asyncio.IncompleteReadError:
                            break
                        if err is not None:
                            raise P2PHandlerError(f"Failed to call handler `{name}` at {peer_id}: {err.message}")
                        yield response
                    await writing_task
                finally:
                    writing_task.cancel()

        return _read_from_stream()

    async def call_protobuf_handler(self, peer_id: PeerID, name: str, input: Union[Message, AsyncIterator[Message]],
                                    output_protobuf_type: Type[Message]) -> Awaitable[Message]:
        if not hasattr(input, "__aiter__"):
            return await self._call_unary_protobuf_handler(peer_id, name, input, output_protobuf_type)
        responses = await self._iterate_protobuf_stream_handler(peer_id, name, input, output_protobuf_type)
        return await asingle(responses)

    async def _call_unary_protobuf_handler(self, peer_id: PeerID, name: str, input: Message,
                                           output_protobuf_type: Type[Message]) -> Message:
        serialized = input.SerializeToString()
        response = await self._client.call_unary_handler(peer_id, name, serialized)
        return output_protobuf_type.FromString(response)

    async def iterate_protobuf_handler(self, peer_id: PeerID, name: str, input: Union[Message, AsyncIterator[Message]],
                                       output_protobuf_type: Type[Message]) -> AsyncIterator[Message]:
        requests = input if hasattr(input, "__aiter__") else as_aiter(input)
        return await self._iterate_protobuf_stream_handler(peer_id, name, requests, output_protobuf_type)

    async def add_binary_stream_handler(self, name: str, handler: Callable, balanced: bool = False) -> None:
        await self._client.stream_handler(name, handler, balanced)

    async def remove_binary_stream_handler(self, name: str) -> None:
        await self._client.remove_stream_handler(name)

    async def call_binary_stream_handler(self, peer_id: PeerID, handler_name: str
                                         ) -> Tuple[StreamInfo, asyncio.StreamReader, asyncio.StreamWriter]:
        try:
            return await self._client.stream_open(peer_id, (handler_name,))
        except P2PDaemonError as e:
            raise P2PHandlerError(f"Failed to open stream `{handler_name}` at {peer_id}: {e}") from e

    # ------------------------------------------------------------------------------------------ shutdown
    def __del__(self):
        self._terminate()

    @property
    def is_alive(self) -> bool:
        return self._alive

    async def shutdown(self) -> None:
        if self._client is not None:
            with suppress(Exception):
                await self._client.close()
            self._client = None
        self._terminate()

    def _terminate(self) -> None:
        self._alive = False
        child, self._child = self._child, None
        if child is not None and child.poll() is None:
            child.terminate()
            try:
                child.wait(timeout=2)
            except Exception:
                child.kill()
            logger.debug(f"terminated transport daemon, pid {child.pid}")
        if child is not None and self._workdir is not None:
            with suppress(OSError):
                for entry in os.listdir(self._workdir):
                    with suppress(OSError):
                        os.unlink(os.path.join(self._workdir, entry))
                os.rmdir(self._workdir)

    @staticmethod
    def _read_outputs(child: Optional[subprocess.Popen], loop: asyncio.AbstractEventLoop, ready: asyncio.Future) -> None:
        """Runs in a thread: wait for the daemon's "Ready" line, then forward its stderr to the logger."""
        if child is None:
            return
        last_words: List[str] = []
        try:
            for line in child.stdout:
                line = line.strip()
                if line == "Ready":
                    loop.call_soon_threadsafe(lambda: ready.done() or ready.set_result(None))
                    break
            for line in child.stderr:
                line = line.rstrip()
                if line:
                    last_words = (last_words + [line])[-5:]
                    logger.debug(line if line.startswith("[hmp2pd]") else f"[hmp2pd] {line}")
        except Exception:
            pass
        finally:
            if not ready.done():
                said = (": " + " | ".join(last_words)) if last_words else ""
                with suppress(RuntimeError):
                    loop.call_soon_threadsafe(
                        lambda: ready.done() or ready.set_exception(P2PDaemonError("transport daemon exited at start" + said)))

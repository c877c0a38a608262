"""A stream reader for large messages.

``asyncio.StreamReader`` appends every received block to one ``bytearray`` and cuts results off its front, which for a
message of several hundred kilobytes means three passes over the bytes (append, slice, close the gap). This reader
keeps the received blocks as they are and assembles a result with a single copy; everything else (flow control through
the transport, EOF, exceptions, the waiter) is inherited. Only the methods the package uses are supported:
``read``, ``readexactly``, ``at_eof`` and iteration helpers that rest on them; ``readline`` / ``readuntil`` are not.
"""
from __future__ import annotations

import asyncio
from collections import deque
from typing import Callable, Deque, Optional, Tuple


class ChunkedStreamReader(asyncio.StreamReader):
    def __init__(self, limit: int = 2 ** 20, loop: Optional[asyncio.AbstractEventLoop] = None):
        super().__init__(limit=limit, loop=loop)
        self._chunks: Deque[bytes] = deque()
        self._offset = 0  # bytes of the first chunk that were handed out already
        self._size = 0    # bytes waiting in all chunks together

    # --- producer side (called by StreamReaderProtocol) -------------------------------------------------------
    def feed_data(self, data) -> None:
        assert not self._eof, "feed_data after feed_eof"
        if not data:
            return
        self._chunks.append(bytes(data) if not isinstance(data, bytes) else data)
        self._size += len(data)
        self._wakeup_waiter()
        if self._transport is not None and not self._paused and self._size > 2 * self._limit:
            try:
                self._transport.pause_reading()
            except NotImplementedError:
                self._transport = None  # cannot be paused: buffer whatever comes
            else:
                self._paused = True

    def _maybe_resume_transport(self) -> None:
        if self._paused and self._size <= self._limit:
            self._paused = False
            self._transport.resume_reading()

    def at_eof(self) -> bool:
        return self._eof and self._size == 0

    # --- consumer side -----------------------------------------------------------------------------------------
    def _take(self, n: int) -> bytes:
        """Remove and return the first ``n`` waiting bytes (``n`` <= ``self._size``)."""
        first = self._chunks[0]
        if self._offset == 0 and len(first) == n:  # a whole block is wanted: hand it over without copying
            self._chunks.popleft()
            self._size -= n
            return first
        pieces, wanted = [], n
        while wanted:
            chunk = self._chunks[0]
            available = len(chunk) - self._offset
            if available <= wanted:
                pieces.append(memoryview(chunk)[self._offset:] if self._offset else chunk)
                self._chunks.popleft()
                self._offset = 0
                wanted -= available
            else:
                pieces.append(memoryview(chunk)[self._offset:self._offset + wanted])
                self._offset += wanted
                wanted = 0
        self._size -= n
        return b"".join(pieces)

    async def read(self, n: int = -1) -> bytes:
        if self._exception is not None:
            raise self._exception
        if n == 0:
            return b""
        if n < 0:
            blocks = []
            while True:
                block = await self.read(self._limit)
                if not block:
                    break
                blocks.append(block)
            return b"".join(blocks)
        if self._size == 0 and not self._eof:
            await self._wait_for_data("read")
        data = self._take(min(n, self._size)) if self._size else b""
        self._maybe_resume_transport()
        return data

    async def readexactly(self, n: int) -> bytes:
        if n < 0:
            raise ValueError("readexactly size can not be less than zero")
        if self._exception is not None:
            raise self._exception
        if n == 0:
            return b""
        while self._size < n:
            if self._eof:
                incomplete = self._take(self._size) if self._size else b""
                raise asyncio.IncompleteReadError(incomplete, n)
            # a read larger than the flow-control limit must not wait for a transport that was paused because of it
            if self._paused:
                self._paused = False
                self._transport.resume_reading()
            await self._wait_for_data("readexactly")
        data = self._take(n)
        self._maybe_resume_transport()
        return data

    async def readline(self) -> bytes:
        raise NotImplementedError("this reader carries length-prefixed frames; there are no lines to read")

    async def readuntil(self, separator: bytes = b"\n") -> bytes:
        raise NotImplementedError("this reader carries length-prefixed frames; there are no separators to look for")


async def open_unix_stream(path: str, limit: int = 2 ** 20) -> Tuple[ChunkedStreamReader, asyncio.StreamWriter]:
    """``asyncio.open_unix_connection`` with a ``ChunkedStreamReader`` on the receiving side."""
    loop = asyncio.get_running_loop()
    reader = ChunkedStreamReader(limit=limit, loop=loop)
    protocol = asyncio.StreamReaderProtocol(reader, loop=loop)
    transport, _ = await loop.create_unix_connection(lambda: protocol, path)
    return reader, asyncio.StreamWriter(transport, protocol, reader, loop)


async def start_unix_stream_server(client_connected: Callable, path: str, limit: int = 2 ** 20) -> asyncio.AbstractServer:
    """``asyncio.start_unix_server`` whose connections read through ``ChunkedStreamReader``."""
    loop = asyncio.get_running_loop()

    def factory() -> asyncio.StreamReaderProtocol:
        reader = ChunkedStreamReader(limit=limit, loop=loop)
        return asyncio.StreamReaderProtocol(reader, client_connected, loop=loop)

    return await loop.create_unix_server(factory, path)

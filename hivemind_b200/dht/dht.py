"""``DHT``: the user-facing handle of a DHT node that runs on its own event-loop thread.

The reference forks a process for this (hivemind/dht/dht.py:22-337) and talks to it through a pipe and MPFutures.
A forked process cannot share a CUDA context, so here the node lives on a daemon thread with a private event loop;
the public methods (``get``, ``store``, ``run_coroutine``, ``add_validators``, ``peer_id``, ``client_mode``,
``get_visible_maddrs``, ``replicate_p2p``, ``shutdown``) keep their signatures, ``return_future=True`` returns an
``MPFuture``, and ``run_coroutine(coro)`` still runs ``coro(dht, node)`` inside the DHT's own loop.
"""
from __future__ import annotations

import asyncio
import threading
from functools import partial
from typing import Awaitable, Callable, Iterable, List, Optional, Sequence, TypeVar, Union

from hivemind_b200.dht.node import DEFAULT_NUM_WORKERS, DHTNode
from hivemind_b200.dht.routing import DHTKey, DHTValue, Subkey
from hivemind_b200.dht.validation import CompositeValidator, RecordValidatorBase
from hivemind_b200.p2p import P2P, PeerID
from hivemind_b200.utils import MPFuture, get_logger
from hivemind_b200.utils.asyncio import LoopThread
from hivemind_b200.utils.multiaddr import Multiaddr
from hivemind_b200.utils.timed_storage import DHTExpiration, ValueWithExpiration

logger = get_logger(__name__)
ReturnType = TypeVar("ReturnType")


class DHT:
    """
    :param initial_peers: multiaddrs of one or more active DHT peers (to join an existing DHT)
    :param start: if True, start the node right away; otherwise call ``run_in_background()``
    :param num_workers: concurrent workers of one get/store traversal
    :param record_validators: validators applied to every stored and retrieved record
    :param shutdown_timeout: seconds to wait for a graceful stop
    :param await_ready: if True, the constructor returns after bootstrap is finished
    :param kwargs: forwarded to ``DHTNode.create`` (and from there to ``P2P.create``)
    """

    _node: DHTNode

    def __init__(self, initial_peers: Optional[Sequence[Union[Multiaddr, str]]] = None, *, start: bool,
                 p2p: Optional[P2P] = None, daemon: bool = True, num_workers: int = DEFAULT_NUM_WORKERS,
                 record_validators: Iterable[RecordValidatorBase] = (), shutdown_timeout: float = 3,
                 await_ready: bool = True, **kwargs):
        self._parent_pid = None
        if not (initial_peers is None or (isinstance(initial_peers, Sequence) and
                                          all(isinstance(item, (Multiaddr, str)) for item in initial_peers))):
            raise TypeError("initial_peers should be of type Optional[Sequence[Union[Multiaddr, str]]]")
        self.initial_peers = initial_peers
        self.kwargs = kwargs
        self.num_workers = num_workers
        self._record_validator = CompositeValidator(record_validators)
        self.shutdown_timeout = shutdown_timeout
        self._ready = MPFuture()
        self._peer_id: Optional[PeerID] = None
        self._client_mode: Optional[bool] = None
        self._p2p_replicas = {}  # event loop -> P2P client attached to the same daemon
        self._origin_p2p = p2p
        self._thread: Optional[LoopThread] = None
        self._node: Optional[DHTNode] = None
        self._shutdown_lock = threading.Lock()
        self.daemon = daemon
        if start:
            self.run_in_background(await_ready=await_ready)

    # ---------------------------------------------------------------------------------------------- lifecycle
    def run_in_background(self, await_ready: bool = True, timeout: Optional[float] = None) -> None:
        """Start the DHT thread; with ``await_ready`` wait until the node has bootstrapped (or raise its error)."""
        if self._thread is not None:
            return
        self._thread = LoopThread(name=f"DHT-{id(self):x}").start()

        async def _start():
            try:
                self._node = await DHTNode.create(initial_peers=self.initial_peers, num_workers=self.num_workers,
                                                  record_validator=self._record_validator, p2p=self._origin_p2p,
                                                  **self.kwargs)
                self._peer_id, self._client_mode = self._node.peer_id, self._node.protocol.client_mode
                self._ready.set_result(None)
            except Exception as e:
                logger.debug(e, exc_info=True)
                self._ready.set_exception(e)

        self._thread.submit(_start())
        if await_ready:
            self.wait_until_ready(timeout)

    def run(self) -> None:
        """Blocking variant kept for interface parity: start and wait until shutdown."""
        self.run_in_background(await_ready=True)
        while self.is_alive():
            threading.Event().wait(0.5)

    def wait_until_ready(self, timeout: Optional[float] = None) -> None:
        self._ready.result(timeout=timeout)

    def is_alive(self) -> bool:
        return self._thread is not None and self._thread.is_alive and self._node is not None and self._node.is_alive

    def shutdown(self) -> None:
        """Stop the node, its transport daemon and the thread."""
        with self._shutdown_lock:
            thread, self._thread = self._thread, None
        if thread is None:
            return
        if self._node is not None:
            try:
                thread.run(self._node.shutdown(), timeout=self.shutdown_timeout)
            except Exception as e:
                logger.debug(f"DHT did not shut down cleanly: {e!r}")
        replicas, self._p2p_replicas = self._p2p_replicas, {}
        for loop, replica in replicas.items():
            try:  # close each replica on the loop that owns its sockets, if that loop still runs
                if loop.is_running():
                    asyncio.run_coroutine_threadsafe(replica.shutdown(), loop).result(self.shutdown_timeout)
            except Exception as e:
                logger.debug(f"Could not close a transport replica: {e!r}")
        thread.stop()

    def __del__(self):
        try:
            self.shutdown()
        except Exception:
            pass

    # ---------------------------------------------------------------------------------------------- calls
    def _submit(self, coro: Awaitable[ReturnType], return_future: bool) -> Union[ReturnType, MPFuture]:
        if self._thread is None:
            raise RuntimeError("DHT is not running (call run_in_background() first, or it was shut down)")
        future: MPFuture = MPFuture()

        async def _runner():
            try:
                result = await coro
                if not future.done():
                    future.set_result(result)
            except BaseException as e:
                if not future.done():
                    future.set_exception(e if isinstance(e, Exception) else RuntimeError(repr(e)))
                if not isinstance(e, Exception):
                    raise

        task_holder = {}

        def _schedule():
            task_holder["task"] = asyncio.ensure_future(_runner())

        self._thread.loop.call_soon_threadsafe(_schedule)
        future.add_done_callback(lambda f: f.cancelled() and "task" in task_holder
                                 and self._thread is not None and self._thread.loop is not None
                                 and self._thread.loop.call_soon_threadsafe(task_holder["task"].cancel))
        return future if return_future else future.result()

    def get(self, key: DHTKey, latest: bool = False, return_future: bool = False, **kwargs
            ) -> Union[Optional[ValueWithExpiration[DHTValue]], MPFuture]:
        """Find the value for ``key``; None if not found.

        :param latest: search for the freshest value instead of the first one found
        :returns: ``ValueWithExpiration(value, expiration)``; for dictionary keys ``value`` maps each sub-key to
          its own ``ValueWithExpiration``
        """
        assert self._ready.done() and self._ready.exception() is None, "DHT is not ready"
        return self._submit(self._node.get(key, latest=latest, **kwargs), return_future)

    def store(self, key: DHTKey, value: DHTValue, expiration_time: DHTExpiration, subkey: Optional[Subkey] = None,
              return_future: bool = False, **kwargs) -> Union[bool, MPFuture]:
        """Store ``value`` under ``key`` (or ``key[subkey]``) until ``expiration_time``; True if a node accepted it."""
        assert self._ready.done() and self._ready.exception() is None, "DHT is not ready"
        return self._submit(self._node.store(key, value, expiration_time, subkey=subkey, **kwargs), return_future)

    def run_coroutine(self, coro: Callable[["DHT", DHTNode], Awaitable[ReturnType]], return_future: bool = False
                      ) -> Union[ReturnType, MPFuture[ReturnType]]:
        """Run ``await coro(dht, node)`` inside the DHT's event loop and return (a future of) its result.

        The coroutine shares the loop with the node: long blocking code in it stalls the DHT.
        """
        assert self._ready.done() and self._ready.exception() is None, "DHT is not ready"
        return self._submit(coro(self, self._node), return_future)

    def add_validators(self, record_validators: Iterable[RecordValidatorBase]) -> None:
        if not self._ready.done():
            raise RuntimeError("validators can only be added once the DHT is ready (or through the constructor)")
        self.run_coroutine(partial(DHT._add_validators, record_validators=record_validators))

    @staticmethod
    async def _add_validators(_dht: "DHT", node: DHTNode, record_validators: Iterable[RecordValidatorBase]) -> None:
        node.protocol.record_validator.extend(record_validators)

    @property
    def peer_id(self) -> PeerID:
        self.wait_until_ready()
        return self._peer_id

    @property
    def client_mode(self) -> bool:
        self.wait_until_ready()
        return self._client_mode

    @property
    def node(self) -> DHTNode:
        """The node object; its coroutines must be awaited on the DHT loop (see ``run_coroutine``)."""
        self.wait_until_ready()
        return self._node

    @property
    def loop(self) -> asyncio.AbstractEventLoop:
        return self._thread.loop

    def get_visible_maddrs(self, latest: bool = False) -> List[Multiaddr]:
        """Addresses through which other peers can reach this one (each ends with ``/p2p/<peer id>``)."""
        return self.run_coroutine(partial(DHT._get_visible_maddrs, latest=latest))

    @staticmethod
    async def _get_visible_maddrs(_dht: "DHT", node: DHTNode, latest: bool = False) -> List[Multiaddr]:
        return await node.get_visible_maddrs(latest=latest)

    async def replicate_p2p(self) -> P2P:
        """A ``P2P`` client attached to the same transport daemon, usable from the calling event loop."""
        loop = asyncio.get_running_loop()
        replica = self._p2p_replicas.get(loop)
        if replica is None:
            # one replica per calling loop: its sockets belong to that loop
            daemon_listen_maddr = self.run_coroutine(DHT._get_p2p_daemon_listen_maddr)
            replica = self._p2p_replicas[loop] = await P2P.replicate(daemon_listen_maddr)
        return replica

    @staticmethod
    async def _get_p2p_daemon_listen_maddr(_dht: "DHT", node: DHTNode) -> Multiaddr:
        return node.p2p.daemon_listen_maddr

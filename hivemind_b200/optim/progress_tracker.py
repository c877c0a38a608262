"""``ProgressTracker``: how many samples the whole swarm has accumulated towards the next epoch.

Every peer publishes a signed ``LocalTrainingProgress`` record under the DHT key ``{prefix}_progress`` (sub-key = the
peer's ``[owner:...]`` public-key marker, so nobody can overwrite another peer's record) and periodically fetches all
records to estimate when ``target_batch_size`` will be reached; the refresh period adapts to that ETA.
Contract: hivemind/optim/progress_tracker.py:20-363. Here the reporter and the fetcher are two tasks on one
event-loop thread, woken through loop-safe events rather than by polling threading events in an executor.
"""
from __future__ import annotations

import asyncio
import contextlib
import logging
import threading
from dataclasses import dataclass
from typing import Dict, Optional

import numpy as np
import pydantic.v1 as pydantic

from hivemind_b200.dht import DHT
from hivemind_b200.dht.crypto import RSASignatureValidator
from hivemind_b200.dht.schema import BytesWithPublicKey, SchemaValidator
from hivemind_b200.utils import DHTExpiration, PerformanceEMA, ValueWithExpiration, get_dht_time, get_logger
from hivemind_b200.utils.asyncio import LoopThread
from hivemind_b200.utils.crypto import RSAPrivateKey

logger = get_logger(__name__)


@dataclass(frozen=False)
class GlobalTrainingProgress:
    epoch: int
    samples_accumulated: int
    target_batch_size: int
    num_peers: int
    num_clients: int
    eta_next_epoch: float
    next_fetch_time: float


class LocalTrainingProgress(pydantic.BaseModel):
    peer_id: bytes
    epoch: pydantic.conint(ge=0, strict=True)
    samples_accumulated: pydantic.conint(ge=0, strict=True)
    samples_per_second: pydantic.confloat(ge=0.0, strict=True)
    time: pydantic.StrictFloat
    client_mode: pydantic.StrictBool


class TrainingProgressSchema(pydantic.BaseModel):
    progress: Dict[BytesWithPublicKey, Optional[LocalTrainingProgress]]


class ProgressTracker:
    """
    :param dht: a running DHT
    :param prefix: run id; all peers of one run share it
    :param target_batch_size: samples per epoch, summed over all peers
    :param min_refresh_period / max_refresh_period / default_refresh_period: bounds (seconds) on how often the
      swarm's records are fetched; the actual period shrinks as the epoch's end approaches
    :param expected_drift_peers / expected_drift_rate: slack for peers joining between two fetches
    :param metadata_expiration: lifetime of a published record; it is re-published at half that age
    :param private_key: key that signs this peer's records (default: a fresh key for this tracker)
    """

    def __init__(self, dht: DHT, prefix: str, target_batch_size: int, *, client_mode: Optional[bool] = None,
                 min_refresh_period: float = 0.5, max_refresh_period: float = 10, default_refresh_period: float = 3,
                 expected_drift_peers: float = 3, expected_drift_rate: float = 0.2, performance_ema_alpha: float = 0.1,
                 metadata_expiration: float = 60.0, status_loglevel: int = logging.DEBUG,
                 private_key: Optional[RSAPrivateKey] = None, daemon: bool = True, start: bool):
        client_mode = client_mode if client_mode is not None else dht.client_mode
        self.dht, self.prefix, self.client_mode = dht, prefix, client_mode
        self.training_progress_key = f"{self.prefix}_progress"
        self.target_batch_size = target_batch_size
        self.min_refresh_period, self.max_refresh_period = min_refresh_period, max_refresh_period
        self.default_refresh_period = default_refresh_period
        self.expected_drift_peers, self.expected_drift_rate = expected_drift_peers, expected_drift_rate
        self.status_loglevel = status_loglevel
        self.performance_ema = PerformanceEMA(alpha=performance_ema_alpha)
        self.metadata_expiration = metadata_expiration

        # peers are threads of one process here, so each tracker signs with a key of its own by default
        # (a process-wide key would make several in-process peers overwrite each other's record)
        signature_validator = RSASignatureValidator(private_key if private_key is not None else RSAPrivateKey())
        self._local_public_key = signature_validator.local_public_key
        dht.add_validators([SchemaValidator(TrainingProgressSchema, prefix=prefix), signature_validator])

        self.local_progress = self._get_local_progress(local_epoch=0, samples_accumulated=0)
        metadata, _expiration = self.dht.get(self.training_progress_key, latest=True) or (None, -float("inf"))
        self.global_progress = self._parse_swarm_progress_data(metadata)
        self.lock_global_progress = threading.Lock()
        self.fetched_global_progress_this_epoch = threading.Event()
        self.shutdown_triggered, self.shutdown_complete = threading.Event(), threading.Event()
        self._thread: Optional[LoopThread] = None
        self._report_evt: Optional[asyncio.Event] = None
        self._refetch_evt: Optional[asyncio.Event] = None
        if start:
            self.start()

    # ---------------------------------------------------------------------------------------------- lifecycle
    def start(self) -> None:
        if self._thread is not None:
            return
        self._thread = LoopThread(name=f"{type(self).__name__}({self.prefix})").start()

        async def _init():
            self._report_evt, self._refetch_evt = asyncio.Event(), asyncio.Event()
            self._tasks = [asyncio.create_task(self._progress_reporter()), asyncio.create_task(self._progress_fetcher())]

        self._thread.run(_init())

    def is_alive(self) -> bool:
        return self._thread is not None and self._thread.is_alive and not self.shutdown_triggered.is_set()

    def _wake(self, event_name: str) -> None:
        thread = self._thread
        if thread is not None and thread.loop is not None:
            event = getattr(self, event_name)
            if event is not None:
                thread.loop.call_soon_threadsafe(event.set)

    def shutdown(self, timeout: Optional[float] = None) -> None:
        """Stop tracking and tell the swarm that this peer is gone (a record with value None)."""
        if self.shutdown_triggered.is_set():
            return
        self.shutdown_triggered.set()
        thread, self._thread = self._thread, None
        if thread is not None:
            async def _stop():
                for task in getattr(self, "_tasks", []):
                    task.cancel()
            with contextlib.suppress(Exception):
                thread.run(_stop(), timeout=timeout or 5)
            thread.stop()
        self.shutdown_complete.set()
        with contextlib.suppress(Exception):
            self.dht.store(self.training_progress_key, subkey=self._local_public_key, value=None,
                           expiration_time=get_dht_time() + self.metadata_expiration, return_future=True)

    def __del__(self):
        with contextlib.suppress(Exception):
            if self.is_alive():
                self.shutdown()

    # ---------------------------------------------------------------------------------------------- queries
    @property
    def global_epoch(self) -> int:
        return self.global_progress.epoch

    @property
    def ready_to_update_epoch(self) -> bool:
        """True if this peer may move to the next epoch right now."""
        return (self.global_epoch > self.local_progress.epoch
                or self.global_progress.samples_accumulated >= self.target_batch_size
                or get_dht_time() >= self.global_progress.eta_next_epoch)

    @property
    def estimated_next_update_time(self) -> DHTExpiration:
        """Absolute time at which the swarm is expected to finish the current epoch."""
        if self.ready_to_update_epoch:
            return get_dht_time()
        return self.global_progress.eta_next_epoch

    def _get_local_progress(self, local_epoch: int, samples_accumulated: int) -> LocalTrainingProgress:
        return LocalTrainingProgress(peer_id=self.dht.peer_id.to_bytes(), epoch=local_epoch,
                                     samples_accumulated=samples_accumulated,
                                     samples_per_second=self.performance_ema.samples_per_second, time=get_dht_time(),
                                     client_mode=self.client_mode)

    # ---------------------------------------------------------------------------------------------- updates
    def report_local_progress(self, local_epoch: int, samples_accumulated: int, update_global_samples: bool = True) -> None:
        """Record how many samples this peer has accumulated in ``local_epoch`` and publish it soon."""
        extra_samples = samples_accumulated - self.local_progress.samples_accumulated
        if update_global_samples and local_epoch == self.local_progress.epoch == self.global_progress.epoch:
            self.global_progress.samples_accumulated += extra_samples
        if extra_samples > 0:
            self.performance_ema.update(task_size=extra_samples)
        else:
            self.performance_ema.reset_timer()  # progress was reset
        self.local_progress = self._get_local_progress(local_epoch, samples_accumulated)
        self._wake("_report_evt")

    @contextlib.contextmanager
    def pause_updates(self):
        """Keep the fetcher from replacing ``global_progress`` (and do not count the time as training time)."""
        with self.lock_global_progress, self.performance_ema.pause():
            yield

    def update_epoch(self, new_epoch: Optional[int] = None) -> int:
        """Move to ``new_epoch`` (default: next), reset sample counters; must be called inside ``pause_updates``."""
        assert self.lock_global_progress.locked(), "ProgressTracker must be paused when incrementing epoch"
        if new_epoch is None:
            new_epoch = self.local_progress.epoch + 1
        if new_epoch > self.global_progress.epoch:
            self.global_progress.epoch = new_epoch
            self.global_progress.samples_accumulated = 0
            self.global_progress.eta_next_epoch = float("inf")
        self.report_local_progress(new_epoch, samples_accumulated=0)
        self.fetched_global_progress_this_epoch.clear()
        return new_epoch

    def trigger_refetch(self) -> None:
        """Fetch the swarm's records now instead of at the scheduled time."""
        self.global_progress.next_fetch_time = get_dht_time()
        self._wake("_refetch_evt")

    # ---------------------------------------------------------------------------------------------- background tasks
    async def _progress_reporter(self) -> None:
        last_report_time = -float("inf")
        last_report_epoch = -float("inf")
        store_task = None
        try:
            while not self.shutdown_triggered.is_set():
                wait_timeout = max(0.0, last_report_time - get_dht_time() + self.metadata_expiration / 2)
                with contextlib.suppress(asyncio.TimeoutError):
                    await asyncio.wait_for(self._report_evt.wait(), wait_timeout)
                self._report_evt.clear()
                local_progress = self.local_progress
                last_report_time = get_dht_time()
                if local_progress.samples_accumulated > 0:
                    last_report_epoch = self.global_epoch
                if last_report_epoch >= self.global_epoch - 1:  # peers that stopped contributing fall silent
                    store_task = asyncio.create_task(asyncio.wait_for(self.dht.store(
                        key=self.training_progress_key, subkey=self._local_public_key, value=local_progress.dict(),
                        expiration_time=last_report_time + self.metadata_expiration, return_future=True),
                        timeout=self.metadata_expiration))
        finally:
            logger.log(self.status_loglevel, f"No longer reporting progress for {self.prefix}")
            if store_task is not None:
                store_task.cancel()

    async def _progress_fetcher(self) -> None:
        try:
            while not self.shutdown_triggered.is_set():
                time_to_next_update = max(0.0, self.global_progress.next_fetch_time - get_dht_time())
                with contextlib.suppress(asyncio.TimeoutError):
                    await asyncio.wait_for(self._refetch_evt.wait(), time_to_next_update)
                self._refetch_evt.clear()
                loop = asyncio.get_event_loop()
                acquired = await loop.run_in_executor(None, self.lock_global_progress.acquire, True, 1.0)
                if not acquired:
                    continue
                try:
                    maybe_metadata = await self.dht.get(self.training_progress_key, latest=True, return_future=True)
                    if self.shutdown_triggered.is_set():
                        break
                    metadata = maybe_metadata.value if isinstance(maybe_metadata, ValueWithExpiration) else None
                    self.global_progress = self._parse_swarm_progress_data(metadata)
                    self.fetched_global_progress_this_epoch.set()
                finally:
                    self.lock_global_progress.release()
        except asyncio.CancelledError:
            pass
        finally:
            logger.log(self.status_loglevel, f"No longer fetching {self.training_progress_key}")

    def _parse_swarm_progress_data(self, metadata) -> GlobalTrainingProgress:
        """Combine all peers' records into the swarm's epoch, sample count and ETA of the next epoch."""
        current_time = get_dht_time()
        if not isinstance(metadata, dict) or len(metadata) == 0:
            logger.log(self.status_loglevel, f"Found no active peers: {metadata}")
            samples_remaining = max(0, self.target_batch_size - self.local_progress.samples_accumulated)
            local_eta = samples_remaining / self.performance_ema.samples_per_second
            return GlobalTrainingProgress(self.local_progress.epoch, self.local_progress.samples_accumulated,
                                          self.target_batch_size, num_peers=0, num_clients=0,
                                          eta_next_epoch=current_time + local_eta,
                                          next_fetch_time=current_time + self.default_refresh_period)
        valid_peer_entries = [LocalTrainingProgress.parse_obj(peer_state.value) for peer_state in metadata.values()
                              if peer_state.value is not None]
        num_peers = len(valid_peer_entries)
        num_clients = sum(peer.client_mode for peer in valid_peer_entries)
        global_epoch = self.local_progress.epoch
        for peer in valid_peer_entries:
            if not peer.client_mode:
                global_epoch = max(global_epoch, peer.epoch)
        total_samples_accumulated = estimated_current_samples = 0
        total_samples_per_second = self.performance_ema.eps
        for peer in valid_peer_entries:
            total_samples_per_second += peer.samples_per_second
            if peer.epoch == global_epoch:
                total_samples_accumulated += peer.samples_accumulated
                estimated_current_samples += (peer.samples_accumulated
                                              + max(0.0, current_time - peer.time) * peer.samples_per_second)
            # samples of peers that lag behind the global epoch do not count towards it
        estimated_samples_remaining = self.target_batch_size - estimated_current_samples
        estimated_time_to_next_epoch = max(0, estimated_samples_remaining) / total_samples_per_second
        expected_max_peers = max(num_peers + self.expected_drift_peers, num_peers * (1 + self.expected_drift_rate))
        time_to_next_fetch = float(np.clip(estimated_time_to_next_epoch * num_peers / expected_max_peers,
                                           self.min_refresh_period, self.max_refresh_period))
        logger.log(self.status_loglevel,
                   f"{self.prefix} accumulated {total_samples_accumulated} samples for epoch #{global_epoch} from "
                   f"{num_peers} peers. ETA {estimated_time_to_next_epoch:.2f} sec (refresh in {time_to_next_fetch:.2f} sec)")
        return GlobalTrainingProgress(global_epoch, total_samples_accumulated, target_batch_size=self.target_batch_size,
                                      num_peers=num_peers, num_clients=num_clients,
                                      eta_next_epoch=current_time + estimated_time_to_next_epoch,
                                      next_fetch_time=current_time + time_to_next_fetch)

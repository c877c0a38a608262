"""``Server``: hosts experts — connection handlers in front, one ``Runtime`` behind, DHT declarations on the side.

Behavioural contract from the reference (hivemind/moe/server/server.py:36-411): ``Server.create`` builds N identical
experts of a registered class with uids drawn from a pattern such as ``ffn.[0:32].[0:256]`` (skipping uids already
taken in the DHT), restores checkpoints, and starts; a running server answers forward/backward RPCs and re-declares
its experts every ``update_period`` seconds. Everything runs as threads of one process that owns one GPU: handler
event loops, the DHT loop, the checkpoint saver and the runtime thread that launches kernels.
"""
from __future__ import annotations

import random
import threading
from contextlib import contextmanager
from functools import partial
from pathlib import Path
from typing import Dict, List, Optional, Sequence

import torch

from hivemind_b200.dht import DHT
from hivemind_b200.moe.expert_uid import UID_DELIMITER
from hivemind_b200.moe.server.checkpoints import LAST_CHECKPOINT, CheckpointSaver, is_directory, load_experts
from hivemind_b200.moe.server.connection_handler import ConnectionHandler
from hivemind_b200.moe.server.dht_handler import DHTHandlerThread, get_experts
from hivemind_b200.moe.server.layers import (add_custom_models_from_file, name_to_block, name_to_input,
                                             schedule_name_to_scheduler)
from hivemind_b200.moe.server.layers.optim import ClippingWrapper
from hivemind_b200.moe.server.module_backend import ModuleBackend
from hivemind_b200.moe.server.runtime import Runtime
from hivemind_b200.p2p import PeerInfo
from hivemind_b200.proto.runtime_pb2 import CompressionType
from hivemind_b200.utils.logging import get_logger
from hivemind_b200.utils.tensor_descr import DUMMY_BATCH_SIZE, BatchTensorDescriptor

logger = get_logger(__name__)


class Server(threading.Thread):
    """
    :param dht: the DHT (and transport endpoint) used for all network interactions
    :param module_backends: uid -> ModuleBackend for every hosted expert
    :param num_connection_handlers: number of handler event loops sharing the incoming calls
    :param update_period: seconds between DHT re-declarations (and checkpoints)
    :param expiration: lifetime of a DHT declaration (default: max(2 * update_period, clock tolerance))
    :param start: start in the background and return once ready
    :param kwargs: forwarded to ``Runtime`` (device, stats_report_interval, ...)
    """

    def __init__(self, dht: DHT, module_backends: Dict[str, ModuleBackend], num_connection_handlers: int = 1,
                 update_period: float = 30, expiration: Optional[float] = None, start: bool = False,
                 checkpoint_dir: Optional[Path] = None, **kwargs):
        super().__init__(daemon=True, name="Server")
        self.dht, self.module_backends, self.update_period = dht, module_backends, update_period
        self.conn_handlers = [ConnectionHandler(dht, self.module_backends) for _ in range(num_connection_handlers)]
        self.checkpoint_saver = None
        if checkpoint_dir is not None:
            self.checkpoint_saver = CheckpointSaver(module_backends, checkpoint_dir, update_period)
        self.runtime = Runtime(self.module_backends, **kwargs)
        self.dht_handler_thread = None
        if self.module_backends:
            self.dht_handler_thread = DHTHandlerThread(module_backends=self.module_backends, dht=self.dht,
                                                       update_period=self.update_period, expiration=expiration,
                                                       daemon=True)
        self._shutdown_lock = threading.Lock()
        self._is_shut_down = False
        if start:
            self.run_in_background(await_ready=True)

    @classmethod
    def create(cls, num_experts: int = None, expert_uids: Sequence[str] = None, expert_pattern: str = None,
               expert_cls: str = "ffn", hidden_dim: int = 1024, optim_cls=torch.optim.Adam, scheduler: str = "none",
               num_warmup_steps: Optional[int] = None, num_training_steps: Optional[int] = None,
               clip_grad_norm: Optional[float] = None, num_handlers: Optional[int] = None, min_batch_size: int = 1,
               max_batch_size: int = 4096, device=None, initial_peers=(), checkpoint_dir: Optional[Path] = None,
               compression=CompressionType.NONE, stats_report_interval: Optional[int] = None,
               custom_module_path=None, update_period: float = 30, expiration: Optional[float] = None, *,
               start: bool, **kwargs) -> "Server":
        """
        Build a server with several identical experts.

        :param num_experts: how many experts to host; uids are sampled from ``expert_pattern``
        :param expert_pattern: e.g. ``myprefix.[0:32].[0:256]`` = uids between myprefix.0.0 and myprefix.31.255
        :param expert_uids: host exactly these uids (excludes num_experts / expert_pattern)
        :param expert_cls: a name registered with ``register_expert_class`` ('ffn', 'transformer', 'nop', ...)
        :param hidden_dim: main dimension passed to the expert class
        :param optim_cls: optimizer factory applied to each expert's parameters (None = frozen experts)
        :param scheduler: learning-rate schedule name ('none' or 'linear')
        :param clip_grad_norm: clip each expert's gradient norm to this value before its optimizer step
        :param num_handlers: number of connection handlers
        :param min_batch_size / max_batch_size: batching limits of every task pool
        :param device: torch device of all experts (default: cuda if available)
        :param initial_peers: multiaddrs of DHT peers to join
        :param checkpoint_dir: where to save, and on start restore, expert checkpoints
        :param compression: compression applied to every input, output and gradient of these experts
        :param kwargs: forwarded to the DHT
        """
        if custom_module_path is not None:
            add_custom_models_from_file(custom_module_path)
        assert expert_cls in name_to_block, f"unknown expert class {expert_cls}; known: {sorted(name_to_block)}"
        have_uids = expert_uids is not None
        assert have_uids != (num_experts is not None) and not (have_uids and expert_pattern is not None), \
            "Please provide either expert_uids *or* num_experts (possibly with expert_pattern), but not both"

        dht = DHT(initial_peers=initial_peers, start=True, **kwargs)
        logger.info(f"Running DHT node on {[str(a) for a in dht.get_visible_maddrs()]}, initial peers = {initial_peers}")
        try:
            if expert_uids is None:
                expert_uids = []
                if checkpoint_dir is not None:
                    assert is_directory(checkpoint_dir)
                    expert_uids = [child.name for child in checkpoint_dir.iterdir() if (child / LAST_CHECKPOINT).exists()]
                    logger.info(f"Located {len(expert_uids)} checkpoints for experts {expert_uids}")
                    if len(expert_uids) > num_experts:
                        raise ValueError(f"Found {len(expert_uids)} checkpoints, but num_experts is set to {num_experts}, "
                                         f"which is smaller. Either increase num_experts or remove unneeded checkpoints.")
                missing = num_experts - len(expert_uids)
                if missing > 0:
                    logger.info(f"Generating {missing} expert uids from pattern {expert_pattern}")
                    expert_uids.extend(_generate_uids(missing, expert_pattern, dht))
            expert_uids = list(expert_uids)
            num_handlers = num_handlers if num_handlers is not None else max(1, min(len(expert_uids), 4))
            device = device or ("cuda" if torch.cuda.is_available() else "cpu")

            sample_input = name_to_input[expert_cls](DUMMY_BATCH_SIZE, hidden_dim)
            samples = sample_input if isinstance(sample_input, tuple) else (sample_input,)
            args_schema = tuple(BatchTensorDescriptor.from_tensor(sample, compression) for sample in samples)

            make_scheduler = schedule_name_to_scheduler[scheduler]
            if make_scheduler is not None:
                make_scheduler = partial(make_scheduler, num_warmup_steps=num_warmup_steps,
                                         num_training_steps=num_training_steps)

            backends = {}
            for uid in expert_uids:
                module = name_to_block[expert_cls](hidden_dim)
                optimizer = optim_cls(module.parameters()) if optim_cls is not None else None
                lr_scheduler = make_scheduler(optimizer) if make_scheduler is not None and optimizer is not None else None
                if clip_grad_norm is not None and optimizer is not None:
                    optimizer = ClippingWrapper(optimizer, clip_grad_norm)
                backends[uid] = ModuleBackend(name=uid, module=module, args_schema=args_schema, optimizer=optimizer,
                                              scheduler=lr_scheduler, min_batch_size=min_batch_size,
                                              max_batch_size=max_batch_size)
            if checkpoint_dir is not None:
                load_experts(backends, checkpoint_dir)
        except BaseException:
            dht.shutdown()
            raise
        return cls(dht, backends, num_connection_handlers=num_handlers, device=device, checkpoint_dir=checkpoint_dir,
                   stats_report_interval=stats_report_interval, update_period=update_period, expiration=expiration,
                   start=start)

    def run(self) -> None:
        """Start handlers, declarations and checkpoints, then serve batches until ``shutdown``."""
        logger.info(f"Server started with {len(self.module_backends)} modules:")
        for uid, backend in self.module_backends.items():
            count = sum(p.numel() for p in backend.module.parameters() if p.requires_grad)
            logger.info(f"{uid}: {backend.module.__class__.__name__}, {count} parameters")
        if not self.dht.is_alive():
            self.dht.run_in_background(await_ready=True)
        for handler in self.conn_handlers:
            handler.run_in_background(await_ready=True)
        if self.dht_handler_thread is not None:
            self.dht_handler_thread.start()
        if self.checkpoint_saver is not None:
            self.checkpoint_saver.start()
        self.runtime.start()
        try:
            self.runtime.join()
        finally:
            self.shutdown()

    def run_in_background(self, await_ready: bool = True, timeout: Optional[float] = None) -> None:
        self.start()
        if await_ready and not self.ready.wait(timeout=timeout):
            raise TimeoutError(f"Server didn't notify .ready in {timeout} seconds")

    @property
    def ready(self) -> threading.Event:
        """Set while the server can process batches."""
        return self.runtime.ready

    def shutdown(self) -> None:
        """Stop handlers, declarations, checkpoints, the DHT and the runtime (idempotent)."""
        with self._shutdown_lock:
            if self._is_shut_down:
                return
            self._is_shut_down = True
        self.ready.clear()
        for handler in self.conn_handlers:
            handler.shutdown()
        logger.debug("Connection handlers terminated")
        if self.dht_handler_thread is not None:
            self.dht_handler_thread.stop.set()
            if self.dht_handler_thread.is_alive():
                self.dht_handler_thread.join(timeout=10)
        if self.checkpoint_saver is not None:
            self.checkpoint_saver.stop.set()
            if self.checkpoint_saver.is_alive():
                self.checkpoint_saver.join(timeout=30)
        self.dht.shutdown()
        logger.debug("Shutting down runtime")
        self.runtime.shutdown()
        logger.info("Server shutdown successfully")


@contextmanager
def background_server(*args, shutdown_timeout: float = 5, **kwargs):
    """Context manager: ``Server.create(..., start=True)`` on entry (yields the server's ``PeerInfo``), shutdown on exit.

    The server runs as threads of the calling process. Do not call its CUDA experts from a client layer's backward
    pass in the same process: the client blocks autograd's worker thread of that GPU while it waits for the experts,
    and the experts' own backward pass needs the same thread. Run the server as its own process in that case
    (``python -m hivemind_b200.hivemind_cli.run_server``), as the reference always does."""
    server = Server.create(*args, start=True, **kwargs)
    try:
        yield PeerInfo(server.dht.peer_id, server.dht.get_visible_maddrs())
    finally:
        logger.info("Shutting down server...")
        server.shutdown()
        server.join(timeout=shutdown_timeout)


def _generate_uids(num_experts: int, expert_pattern: Optional[str], dht: Optional[DHT] = None,
                   attempts_per_expert: int = 10) -> List[str]:
    """
    Sample ``num_experts`` distinct uids from ``expert_pattern`` (blocks are literals or ranges ``[from:to]``);
    with a ``dht``, uids that some peer already declared are skipped. Not race-free between concurrent servers.
    """
    budget = attempts_per_expert * num_experts
    attempts_left = budget
    chosen: List[str] = []
    seen = set()

    def sample_uid() -> str:
        if expert_pattern is None:
            return f"expert{UID_DELIMITER}{budget - attempts_left}"
        blocks = []
        for block in expert_pattern.split(UID_DELIMITER):
            if "[" not in block and "]" not in block:
                blocks.append(block)
                continue
            try:
                if not (block.startswith("[") and block.endswith("]") and ":" in block):
                    raise ValueError("Block must be either fixed or a range [from:to]")
                low, high = (int(bound) for bound in block[1:-1].split(":"))
                blocks.append(str(random.randint(low, high - 1)))
            except Exception as e:
                raise ValueError(f"Expert pattern {expert_pattern} has invalid block {block}, {e}")
        return UID_DELIMITER.join(blocks)

    while attempts_left > 0 and len(chosen) < num_experts:
        candidates = []
        want = num_experts - len(chosen)
        while len(candidates) < want and attempts_left > 0:
            uid = sample_uid()
            attempts_left -= 1
            if uid not in seen:
                seen.add(uid)
                candidates.append(uid)
        if dht is not None and candidates:
            taken = get_experts(dht, candidates)
            candidates = [uid for uid, found in zip(candidates, taken) if found is None]
        chosen.extend(candidates)
    if len(chosen) != num_experts:
        logger.warning(f"Found only {len(chosen)} out of {num_experts} free expert uids after {budget} attempts")
    return chosen

"""Periodic expert checkpoints: ``<dir>/<uid>/checkpoint_<timestamp>.pt`` plus a ``checkpoint_last.pt`` link.

Same on-disk layout as the reference (hivemind/moe/server/checkpoints.py:36-75) so that a server restarted with the
same ``checkpoint_dir`` finds its experts again. A checkpoint is written under a temporary name inside the expert's
directory and renamed, so a reader never sees a half-written file.
"""
from __future__ import annotations

import os
import threading
from datetime import datetime
from pathlib import Path
from typing import Dict

import torch

from hivemind_b200.moe.server.module_backend import ModuleBackend
from hivemind_b200.utils.logging import get_logger

logger = get_logger(__name__)
LAST_CHECKPOINT = "checkpoint_last.pt"


def is_directory(directory: Path) -> bool:
    assert directory is not None, "checkpoint directory is not set"
    assert directory.exists() and directory.is_dir(), f"{directory} is not an existing directory"
    return True


def store_experts(experts: Dict[str, ModuleBackend], checkpoint_dir: Path) -> None:
    """Write one timestamped checkpoint per expert and repoint ``checkpoint_last.pt`` at it."""
    assert is_directory(checkpoint_dir)
    logger.debug(f"Storing experts at {checkpoint_dir.absolute()}")
    stamp = datetime.now().isoformat(sep="_")
    for uid, backend in experts.items():
        expert_dir = checkpoint_dir / uid
        expert_dir.mkdir(exist_ok=True)
        final = expert_dir / f"checkpoint_{stamp}.pt"
        partial = expert_dir / f".checkpoint_{stamp}.pt.partial"
        torch.save(backend.state_dict(), partial)
        os.replace(partial, final)
        link_tmp = expert_dir / f".{LAST_CHECKPOINT}.{os.getpid()}"
        if link_tmp.is_symlink() or link_tmp.exists():
            link_tmp.unlink()
        os.symlink(final.name, link_tmp)  # relative link: the directory can be moved as a whole
        os.replace(link_tmp, expert_dir / LAST_CHECKPOINT)


def load_experts(experts: Dict[str, ModuleBackend], checkpoint_dir: Path) -> None:
    """Restore every expert that has a ``checkpoint_last.pt``; warn about the others."""
    assert is_directory(checkpoint_dir)
    for uid, backend in experts.items():
        latest = checkpoint_dir / uid / LAST_CHECKPOINT
        if latest.exists():
            backend.load_state_dict(torch.load(latest, map_location="cpu"))
        else:
            logger.warning(f"Failed to load checkpoint for expert {uid}")


class CheckpointSaver(threading.Thread):
    """Saves all experts every ``update_period`` seconds until ``stop`` is set."""

    def __init__(self, module_backends: Dict[str, ModuleBackend], checkpoint_dir: Path, update_period: float):
        super().__init__(daemon=True)
        assert is_directory(checkpoint_dir)
        self.module_backends, self.checkpoint_dir, self.update_period = module_backends, checkpoint_dir, update_period
        self.stop = threading.Event()
        store_experts(self.module_backends, self.checkpoint_dir)  # fail early if the directory is not writable

    def run(self) -> None:
        while not self.stop.wait(self.update_period):
            store_experts(self.module_backends, self.checkpoint_dir)

#!/usr/bin/env python3
"""A peer that does not train: it welcomes others into the DHT, aggregates the metrics that trainers publish and
(optionally) keeps checkpoints by downloading the swarm's current state, like the reference's
examples/albert/run_training_monitor.py:150-227 (the Weights & Biases and model-hub uploads are left out).

    python examples/albert/run_training_monitor.py --run_id demo --refresh_period 10
"""
import argparse
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch

import hivemind_b200 as hivemind
from hivemind_b200.models.albert import AlbertConfig, AlbertForMaskedLM
from hivemind_b200.optim.fused import FusedLAMB
from hivemind_b200.optim.state_averager import TrainingStateAverager
from hivemind_b200.utils.logging import get_logger, use_hivemind_log_handler
from hivemind_b200.utils.networking import log_visible_maddrs

import utils
from arguments import BaseTrainingArguments, add_dataclass_arguments, parse_into

use_hivemind_log_handler("in_root_logger")
logger = get_logger(__name__)


class CheckpointKeeper:
    """Downloads parameters and optimizer statistics from the trainers and writes them to disk."""

    def __init__(self, dht: hivemind.DHT, run_id: str, model_name: str, directory: str):
        cfg = AlbertConfig.large() if model_name == "large" else AlbertConfig.tiny()
        self.model = AlbertForMaskedLM(cfg)
        self.directory = directory
        os.makedirs(directory, exist_ok=True)
        self.state_averager = TrainingStateAverager(
            dht=dht, optimizer=lambda params: FusedLAMB(params, lr=0.00176), params=list(self.model.parameters()),
            prefix=f"{run_id}_state_averager", state_compression=hivemind.Float16Compression(), start=True,
            auxiliary=True, offload_optimizer=False)
        self.saved_step = -1

    def maybe_save(self, step: int, interval: int) -> None:
        if step - self.saved_step < interval:
            return
        logger.info(f"downloading the swarm's state at step {step}")
        self.state_averager.load_state_from_peers()
        path = os.path.join(self.directory, f"state_{step}.pt")
        torch.save({"model": self.model.state_dict(), "optimizer": self.state_averager.optimizer.state_dict(),
                    "step": step}, path)
        self.saved_step = step
        logger.info(f"saved {path}")

    def shutdown(self) -> None:
        self.state_averager.shutdown()


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    add_dataclass_arguments(parser, BaseTrainingArguments)
    parser.add_argument("--refresh_period", type=float, default=30, help="seconds between reads of the metrics key")
    parser.add_argument("--store_checkpoints", action="store_true", help="periodically download and save the state")
    parser.add_argument("--save_checkpoint_step_interval", type=int, default=5)
    parser.add_argument("--checkpoint_dir", default="monitor_checkpoints")
    parser.add_argument("--model", default="large", choices=["large", "tiny"])
    parser.add_argument("--max_reports", type=int, default=None, help="exit after this many aggregated reports")
    ns = parser.parse_args()
    base = parse_into(ns, BaseTrainingArguments)

    validators, _ = utils.make_validators(base.run_id)
    dht = hivemind.DHT(start=True, initial_peers=base.initial_peers, record_validators=validators,
                       host_maddrs=base.host_maddrs, announce_maddrs=base.announce_maddrs or None,
                       identity_path=base.identity_path)
    log_visible_maddrs(dht.get_visible_maddrs(), only_p2p=False)
    keeper = CheckpointKeeper(dht, base.run_id, ns.model, ns.checkpoint_dir) if ns.store_checkpoints else None

    current_step, reports = 0, 0
    try:
        while ns.max_reports is None or reports < ns.max_reports:
            entry = dht.get(base.run_id + "_metrics", latest=True)
            if entry is not None and isinstance(entry.value, dict):
                metrics = [utils.LocalMetrics.parse_obj(item.value) for item in entry.value.values()]
                latest_step = max(m.step for m in metrics)
                if latest_step != current_step:
                    current_step = latest_step
                    alive = [m for m in metrics if m.step == latest_step] or metrics
                    mini = sum(m.mini_steps for m in alive)
                    loss = sum(m.loss * m.mini_steps for m in alive) / max(mini, 1)
                    logger.info(f"step {current_step}: {len(alive)} peers alive, "
                                f"{sum(m.samples_accumulated for m in alive)} samples, "
                                f"{sum(m.samples_per_second for m in alive):.1f} samples/s, loss {loss:.4f}")
                    reports += 1
                    if keeper is not None:
                        keeper.maybe_save(current_step, ns.save_checkpoint_step_interval)
            time.sleep(ns.refresh_period)
    finally:
        if keeper is not None:
            keeper.shutdown()
        dht.shutdown()


if __name__ == "__main__":
    main()

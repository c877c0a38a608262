#!/usr/bin/env python3
"""Collaborative masked-LM training of an ALBERT-large-shaped model: one peer of a ``hivemind_b200.Optimizer`` run.

Every peer runs this script on its own GPU. The first peer starts a new DHT and prints its address; the others pass
it as ``--initial_peers``. Peers accumulate gradients locally; once the swarm as a whole has processed
``--target_batch_size`` samples they average gradients (8-bit by default) and take one LAMB step, all in the
background of the next forward/backward passes. Mirrors the reference's examples/albert/run_trainer.py:204-325 with
this package's model, kernels and fused LAMB.

    python examples/albert/run_trainer.py --run_id demo                    # first peer
    python examples/albert/run_trainer.py --run_id demo --initial_peers /ip4/.../tcp/.../p2p/...
"""
import argparse
import os
import sys
import time
from functools import partial

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch

import hivemind_b200 as hivemind
from hivemind_b200.models.albert import AlbertConfig, AlbertForMaskedLM, AlbertForPreTraining, make_mlm_batch
from hivemind_b200.optim.fused import FusedLAMB
from hivemind_b200.optim.power_sgd_averager import PowerSGDGradientAverager
from hivemind_b200.utils.logging import get_logger, use_hivemind_log_handler
from hivemind_b200.utils.networking import log_visible_maddrs

import utils
from arguments import (AveragerArguments, BaseTrainingArguments, OptimizerArguments, ProgressTrackerArguments,
                       TrainingArguments, add_dataclass_arguments, parse_into)

use_hivemind_log_handler("in_root_logger")
logger = get_logger(__name__)


class BatchSource:
    """Endless stream of pinned MLM batches: from a tokenized file if given, synthetic token ids otherwise."""

    def __init__(self, cfg: AlbertConfig, args: TrainingArguments, seed: int):
        self.cfg, self.args = cfg, args
        self.generator = torch.Generator().manual_seed(seed)
        self.tokens = None
        self.token_types = self.sentence_order = None
        if args.dataset_path:
            data = torch.load(args.dataset_path)
            self.tokens = data["input_ids"].to(torch.int64)
            assert self.tokens.shape[1] >= args.seq_length, "sequences in the dataset are shorter than --seq_length"
            if args.sentence_order:
                assert "sentence_order_label" in data, "--sentence_order needs a dataset made with --sentence_order"
                assert self.tokens.shape[1] == args.seq_length, "two-segment rows cannot be shortened"
                self.token_types, self.sentence_order = data["token_type_ids"], data["sentence_order_label"]

    def next(self):
        if self.tokens is None:
            batch = make_mlm_batch(self.cfg, self.args.per_device_train_batch_size, self.args.seq_length,
                                   generator=self.generator, pin=not self.args.sentence_order)
            if self.args.sentence_order:  # synthetic segments: the second one starts somewhere in the middle half
                size, length = self.args.per_device_train_batch_size, self.args.seq_length
                starts = torch.randint(length // 4, max(length // 4 + 1, 3 * length // 4), (size, 1), generator=self.generator)
                batch["token_type_ids"] = (torch.arange(length).unsqueeze(0) >= starts).long()
                batch["sentence_order_label"] = torch.randint(0, 2, (size,), generator=self.generator)
                if torch.cuda.is_available():
                    batch = {k: v.pin_memory() for k, v in batch.items()}
            return batch
        rows = torch.randint(0, self.tokens.shape[0], (self.args.per_device_train_batch_size,), generator=self.generator)
        ids = self.tokens[rows, :self.args.seq_length].clone()
        n_mask = max(1, int(round(0.15 * self.args.seq_length)))
        # padding and the [CLS] / [SEP] / [MASK] pieces (the lowest ids of the vocabulary) are never masked: they sort
        # behind every ordinary token, and a short sequence that still reaches them scores nothing there
        special = ids <= self.cfg.mask_token_id
        order = torch.rand(ids.shape, generator=self.generator).masked_fill_(special, 2.0)
        pos = order.argsort(dim=1)[:, :n_mask].contiguous()
        originals, untouched = ids.gather(1, pos), special.gather(1, pos)
        labels = torch.full_like(ids, -100)
        labels.scatter_(1, pos, originals.masked_fill(untouched, -100))
        ids.scatter_(1, pos, torch.where(untouched, originals, torch.full_like(originals, self.cfg.mask_token_id)))
        batch = {"input_ids": ids, "labels": labels, "masked_positions": pos}
        if self.sentence_order is not None:
            batch["token_type_ids"] = self.token_types[rows]
            batch["sentence_order_label"] = self.sentence_order[rows]
        return {k: v.pin_memory() for k, v in batch.items()} if torch.cuda.is_available() else batch


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    add_dataclass_arguments(parser, BaseTrainingArguments, AveragerArguments, ProgressTrackerArguments,
                            OptimizerArguments, TrainingArguments)
    ns = parser.parse_args()
    base, averager_args = parse_into(ns, BaseTrainingArguments), parse_into(ns, AveragerArguments)
    tracker_args, opt_args = parse_into(ns, ProgressTrackerArguments), parse_into(ns, OptimizerArguments)
    args = parse_into(ns, TrainingArguments)

    device = torch.device(args.device or ("cuda" if torch.cuda.is_available() else "cpu"))
    torch.manual_seed(args.seed)  # every peer starts from the same weights; late joiners download the current state
    cfg = AlbertConfig.large() if args.model == "large" else AlbertConfig.tiny()
    args.seq_length = min(args.seq_length, cfg.max_position_embeddings)
    model = (AlbertForPreTraining(cfg) if args.sentence_order else AlbertForMaskedLM(cfg)).to(device)

    validators, local_public_key = utils.make_validators(base.run_id)
    dht = hivemind.DHT(start=True, initial_peers=base.initial_peers, client_mode=opt_args.client_mode,
                       record_validators=validators, host_maddrs=base.host_maddrs,
                       announce_maddrs=base.announce_maddrs or None, identity_path=base.identity_path)
    log_visible_maddrs(dht.get_visible_maddrs(), only_p2p=False)

    no_decay = ("bias", "ln_weight", "ln_bias")
    groups = [
        {"params": [p for n, p in model.named_parameters() if not any(tag in n for tag in no_decay)],
         "weight_decay": args.weight_decay},
        {"params": [p for n, p in model.named_parameters() if any(tag in n for tag in no_decay)], "weight_decay": 0.0},
    ]
    make_optimizer = partial(FusedLAMB, lr=args.learning_rate, betas=(0.9, 0.999), eps=args.adam_epsilon,
                             clamp_value=args.clamp_value, debias=True)
    make_scheduler = lambda opt: torch.optim.lr_scheduler.LambdaLR(opt, lambda step: min(
        (step + 1) / max(args.warmup_steps, 1), max(0.0, (args.total_steps - step) / max(args.total_steps - args.warmup_steps, 1))))

    grad_averager_factory = None
    if opt_args.power_sgd_rank > 0:
        grad_averager_factory = partial(PowerSGDGradientAverager, averager_rank=opt_args.power_sgd_rank)
    averager_opts = dict(request_timeout=averager_args.request_timeout, target_group_size=averager_args.target_group_size)
    if averager_args.min_matchmaking_time is not None:
        averager_opts["min_matchmaking_time"] = averager_args.min_matchmaking_time

    optimizer = hivemind.Optimizer(
        dht=dht, run_id=base.run_id, target_batch_size=opt_args.target_batch_size,
        batch_size_per_step=args.per_device_train_batch_size * args.gradient_accumulation_steps,
        optimizer=make_optimizer, params=groups, scheduler=make_scheduler,
        matchmaking_time=opt_args.matchmaking_time, averaging_timeout=opt_args.averaging_timeout,
        next_chunk_timeout=opt_args.next_chunk_timeout, offload_optimizer=True,
        delay_optimizer_step=opt_args.delay_optimizer_step, delay_grad_averaging=opt_args.delay_grad_averaging,
        average_state_every=opt_args.average_state_every, use_local_updates=opt_args.use_local_updates,
        reuse_grad_buffers=not opt_args.use_local_updates and opt_args.power_sgd_rank == 0,
        client_mode=opt_args.client_mode, grad_compression=utils.make_compression(opt_args.grad_compression),
        state_averaging_compression=utils.make_compression(opt_args.state_compression),
        grad_averager_factory=grad_averager_factory, averager_opts=averager_opts,
        tracker_opts=dict(min_refresh_period=tracker_args.min_refresh_period,
                          max_refresh_period=tracker_args.max_refresh_period,
                          default_refresh_period=tracker_args.default_refresh_period,
                          expected_drift_peers=tracker_args.expected_drift_peers,
                          expected_drift_rate=tracker_args.expected_drift_rate,
                          metadata_expiration=tracker_args.metadata_expiration),
        verbose=True)
    if base.initial_peers:
        optimizer.load_state_from_peers()  # catch up with the swarm before contributing

    def params_are_finite() -> bool:
        return all(bool(torch.isfinite(p).all()) for p in model.parameters())

    def make_backup():
        return {"model": {k: v.detach().clone() for k, v in model.state_dict().items()}, "epoch": optimizer.local_epoch}

    backup = make_backup()  # restored if a collaborative step leaves non-finite weights behind
    source = BatchSource(cfg, args, seed=args.seed + 1 + hash(str(dht.peer_id)) % 10 ** 6)
    os.makedirs(args.output_dir, exist_ok=True)
    local_steps = samples = 0
    loss_sum, mini_steps, last_epoch, last_report = 0.0, 0, optimizer.local_epoch, time.perf_counter()
    try:
        while True:
            batch = {k: v.to(device, non_blocking=True) for k, v in source.next().items()}
            loss = model(**batch)
            loss.backward()
            local_steps += 1
            loss_sum += float(loss.item())
            mini_steps += 1
            samples += args.per_device_train_batch_size
            if local_steps % args.gradient_accumulation_steps == 0:
                optimizer.step()
                if not optimizer.grad_averager or not getattr(optimizer.grad_averager, "reuse_grad_buffers", False):
                    optimizer.zero_grad()
            if optimizer.local_epoch != last_epoch:  # a collaborative step has just been applied
                if not params_are_finite():
                    logger.warning("non-finite parameters after a collaborative step: restoring the last good state")
                    model.load_state_dict(backup["model"])
                    if base.initial_peers:
                        optimizer.load_state_from_peers()
                elif optimizer.local_epoch % args.backup_every_steps == 0:
                    backup = make_backup()
                now = time.perf_counter()
                record = utils.LocalMetrics(step=optimizer.local_epoch, samples_per_second=samples / max(now - last_report, 1e-9),
                                            samples_accumulated=samples, loss=loss_sum / max(mini_steps, 1),
                                            mini_steps=mini_steps)
                logger.info(f"step {record.step}: loss {record.loss:.4f}, {record.samples_per_second:.1f} samples/s locally")
                dht.store(key=base.run_id + "_metrics", subkey=local_public_key, value=record.dict(),
                          expiration_time=hivemind.get_dht_time() + args.statistics_expiration, return_future=True)
                if args.save_steps and optimizer.local_epoch % args.save_steps == 0:
                    torch.save({"model": model.state_dict(), "epoch": optimizer.local_epoch},
                               os.path.join(args.output_dir, f"checkpoint_{optimizer.local_epoch}.pt"))
                last_epoch, last_report, samples, loss_sum, mini_steps = optimizer.local_epoch, now, 0, 0.0, 0
            if args.max_local_steps is not None and local_steps >= args.max_local_steps:
                break
            if args.max_epochs is not None and optimizer.local_epoch >= args.max_epochs:
                break
    finally:
        optimizer.shutdown()
        dht.shutdown()


if __name__ == "__main__":
    main()

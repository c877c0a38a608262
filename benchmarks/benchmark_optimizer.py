"""Convergence of ``hivemind_b200.Optimizer`` with heterogeneous peers (reference: benchmarks/benchmark_optimizer.py).

``num_peers`` trainers (threads here; ``num_clients`` of them in client mode) with random batch sizes and random
per-batch delays train one small classifier together for ``max_epoch`` collaborative steps of ``target_batch_size``
samples. The data is a synthetic 10-class problem (the reference downloads MNIST; there is no network here).
Prints one JSON line with the final loss / accuracy of the first peer and the wall time.
"""
import argparse
import json
import os
import random
import sys
import threading
import time
from functools import partial

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.nn as nn
import torch.nn.functional as F

from hivemind_b200 import DHT, Float16Compression, Optimizer
from hivemind_b200.utils.crypto import RSAPrivateKey


def make_dataset(seed: int, samples: int = 8192, features: int = 784, classes: int = 10):
    g = torch.Generator().manual_seed(seed)
    prototypes = torch.randn(classes, features, generator=g)
    labels = torch.randint(0, classes, (samples,), generator=g)
    data = prototypes[labels] + 2.0 * torch.randn(samples, features, generator=g)
    return data, labels


def benchmark_optimizer(args):
    random.seed(args.seed)
    torch.manual_seed(args.seed)
    x_train, y_train = make_dataset(args.seed)
    dht_root = DHT(start=True)
    results = {}

    def run_trainer(index: int, batch_size: int, batch_time: float, client_mode: bool):
        torch.manual_seed(args.seed)  # identical initial weights
        model = nn.Sequential(nn.Linear(x_train.shape[1], args.hidden), nn.ReLU(), nn.Linear(args.hidden, 10)).to(args.device)
        dht = DHT(initial_peers=dht_root.get_visible_maddrs(), client_mode=client_mode, start=True)
        optimizer = Optimizer(
            run_id=args.run_id, target_batch_size=args.target_batch_size, batch_size_per_step=batch_size,
            params=model.parameters(), optimizer=partial(torch.optim.Adam, lr=args.lr),
            scheduler=partial(torch.optim.lr_scheduler.StepLR, gamma=args.lr_gamma, step_size=args.lr_step_size),
            dht=dht, tracker_opts=dict(private_key=RSAPrivateKey(), max_refresh_period=args.max_refresh_period),
            matchmaking_time=args.matchmaking_time, averaging_timeout=args.averaging_timeout,
            grad_compression=Float16Compression(), reuse_grad_buffers=args.reuse_grad_buffers,
            delay_grad_averaging=args.delay_grad_averaging, delay_optimizer_step=args.delay_optimizer_step,
            average_state_every=args.average_state_every, client_mode=client_mode, verbose=args.verbose and index == 0)
        rng = random.Random(args.seed + index)
        previous = time.perf_counter()
        loss = None
        while optimizer.local_epoch < args.max_epoch:
            time.sleep(max(0.0, previous + rng.gauss(batch_time, args.batch_time_std) - time.perf_counter()))
            batch = torch.randint(0, len(x_train), (batch_size,))
            loss = F.cross_entropy(model(x_train[batch].to(args.device)), y_train[batch].to(args.device))
            loss.backward()
            optimizer.step()
            if not args.reuse_grad_buffers:
                optimizer.zero_grad()
            previous = time.perf_counter()
        with torch.no_grad():
            logits = model(x_train[:2048].to(args.device))
            results[index] = dict(loss=float(F.cross_entropy(logits, y_train[:2048].to(args.device))),
                                  accuracy=float((logits.argmax(1).cpu() == y_train[:2048]).float().mean()),
                                  epoch=optimizer.local_epoch)
        time.sleep(args.winddown_time)
        optimizer.shutdown()
        dht.shutdown()

    threads = []
    for index in range(args.num_peers):
        threads.append(threading.Thread(target=run_trainer, kwargs=dict(
            index=index, batch_size=random.randint(args.batch_size_min, args.batch_size_max),
            batch_time=random.uniform(args.batch_time_min, args.batch_time_max),
            client_mode=index >= args.num_peers - args.num_clients)))
    started = time.perf_counter()
    for thread in threads:
        thread.start()
    for thread in threads:
        thread.join()
    elapsed = time.perf_counter() - started
    dht_root.shutdown()
    first = results.get(0, {})
    print(json.dumps({"benchmark": "optimizer_convergence", "seconds": elapsed, "final_loss": first.get("loss"),
                      "final_accuracy": first.get("accuracy"), "epochs": first.get("epoch"),
                      "samples_per_s": args.max_epoch * args.target_batch_size / elapsed,
                      "peers_finished": len(results), "config": vars(args)}), flush=True)
    return results


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--seed", type=int, default=42)
    parser.add_argument("--run_id", default="my_exp")
    parser.add_argument("--num_peers", type=int, default=8)
    parser.add_argument("--num_clients", type=int, default=3)
    parser.add_argument("--target_batch_size", type=int, default=256)
    parser.add_argument("--hidden", type=int, default=64)
    parser.add_argument("--reuse_grad_buffers", type=lambda s: s.lower() == "true", default=True)
    parser.add_argument("--delay_grad_averaging", type=lambda s: s.lower() == "true", default=True)
    parser.add_argument("--delay_optimizer_step", type=lambda s: s.lower() == "true", default=True)
    parser.add_argument("--average_state_every", type=int, default=1)
    parser.add_argument("--lr", type=float, default=0.01)
    parser.add_argument("--lr_gamma", type=float, default=0.1)
    parser.add_argument("--lr_step_size", type=int, default=10)
    parser.add_argument("--max_epoch", type=int, default=25)
    parser.add_argument("--batch_size_min", type=int, default=2)
    parser.add_argument("--batch_size_max", type=int, default=16)
    parser.add_argument("--batch_time_min", type=float, default=1.0)
    parser.add_argument("--batch_time_max", type=float, default=4.5)
    parser.add_argument("--batch_time_std", type=float, default=0.5)
    parser.add_argument("--matchmaking_time", type=float, default=5.0)
    parser.add_argument("--max_refresh_period", type=float, default=5.0)
    parser.add_argument("--averaging_timeout", type=float, default=15.0)
    parser.add_argument("--winddown_time", type=float, default=5.0)
    parser.add_argument("--verbose", action="store_true")
    parser.add_argument("--device", default="cpu")
    benchmark_optimizer(parser.parse_args())

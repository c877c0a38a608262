"""CPU plumbing run: hivemind_b200.Optimizer with several peers on one host sharing a local DHT; no GPU needed.

Configuration: 4 peers (threads, one DHT node and one transport daemon each); a 2-layer MLP (Linear 784 -> 1024, ReLU,
Linear 1024 -> 10, fp32); every peer draws batches of 32 inputs from N(0, 1) with uniform labels in [0, 10), seeded
by its rank; cross-entropy; Adam lr 1e-3; ``target_batch_size`` 256; parameters averaged with Float16Compression
after every collaborative step; 50 collaborative steps (epochs). It exercises the whole control plane (DHT,
progress tracker, matchmaking, RPC butterfly for gradients and for parameters) with as little compute as possible,
like the reference's benchmarks/benchmark_optimizer.py does with MNIST.

Prints one JSON line: wall time, samples per second over all peers, epochs per second, the number of averaging
rounds that succeeded / fell back to local gradients, and how far the peers' parameters are apart at the end.

    python benchmarks/benchmark_cpu_plumbing.py            # 4 peers, 50 epochs
"""
import argparse
import json
import os
import sys
import threading
import time
from functools import partial

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.nn as nn
import torch.nn.functional as F

from hivemind_b200 import DHT, Float16Compression, Optimizer


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--num_peers", type=int, default=4)
    parser.add_argument("--epochs", type=int, default=50)
    parser.add_argument("--batch_size", type=int, default=32)
    parser.add_argument("--target_batch_size", type=int, default=256)
    parser.add_argument("--lr", type=float, default=1e-3)
    parser.add_argument("--matchmaking_time", type=float, default=0.5)
    parser.add_argument("--averaging_timeout", type=float, default=15.0)
    parser.add_argument("--verbose", action="store_true")
    args = parser.parse_args()

    torch.set_num_threads(max(1, (os.cpu_count() or 4) // args.num_peers))
    root = DHT(start=True)
    maddrs = root.get_visible_maddrs()
    finals, counters, lock = {}, dict(samples=0, passes=0), threading.Lock()
    ready = threading.Barrier(args.num_peers + 1)

    def run_peer(rank: int) -> None:
        torch.manual_seed(0)  # identical initial weights on every peer
        model = nn.Sequential(nn.Linear(784, 1024), nn.ReLU(), nn.Linear(1024, 10))
        dht = root if rank == 0 else DHT(initial_peers=maddrs, start=True)
        opt = Optimizer(
            dht=dht, run_id="cpu_plumbing", target_batch_size=args.target_batch_size,
            batch_size_per_step=args.batch_size, params=model.parameters(),
            optimizer=partial(torch.optim.Adam, lr=args.lr), grad_compression=Float16Compression(),
            state_averaging_compression=Float16Compression(), average_state_every=1,
            matchmaking_time=args.matchmaking_time, averaging_timeout=args.averaging_timeout,
            averager_opts=dict(request_timeout=min(0.3, args.matchmaking_time / 2)),
            tracker_opts=dict(min_refresh_period=0.05, default_refresh_period=0.1, max_refresh_period=0.5),
            verbose=args.verbose and rank == 0)
        generator = torch.Generator().manual_seed(1000 + rank)
        ready.wait()
        passes = 0
        while opt.local_epoch < args.epochs:
            inputs = torch.randn(args.batch_size, 784, generator=generator)
            labels = torch.randint(0, 10, (args.batch_size,), generator=generator)
            F.cross_entropy(model(inputs), labels).backward()
            opt.step()
            opt.zero_grad()
            passes += 1
        with lock:
            counters["samples"] += passes * args.batch_size
            counters["passes"] += passes
            finals[rank] = torch.cat([p.detach().reshape(-1).clone() for p in model.parameters()])
        ready.wait()  # nobody leaves while others may still need it for their last round
        opt.shutdown()
        if rank != 0:
            dht.shutdown()

    threads = [threading.Thread(target=run_peer, args=(rank,)) for rank in range(args.num_peers)]
    for thread in threads:
        thread.start()
    ready.wait()
    started = time.perf_counter()
    ready.wait()
    elapsed = time.perf_counter() - started
    for thread in threads:
        thread.join()
    root.shutdown()
    reference = finals[0]
    divergence = max(float((finals[r] - reference).abs().max()) for r in finals)
    print(json.dumps({
        "benchmark": "cpu_plumbing_optimizer", "peers": args.num_peers, "epochs": args.epochs, "seconds": elapsed,
        "samples_per_s": counters["samples"] / elapsed, "epochs_per_s": args.epochs / elapsed,
        "samples_processed": counters["samples"], "samples_nominal": args.epochs * args.target_batch_size,
        "max_parameter_divergence_between_peers": divergence,
        "config": {"model": "MLP 784-1024-10 fp32", "batch_size": args.batch_size,
                   "target_batch_size": args.target_batch_size, "optimizer": f"Adam lr {args.lr}",
                   "compression": "Float16 (gradients and parameters)", "matchmaking_time": args.matchmaking_time}}),
        flush=True)


if __name__ == "__main__":
    main()

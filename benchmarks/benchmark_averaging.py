"""Averaging benchmarks.

``--mode swarm`` (default) is the reference's benchmarks/benchmark_averaging.py: ``num_peers`` averagers (threads of
this process, CPU tensors shaped like a small transformer) find groups of ``target_group_size`` through the DHT for
``num_rounds`` rounds; the result is the success rate and the wall time.

``--mode device`` measures the device butterfly all-reduce between GPUs of one box, one process per GPU under
``torchrun`` (peer arenas mapped through CUDA IPC): for each tensor size and codec it times whole rounds (encode,
publish, pull + reduce, delta encode, pull + apply) with CUDA events on the round's stream, takes the max over ranks
and reports the bus bandwidth ``2 (n - 1) / n * bytes / time`` next to NCCL's all_reduce of the same fp32 tensor.
With one GPU, ``--emulate-ranks N`` runs an N-rank group stage by stage on that GPU (no NVLink traffic: it measures
the kernels only).
"""
import argparse
import json
import math
import os
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import numpy as np
import torch

from hivemind_b200 import DHT, DecentralizedAverager
from hivemind_b200.compression import (BlockwiseQuantization, CompressionInfo, Float16Compression, NoCompression,
                                       Quantile8BitQuantization, ScaledFloat16Compression, Uniform8BitQuantization)
from hivemind_b200.utils.limits import increase_file_limit
from hivemind_b200.utils.logging import get_logger

logger = get_logger(__name__)
CODECS = {"none": NoCompression, "float16": Float16Compression, "meanstd16": ScaledFloat16Compression,
          "uniform8": Uniform8BitQuantization, "quantile8": Quantile8BitQuantization, "blockwise8": BlockwiseQuantization}


def sample_tensors(hid_size, num_layers):
    tensors = []
    for _ in range(num_layers):
        tensors += [torch.randn(hid_size, 3 * hid_size), torch.randn(3 * hid_size), torch.randn(3 * hid_size),
                    torch.randn(hid_size, hid_size), torch.ones(hid_size), torch.zeros(hid_size),
                    torch.randn(hid_size, 4 * hid_size), torch.randn(4 * hid_size), torch.ones(4 * hid_size),
                    torch.randn(2, hid_size, hid_size, 2), torch.randn(hid_size), torch.randn(hid_size),
                    torch.randn(hid_size)]
    return tuple(tensors)


def benchmark_swarm(num_peers, target_group_size, num_rounds, min_matchmaking_time, request_timeout, round_timeout,
                    hid_size, num_layers, spawn_dtime):
    dht_root = DHT(start=True)
    initial_peers = dht_root.get_visible_maddrs()
    num_groups = 2 ** int(round(math.log2(num_peers / target_group_size)))
    nbits = int(round(math.log2(num_groups)))
    peer_tensors = [sample_tensors(hid_size, num_layers) for _ in range(num_peers)]
    to_close = [dht_root]
    lock = threading.Lock()
    stats = dict(ok=0, total=0)

    def run_averager(index):
        dht = DHT(initial_peers=initial_peers, start=True)
        bits = bin(index % num_groups)[2:].rjust(nbits, "0") if nbits else ""
        averager = DecentralizedAverager(peer_tensors[index], dht, prefix="my_tensor", initial_group_bits=bits,
                                         compression=Float16Compression(), target_group_size=target_group_size,
                                         min_matchmaking_time=min_matchmaking_time, request_timeout=request_timeout,
                                         start=True)
        with lock:
            to_close.extend([averager, dht])
        for step in range(num_rounds):
            reason = ""
            try:
                success = averager.step(timeout=round_timeout) is not None
            except Exception as e:
                success, reason = False, f" ({e!r})"
            with lock:
                stats["ok"] += int(success)
                stats["total"] += 1
            logger.info(f"Averager {index}: {'finished' if success else 'failed'} step #{step}{reason}")

    threads = []
    for i in range(num_peers):
        thread = threading.Thread(target=run_averager, args=[i])
        threads.append(thread)
        thread.start()
        time.sleep(spawn_dtime)
    started = time.time()
    for thread in threads:
        thread.join()
    elapsed = time.time() - started
    print(json.dumps({"benchmark": "averaging_swarm", "success_rate": stats["ok"] / max(stats["total"], 1),
                      "successful_steps": stats["ok"], "total_steps": stats["total"], "seconds": elapsed,
                      "config": dict(num_peers=num_peers, target_group_size=target_group_size, num_rounds=num_rounds,
                                     hid_size=hid_size, num_layers=num_layers)}), flush=True)
    for item in reversed(to_close):
        item.shutdown()


def _rpc_payload_peer(maddrs, numel, codec_name, rounds, part_size_bytes, min_matchmaking_time, num_peers, ready, go):
    """Body of a helper process of ``benchmark_rpc_payload``: one averager that steps whenever it is told to."""
    torch.set_num_threads(2)
    dht = DHT(initial_peers=maddrs, start=True)
    averager = DecentralizedAverager([torch.randn(numel)], dht, prefix="rpc_payload", target_group_size=num_peers,
                                     min_matchmaking_time=min_matchmaking_time, compression=CODECS[codec_name](),
                                     start=True, part_size_bytes=part_size_bytes)
    ready.put(True)
    for _ in range(rounds):
        go.get()
        averager.step(timeout=600)
    ready.put(True)
    averager.shutdown()
    dht.shutdown()


def benchmark_rpc_payload_processes(num_peers, size_mb, codec_name, rounds, part_size_bytes, min_matchmaking_time):
    """Like ``benchmark_rpc_payload`` with every peer but the first in a process of its own (no shared interpreter
    lock, as in a real swarm); the first peer's ``step()`` is timed."""
    import multiprocessing as mp

    numel = int(size_mb * 1e6 / 4)
    torch.set_num_threads(2)
    root = DHT(start=True)
    ctx = mp.get_context("spawn")
    ready, go = ctx.Queue(), ctx.Queue()
    maddrs = [str(m) for m in root.get_visible_maddrs()]
    helpers = [ctx.Process(target=_rpc_payload_peer, daemon=True,
                           args=(maddrs, numel, codec_name, rounds, part_size_bytes, min_matchmaking_time, num_peers, ready, go))
               for _ in range(num_peers - 1)]
    for helper in helpers:
        helper.start()
    averager = DecentralizedAverager([torch.randn(numel)], root, prefix="rpc_payload", target_group_size=num_peers,
                                     min_matchmaking_time=min_matchmaking_time, compression=CODECS[codec_name](),
                                     start=True, part_size_bytes=part_size_bytes)
    for _ in helpers:
        ready.get()
    best = None
    for _ in range(rounds):
        for _ in helpers:
            go.put(True)
        started = time.perf_counter()
        averager.step(timeout=600)
        elapsed = time.perf_counter() - started
        best = elapsed if best is None else min(best, elapsed)
    for helper in helpers:
        ready.get()
        helper.join(timeout=30)
    averager.shutdown()
    root.shutdown()
    print(json.dumps({"benchmark": "averaging_rpc_payload", "peers": num_peers, "processes": num_peers,
                      "payload_mb_per_peer": size_mb, "codec": codec_name, "part_size_bytes": part_size_bytes,
                      "seconds_per_round": best, "payload_mb_per_s_per_peer": size_mb / best}), flush=True)


def benchmark_rpc_payload(num_peers, size_mb, codec_name, rounds, part_size_bytes, min_matchmaking_time):
    """Throughput of the RPC butterfly on CPU tensors: ``num_peers`` averagers of this process (one DHT node and one
    transport daemon each) average one tensor of ``size_mb`` megabytes; a round is timed from ``step()`` to the last
    peer's result, so it contains the time to form the group (a full group closes at once, well before
    ``min_matchmaking_time``). Prints one JSON line per codec with the best round."""
    codec = CODECS[codec_name]()
    numel = int(size_mb * 1e6 / 4)
    root = DHT(start=True)
    dhts = [root] + [DHT(initial_peers=root.get_visible_maddrs(), start=True) for _ in range(num_peers - 1)]
    averagers = [DecentralizedAverager([torch.randn(numel)], dht, prefix="rpc_payload", target_group_size=num_peers,
                                       min_matchmaking_time=min_matchmaking_time, compression=codec, start=True,
                                       part_size_bytes=part_size_bytes) for dht in dhts]
    expected = sum(a._averaged_tensors[0][:1000].clone() for a in averagers) / num_peers
    best = None
    try:
        for _ in range(rounds):
            started, cpu_started = time.perf_counter(), time.process_time()
            controls = [averager.step(wait=False, timeout=600) for averager in averagers]
            for control in controls:
                control.result()
            elapsed, cpu = time.perf_counter() - started, time.process_time() - cpu_started
            if best is None or elapsed < best[0]:
                best = (elapsed, cpu)
        error = max(float((a._averaged_tensors[0][:1000] - expected).abs().max()) for a in averagers)
    finally:
        for item in averagers + dhts:
            item.shutdown()
    print(json.dumps({"benchmark": "averaging_rpc_payload", "peers": num_peers, "processes": 1,
                      "payload_mb_per_peer": size_mb, "codec": codec_name, "part_size_bytes": part_size_bytes,
                      "seconds_per_round": best[0], "payload_mb_per_s_per_peer": size_mb / best[0],
                      "process_cpu_seconds": best[1], "max_abs_error_vs_mean": error}), flush=True)


VERBOSE_ROUNDS = False
TRACE_ROUND = False


def _print_round_trace(endpoint, kwargs, label, rank):
    """One more round with the kernel's per-CTA time stamps switched on; prints, per rank, when (microseconds after the
    first CTA of this GPU started, median and maximum over CTAs) the CTAs entered their first reduce item, knew about
    its flags, left it, entered their first apply item, knew about its flag, left it, and finished."""
    trace = endpoint.enable_trace()
    with torch.cuda.stream(torch.cuda.ExternalStream(endpoint.stream.value, device=endpoint.device)):
        trace.zero_()
        endpoint.tensor_views[0].normal_()
    endpoint.run_round(group_id=f"trace-{label}".encode(), **kwargs)
    stamps = trace.cpu().numpy().astype("float64")
    started = stamps[:, 0][stamps[:, 0] > 0]
    if len(started) == 0:
        return
    origin = started.min()
    names = {1: "reduce entered", 8: "reduce flags known", 2: "first reduce item left", 3: "last reduce item left",
             4: "apply entered", 9: "apply flag known", 5: "first apply item left", 6: "last item left"}
    row = {}
    for column, name in names.items():
        values = stamps[:, column][stamps[:, column] > 0]
        if len(values):
            rel = (values - origin) / 1e3
            row[name] = [round(float(np.median(rel)), 1), round(float(rel.max()), 1)]
    print(json.dumps({"trace": label, "rank": rank, "ctas": int(len(started)), "items_per_cta_max": int(stamps[:, 7].max()),
                      "us_after_start_median_max": row}), flush=True)


def _time_rounds(endpoint, plan_args, rounds, warmup):
    """Device time per round on the endpoint's stream (ms), with a fresh group id (epoch) every round.

    All rounds are enqueued back to back without waiting on the host (like the NCCL column, which times consecutive
    ``all_reduce`` calls): the gate kernel in front of every round keeps the ranks in step on the device. Returns the
    mean time from the launch of a round's gate kernel to the end of its round kernel, and the mean duration of each
    launch by name (the gate's share is mostly waiting for the slowest rank)."""
    stream = torch.cuda.ExternalStream(endpoint.stream.value, device=endpoint.device)
    all_marks = []
    if plan_args["barrier"] is not None:
        plan_args["barrier"]()
    # the host needs longer to prepare a small round than the device needs to run it: a few milliseconds of busy-waiting
    # at the head of the stream let the launches queue up, so that what is timed is the device, not Python
    with torch.cuda.stream(stream):
        torch.cuda._sleep(20_000_000)
    for i in range(warmup + rounds):
        # fresh values every round: repeated averaging of the same tensors converges, and the deltas of converged
        # peers are an unrepresentative (degenerate) input for the quantising codecs
        with torch.cuda.stream(stream):
            endpoint.tensor_views[0].normal_()
        marks = []

        def mark(name, marks=marks):
            marks.append((name, torch.cuda.Event(enable_timing=True)))
            marks[-1][1].record(stream)

        endpoint.launch_hook = mark
        mark("start")
        endpoint.run_round(group_id=f"bench-{plan_args['tag']}-{i}".encode(), wait=False, **plan_args["kwargs"])
        endpoint.launch_hook = None
        all_marks.append(marks)
    status = endpoint.wait_round()
    if status.banned_senders or status.failed_reducers:
        raise RuntimeError(f"round failed: {status.banned_senders} {status.failed_reducers}")
    times, per_launch = [], {}
    for i, marks in enumerate(all_marks):
        if i >= warmup:
            times.append(marks[0][1].elapsed_time(marks[-1][1]))
            for (_, before), (name, after) in zip(marks, marks[1:]):
                per_launch.setdefault(name, []).append(before.elapsed_time(after))
        if plan_args.get("verbose"):  # warm-up rounds too
            print(f"rank {plan_args['kwargs']['my_index']} {plan_args['tag']} round {i}: " + " ".join(
                f"{name}={before.elapsed_time(after) * 1e3:.0f}us"
                for (_, before), (name, after) in zip(marks, marks[1:])), flush=True)
    stages = {name + "_ms": sum(v) / len(v) for name, v in per_launch.items()}
    return sum(times) / len(times), stages


def benchmark_device(sizes_mb, codecs, rounds, warmup, emulate_ranks, part_size_bytes):
    import torch.distributed as dist
    from hivemind_b200.averaging.allreduce import AveragingMode
    from hivemind_b200.parallel.device_butterfly import DeviceEndpoint, run_group_emulated

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    results = []
    for size_mb in sizes_mb:
        numel = int(size_mb * 2 ** 20 / 4)
        nccl_ms = None
        if world > 1:
            buf = torch.randn(numel, device=device)
            for _ in range(warmup):
                dist.all_reduce(buf)
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            dist.barrier()
            start.record()
            for _ in range(rounds):
                dist.all_reduce(buf)
            stop.record()
            torch.cuda.synchronize()
            t = torch.tensor([start.elapsed_time(stop) / rounds], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            nccl_ms = float(t)
            del buf
        for codec_name in codecs:
            codec = CODECS[codec_name]()
            if world > 1:
                tensor = torch.randn(numel, device=device)
                endpoint = DeviceEndpoint([tensor], codec, [CompressionInfo.from_tensor(tensor, key=0)], part_size_bytes)
                infos = [None] * world
                dist.all_gather_object(infos, endpoint.describe())
                n = world
                my_weight = 0.5 + 1.5 * ((rank * 0.37 + 0.11) % 1.0)  # per-peer weights spread over [0.5, 2)
                kwargs = dict(my_index=rank, device_infos=infos, modes=[AveragingMode.NODE] * n,
                              peer_fractions=[1.0 / n] * n, weight=my_weight, alpha=1.0, sender_timeout=10.0,
                              reducer_timeout=20.0)
                ms, stages = _time_rounds(endpoint, dict(tag=f"{size_mb}-{codec_name}", kwargs=kwargs,
                                                         barrier=dist.barrier, verbose=VERBOSE_ROUNDS), rounds, warmup)
                t = torch.tensor([ms] + list(stages.values()), device=device)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t[0])
                stages = {name: float(v) for name, v in zip(stages, t[1:])}
                dist.barrier()
                if TRACE_ROUND:
                    _print_round_trace(endpoint, kwargs, f"{size_mb} MB {codec_name}", rank)
                    dist.barrier()
                endpoint.close()
            else:
                n = emulate_ranks
                endpoints = []
                for r in range(n):
                    tensor = torch.randn(numel, device=device)
                    endpoints.append(DeviceEndpoint([tensor], codec, [CompressionInfo.from_tensor(tensor, key=0)],
                                                    part_size_bytes))
                for i in range(warmup):
                    run_group_emulated(endpoints, weights=[1.0] * n, peer_fractions=[1.0 / n] * n,
                                       group_id=f"w{size_mb}{codec_name}{i}".encode())
                torch.cuda.synchronize()
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                total_ms, stage_ms = 0.0, {}
                for i in range(rounds):
                    for e in endpoints:
                        e.tensor_views[0].normal_()  # fresh values every round (see _time_rounds)
                    marks = []

                    def mark(name, marks=marks):  # rank 0's launches: device time of each stage kernel by itself
                        marks.append((name, torch.cuda.Event(enable_timing=True)))
                        marks[-1][1].record()

                    endpoints[0].launch_hook = mark
                    start.record()
                    run_group_emulated(endpoints, weights=[1.0] * n, peer_fractions=[1.0 / n] * n,
                                       group_id=f"t{size_mb}{codec_name}{i}".encode())
                    stop.record()
                    torch.cuda.synchronize()
                    endpoints[0].launch_hook = None
                    total_ms += start.elapsed_time(stop)
                    previous = start
                    for name, event in marks:
                        stage_ms.setdefault(name + "_ms", []).append(previous.elapsed_time(event))
                        previous = event
                ms = total_ms / rounds / n  # n ranks share one GPU: per-rank share of the time
                for e in endpoints:
                    e.close()
                # time from the previous mark to the end of each of rank 0's launches; "send" follows the round's
                # start directly, "reduce" and "apply" also contain the other ranks' launches of the stage before
                stages = {name: sum(v) / len(v) for name, v in stage_ms.items()}
            nbytes = numel * 4
            bus = 2 * (n - 1) / n * nbytes / (ms / 1e3) / 1e9
            row = {"size_mb": size_mb, "codec": codec_name, "n_ranks": n, "ms_per_round": ms, "bus_gb_s": bus,
                   "algo_gb_s": nbytes / (ms / 1e3) / 1e9}
            if stages is not None:
                row["launches_max_over_ranks"] = stages
            if nccl_ms is not None:
                row["nccl_fp32_ms"] = nccl_ms
                row["nccl_fp32_bus_gb_s"] = 2 * (n - 1) / n * nbytes / (nccl_ms / 1e3) / 1e9
            results.append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)
    if rank == 0:
        print(json.dumps({"benchmark": "averaging_device_butterfly", "emulated": world == 1, "n_gpus": world,
                          "rounds": rounds, "warmup": warmup, "part_size_bytes": part_size_bytes, "rows": results}),
              flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--mode", choices=["swarm", "device", "rpc_payload"], default="swarm")
    parser.add_argument("--num_peers", type=int, default=16)
    parser.add_argument("--target_group_size", type=int, default=4)
    parser.add_argument("--num_rounds", type=int, default=5)
    parser.add_argument("--hid_size", type=int, default=256)
    parser.add_argument("--num_layers", type=int, default=3)
    parser.add_argument("--min_matchmaking_time", type=float, default=5)
    parser.add_argument("--round_timeout", type=float, default=15)
    parser.add_argument("--request_timeout", type=float, default=1)
    parser.add_argument("--spawn_dtime", type=float, default=0.1)
    parser.add_argument("--increase_file_limit", action="store_true")
    parser.add_argument("--sizes-mb", type=float, nargs="+", default=[1, 16, 64, 256])
    parser.add_argument("--codecs", nargs="+", default=["none", "float16", "uniform8"], choices=sorted(CODECS))
    parser.add_argument("--rounds", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--emulate-ranks", type=int, default=4)
    parser.add_argument("--part-size-bytes", type=int, default=2 ** 19)
    parser.add_argument("--peer-processes", action="store_true",
                        help="rpc_payload mode: every peer in a process of its own instead of threads of this one")
    parser.add_argument("--verbose-rounds", action="store_true", help="print every launch of every timed round")
    parser.add_argument("--trace-round", action="store_true",
                        help="device mode with several GPUs: after the timed rounds, one round with per-CTA time stamps")
    args = parser.parse_args()
    VERBOSE_ROUNDS = args.verbose_rounds
    TRACE_ROUND = args.trace_round
    if args.increase_file_limit:
        increase_file_limit()
    if args.mode == "rpc_payload":
        for size_mb in args.sizes_mb:
            for codec_name in args.codecs:
                run = benchmark_rpc_payload_processes if args.peer_processes else benchmark_rpc_payload
                run(args.num_peers, size_mb, codec_name, args.rounds, args.part_size_bytes, 0.5)
    elif args.mode == "device":
        benchmark_device(args.sizes_mb, args.codecs, args.rounds, args.warmup, args.emulate_ranks, args.part_size_bytes)
    else:
        benchmark_swarm(args.num_peers, args.target_group_size, args.num_rounds, args.min_matchmaking_time,
                        args.request_timeout, args.round_timeout, args.hid_size, args.num_layers, args.spawn_dtime)

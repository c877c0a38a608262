"""Mixture-of-experts throughput.

``--mode server`` measures what the reference's benchmarks/benchmark_throughput.py measures: one server with
``num_experts`` ``ffn`` experts on one device, ``num_clients`` clients that each send ``num_batches_per_client``
batches of ``batch_size`` rows to random experts over RPC (forward, and backward unless ``--no-backprop``);
the result is examples / second between "server ready" and "all clients finished". Clients are threads spread over
``--client-processes`` processes (each process has its own transport daemon).

``--mode device`` measures the device path: ``DeviceMixtureOfExperts`` (gate top-k kernel, dispatch, tcgen05 expert
GEMMs, combine) on tokens that are already on the GPU, forward + backward, timed with CUDA events; under
``torchrun`` the experts are sharded over the ranks and every rank is a client with its own tokens.

Prints one JSON line with the configuration and samples (tokens) per second.
"""
import argparse
import json
import multiprocessing as mp
import os
import random
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from hivemind_b200.dht import DHT
from hivemind_b200.moe.client.expert import RemoteExpert
from hivemind_b200.moe.client.remote_expert_worker import RemoteExpertWorker
from hivemind_b200.moe.expert_uid import ExpertInfo
from hivemind_b200.moe.server import ModuleBackend, Server
from hivemind_b200.moe.server.layers import name_to_block
from hivemind_b200.p2p import P2P
from hivemind_b200.utils.limits import increase_file_limit
from hivemind_b200.utils.logging import get_logger
from hivemind_b200.utils.tensor_descr import BatchTensorDescriptor

logger = get_logger(__name__)


def _client_process(ready, can_start, failed, server_maddrs, server_peer_id, num_experts, batch_size, hid_dim, num_batches,
                    backprop, num_threads):
    torch.set_num_threads(1)
    p2p = RemoteExpertWorker.run_coroutine(P2P.create(initial_peers=server_maddrs))
    experts = [RemoteExpert(ExpertInfo(uid=f"expert.{i}", peer_id=server_peer_id), p2p) for i in range(num_experts)]
    for attempt in range(120):  # fetch the schema once before the clock starts; the server may still be starting
        try:
            experts[0].info
            break
        except Exception:
            time.sleep(0.5)
    for expert in experts[1:]:
        expert._rpc_info = experts[0]._rpc_info

    def client():
        try:
            batch = torch.randn(batch_size, hid_dim)
            for _ in range(num_batches):
                out = random.choice(experts)(batch)
                if backprop:
                    out.sum().backward()
        except BaseException:
            failed.set()
            raise

    ready.wait()
    can_start.wait()
    threads = [threading.Thread(target=client) for _ in range(num_threads)]
    for thread in threads:
        thread.start()
    for thread in threads:
        thread.join()


def benchmark_server(num_experts=16, num_handlers=None, num_clients=128, num_batches_per_client=16, expert_cls="ffn",
                     hid_dim=1024, batch_size=2048, max_batch_size=None, backprop=True, device=None,
                     client_processes=8):
    assert expert_cls in name_to_block
    max_batch_size = max_batch_size or batch_size * 4
    num_handlers = max(1, num_handlers or min(num_clients // 2, 16))
    client_processes = max(1, min(client_processes, num_clients))
    ctx = mp.get_context("spawn")
    failed, can_start = ctx.Event(), ctx.Event()
    stamps = dict(started=time.perf_counter())
    server_dht = DHT(start=True)
    threads_per_process = [num_clients // client_processes + (i < num_clients % client_processes)
                           for i in range(client_processes)]
    ready = ctx.Barrier(sum(1 for n in threads_per_process if n > 0) + 1)
    clients = [ctx.Process(target=_client_process, daemon=True,
                           args=(ready, can_start, failed, server_dht.get_visible_maddrs(), server_dht.peer_id, num_experts,
                                 batch_size, hid_dim, num_batches_per_client, backprop, n))
               for n in threads_per_process if n > 0]
    for client in clients:
        client.start()
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    backends = {}
    for i in range(num_experts):
        expert = name_to_block[expert_cls](hid_dim)
        backends[f"expert.{i}"] = ModuleBackend(
            name=f"expert.{i}", module=expert, optimizer=torch.optim.Adam(expert.parameters()),
            args_schema=(BatchTensorDescriptor(hid_dim),), outputs_schema=BatchTensorDescriptor(hid_dim),
            max_batch_size=max_batch_size)
    stamps["created_experts"] = time.perf_counter()
    server = Server(dht=server_dht, module_backends=backends, num_connection_handlers=num_handlers, device=device)
    try:
        server.start()
        if not server.ready.wait(timeout=300):
            raise TimeoutError("the server did not become ready")
        ready.wait(timeout=300)  # every client process has imported, connected and fetched the schema
        stamps["server_ready"] = time.perf_counter()
        can_start.set()
        for client in clients:
            client.join()
        stamps["clients_finished"] = time.perf_counter()
    finally:
        for client in clients:
            if client.is_alive():
                client.terminate()
        server.shutdown()
    total = batch_size * num_clients * num_batches_per_client
    elapsed = stamps["clients_finished"] - stamps["server_ready"]
    result = {"benchmark": "moe_server_throughput", "passes": "forward+backward" if backprop else "forward",
              "samples_per_s": total / elapsed, "examples": total, "seconds": elapsed, "failed": failed.is_set(),
              "config": dict(num_experts=num_experts, num_handlers=num_handlers, num_clients=num_clients,
                             client_processes=len(clients), num_batches_per_client=num_batches_per_client,
                             batch_size=batch_size, max_batch_size=max_batch_size, expert_cls=expert_cls,
                             hid_dim=hid_dim, device=str(device))}
    print(json.dumps(result), flush=True)
    assert not failed.is_set()
    return result


def benchmark_device(grid=(8, 8), k_best=4, tokens=4096, hid_dim=1024, steps=20, warmup=5, switch=False,
                     backprop=True, exchange="all_to_all"):
    import torch.distributed as dist
    from hivemind_b200.ops import _lib
    from hivemind_b200.parallel.expert_parallel import DeviceMixtureOfExperts

    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        group = dist.group.WORLD
    torch.manual_seed(1234 + local_rank)
    layer = DeviceMixtureOfExperts(in_features=hid_dim, grid_size=grid, k_best=1 if switch else k_best, switch=switch,
                                   group=group, exchange=exchange, max_tokens=tokens).cuda()
    optimizer = torch.optim.Adam(layer.parameters(), lr=1e-4, fused=True)
    x = torch.randn(tokens, hid_dim, device="cuda", dtype=torch.bfloat16, requires_grad=True)

    def step():
        result = layer(x)
        out = result[0] if switch else result
        if backprop:
            loss = out.float().pow(2).mean() + (result[1] if switch else 0)
            loss.backward()
            optimizer.step()
            optimizer.zero_grad(set_to_none=False)
            x.grad = None

    for _ in range(warmup):
        step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    launches_before = _lib.launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        step()
    stop.record()
    torch.cuda.synchronize()
    elapsed_ms = torch.tensor([start.elapsed_time(stop)], device="cuda")
    if world > 1:
        dist.all_reduce(elapsed_ms, op=dist.ReduceOp.MAX)
    ms = float(elapsed_ms) / steps
    flops_per_row = 2 * 2 * hid_dim * 4 * hid_dim * (3 if backprop else 1)
    rows = tokens * layer.k_best * world
    if local_rank == 0:
        print(json.dumps({"benchmark": "moe_device_layer", "passes": "forward+backward+adam" if backprop else "forward",
                          "tokens_per_s": tokens * world / (ms / 1e3), "ms_per_step": ms, "n_gpus": world,
                          "expert_tflops": rows * flops_per_row / (ms / 1e3) / 1e12,
                          "own_kernel_launches": _lib.launch_count() - launches_before,
                          "config": dict(grid=list(grid), k_best=layer.k_best, tokens_per_gpu=tokens, hid_dim=hid_dim,
                                         switch=switch, steps=steps, warmup=warmup, dtype="bf16",
                                         exchange=exchange if world > 1 else "local")}), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--mode", choices=["server", "device"], default="server")
    parser.add_argument("--preset", default="default")
    parser.add_argument("--num_batches_per_client", type=int, default=16)
    parser.add_argument("--num_clients", type=int, default=None)
    parser.add_argument("--client-processes", type=int, default=8)
    parser.add_argument("--no-backprop", action="store_true")
    parser.add_argument("--switch", action="store_true")
    parser.add_argument("--tokens", type=int, default=4096)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--device", default=None)
    parser.add_argument("--exchange", default="all_to_all", choices=["all_to_all", "peer"],
                        help="device mode with several GPUs: NCCL all-to-all or our kernels over peer-mapped memory")
    args = parser.parse_args()
    if args.mode == "device":
        benchmark_device(tokens=args.tokens, steps=args.steps, switch=args.switch, backprop=not args.no_backprop,
                         exchange=args.exchange)
    else:
        increase_file_limit()
        common = dict(num_batches_per_client=args.num_batches_per_client, device=args.device,
                      client_processes=args.client_processes)
        if args.num_clients is not None:
            common["num_clients"] = args.num_clients
        presets = {
            "default": dict(backprop=not args.no_backprop),
            "ffn_forward_backward": dict(backprop=True),
            "ffn_forward": dict(backprop=False),
            "ffn_small_batch": dict(backprop=False, num_experts=4, batch_size=32, max_batch_size=8192),
            "ffn_small_batch_512clients": dict(backprop=True, num_experts=1, batch_size=1, max_batch_size=8192,
                                               num_clients=512),
            "ffn_massive": dict(backprop=False, num_clients=512, batch_size=512, max_batch_size=8192),
            "minimalistic": dict(num_experts=1, num_clients=1, num_handlers=1),
            "nop": dict(expert_cls="nop", backprop=False),
        }
        if args.preset not in presets:
            raise ValueError(f"No such benchmark preset: {args.preset}")
        benchmark_server(**{**presets[args.preset], **common})

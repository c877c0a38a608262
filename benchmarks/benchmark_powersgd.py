"""GPT-2-medium-shaped causal LM trained under hivemind_b200.Optimizer with PowerSGD gradient averaging.

Workload: 24 layers, d_model 1024, 16 heads, FFN 4096, vocabulary 50257, sequences of 1024 uniform random tokens,
bf16 compute with fp32 master weights, AdamW lr 3e-4, per-GPU batch 8; every GPU is one peer. 2-D weight gradients are
compressed to rank 32 (P = M Q, Q = M^T P, Q initialised from N(0, 1)), 1-D parameters are averaged as they are
(the reference's averager: hivemind/optim/power_sgd_averager.py:28-222).

A *step* is one collaborative optimizer step: ``accumulation`` forward/backward passes per peer, the two-phase
PowerSGD averaging round, and the AdamW update. Timed with CUDA events on the device, maximum over ranks.
``--averager`` selects what averages the gradients:

    powersgd  PowerSGDGradientAverager (P and Q averaged by the device butterfly over peer memory)
    plain     GradientAverager without compression (device butterfly on the full gradients)
    nccl      no hivemind at all: one NCCL all-reduce of the flat gradient + the same fused AdamW (the baseline that
              a data-parallel trainer would run)

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29511 \
        benchmarks/benchmark_powersgd.py --steps 5 --warmup 3
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from functools import partial

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--steps", type=int, default=5)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--averager", default="powersgd", choices=["powersgd", "plain", "nccl"])
    parser.add_argument("--rank-r", type=int, default=32, help="rank of the PowerSGD approximation")
    parser.add_argument("--batch", type=int, default=8, help="per-GPU batch of one forward/backward pass")
    parser.add_argument("--seq-len", type=int, default=1024)
    parser.add_argument("--accumulation", type=int, default=1, help="forward/backward passes per peer and step")
    parser.add_argument("--model", default="medium", choices=["medium", "small", "tiny"])
    args = parser.parse_args()

    import torch
    import torch.distributed as dist

    import hivemind_b200 as hivemind
    from hivemind_b200.models.gpt2 import GPT2Config, GPT2LMHeadModel, make_lm_batch
    from hivemind_b200.ops import _lib
    from hivemind_b200.ops.gemm import check_kernel_errors
    from hivemind_b200.optim import PowerSGDGradientAverager
    from hivemind_b200.optim.fused import FusedAdamW

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available()  # without a GPU the script still runs (tiny model, host timers)
    if use_cuda:
        torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank) if use_cuda else torch.device("cpu")
    host_group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if use_cuda:
            dist.init_process_group("nccl", device_id=device)
        else:
            dist.init_process_group("gloo")
        host_group = dist.new_group(backend="gloo")  # host-side barriers: no collective kernels between rounds

    class Stopwatch:
        """CUDA events on the current stream (host clock without a GPU)."""

        def start(self):
            if use_cuda:
                self.events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                self.events[0].record()
            self.t0 = time.perf_counter()

        def stop(self):
            if use_cuda:
                self.events[1].record()
            self.t1 = time.perf_counter()

        def milliseconds(self) -> float:
            if use_cuda:
                self.events[1].synchronize()
                return self.events[0].elapsed_time(self.events[1])
            return (self.t1 - self.t0) * 1e3

    torch.manual_seed(1234)
    cfg = getattr(GPT2Config, args.model)()
    seq_len = min(args.seq_len, cfg.n_positions)
    model = GPT2LMHeadModel(cfg).to(device)
    params = list(model.parameters())
    samples_per_step = args.batch * args.accumulation * world

    opt = dht = None
    if args.averager == "nccl":
        for p in params:
            p.grad = torch.zeros_like(p)
        inner = FusedAdamW(params, lr=3e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    else:
        if rank == 0:
            dht = hivemind.DHT(start=True)
            maddrs = [str(m) for m in dht.get_visible_maddrs()]
        else:
            maddrs = None
        if world > 1:
            box = [maddrs]
            dist.broadcast_object_list(box, src=0, group=host_group)
            if rank != 0:
                dht = hivemind.DHT(initial_peers=box[0], start=True)
        factory = None
        if args.averager == "powersgd":
            factory = partial(PowerSGDGradientAverager, averager_rank=args.rank_r, q_init="normal")
        opt = hivemind.Optimizer(
            dht=dht, run_id="gpt2_powersgd_bench", target_batch_size=samples_per_step,
            batch_size_per_step=args.batch, params=params,
            optimizer=lambda ps: FusedAdamW(ps, lr=3e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01),
            grad_averager_factory=factory, grad_compression=hivemind.NoCompression(),
            state_averaging_compression=hivemind.Float16Compression(), reuse_grad_buffers=True,
            offload_optimizer=True, delay_optimizer_step=False, delay_grad_averaging=False,
            matchmaking_time=0.5, averaging_timeout=30.0, next_chunk_timeout=5.0, average_state_every=10 ** 9,
            averager_opts=dict(request_timeout=0.5, target_group_size=world if world > 1 else None),
            tracker_opts=dict(min_refresh_period=0.02, default_refresh_period=0.05, max_refresh_period=0.2),
            verbose=False)

    gen = torch.Generator().manual_seed(1000 + rank)
    pool = [{k: v.to(device) for k, v in make_lm_batch(cfg, args.batch, seq_len, generator=gen).items()}
            for _ in range(4)]

    def barrier():
        if use_cuda:
            torch.cuda.synchronize()
        if world > 1:
            dist.barrier(group=host_group)

    def nccl_step(i: int):
        for a in range(args.accumulation):
            batch = pool[(i * args.accumulation + a) % len(pool)]
            loss = model(batch["input_ids"], batch["labels"])
            loss.backward()
        grads = [p.grad for p in params]
        if world > 1:
            flat = torch.cat([g.reshape(-1) for g in grads])
            dist.all_reduce(flat)
            flat.div_(world * args.accumulation)
            offset = 0
            for g in grads:
                g.copy_(flat[offset:offset + g.numel()].view_as(g))
                offset += g.numel()
        inner.step()
        for g in grads:
            g.zero_()
        return loss

    def run_steps(num_steps: int):
        """Run forward/backward passes until ``num_steps`` more collaborative steps are done; returns passes run."""
        passes, loss = 0, None
        if opt is None:
            for i in range(num_steps):
                loss = nccl_step(i)
            return num_steps * args.accumulation, loss
        target_epoch = opt.local_epoch + num_steps
        while opt.local_epoch < target_epoch:
            batch = pool[passes % len(pool)]
            loss = model(batch["input_ids"], batch["labels"])
            loss.backward()
            opt.step()
            passes += 1
        return passes, loss

    def timed(num_steps: int):
        barrier()
        launches0 = _lib.launch_count()
        watch = Stopwatch()
        wall0 = time.perf_counter()
        watch.start()
        passes, loss = run_steps(num_steps)
        watch.stop()
        barrier()
        wall = time.perf_counter() - wall0
        ms = torch.tensor([watch.milliseconds()], dtype=torch.float64)
        samples = torch.tensor([float(passes * args.batch)], dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX, group=host_group)
            dist.all_reduce(samples, op=dist.ReduceOp.SUM, group=host_group)
        return float(ms.item()), float(samples.item()), _lib.launch_count() - launches0, float(loss.item()), wall

    # forward/backward alone (no optimizer, no averaging): the ceiling that averaging overhead is judged against
    for _ in range(2):
        model(pool[0]["input_ids"], pool[0]["labels"]).backward()
    barrier()
    watch = Stopwatch()
    watch.start()
    for i in range(4):
        model(pool[i % len(pool)]["input_ids"], pool[i % len(pool)]["labels"]).backward()
    watch.stop()
    fwd_bwd_ms = watch.milliseconds() / 4
    for p in params:
        if p.grad is not None:
            p.grad.zero_()

    run_steps(max(3, args.warmup))
    ms, samples, launches, last_loss, wall = timed(args.steps)
    check_kernel_errors()
    n_params = sum(p.numel() for p in params)
    compressed_elems = None
    if opt is not None and args.averager == "powersgd":
        ga = opt.grad_averager
        compressed_elems = int(sum(p.numel() for p in ga._ps) + sum(q.numel() for q in ga._qs) + sum(
            g.numel() for i, g in enumerate(ga._averaged_tensors) if i in ga._uncompressed_gradients_indexes))
    if rank == 0:
        value = samples / (ms / 1e3)
        print(json.dumps({
            "metric": f"Optimizer samples/s (GPT-2-{args.model}, {args.averager} gradient averaging)",
            "value": value, "unit": "samples/s", "tokens_per_s": value * seq_len, "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms / args.steps,
            "wall_ms_per_step": wall * 1e3 / args.steps, "forward_backward_ms_per_pass": fwd_bwd_ms,
            "samples_in_timed_region": samples, "gpu_launches": launches, "last_loss": last_loss, "dtype": "bf16" if use_cuda else "fp32",
            "data": "synthetic", "parameters": n_params, "averaged_elements_per_round": compressed_elems or n_params,
            "config": {"model": f"gpt2-{args.model}", "per_gpu_batch": args.batch, "seq_len": seq_len,
                       "accumulation": args.accumulation, "optimizer": "AdamW lr 3e-4", "powersgd_rank": args.rank_r,
                       "parallelism": f"dp{world}"}}))
    if opt is not None:
        opt.shutdown()
        dht.shutdown()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

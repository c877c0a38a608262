"""Headline benchmark: hivemind_b200.Optimizer samples/s on the ALBERT-large-shaped masked-LM workload.

Workload (the reference's ALBERT example, examples/albert/arguments.py:75-135 and run_trainer.py:240-285):
ALBERT-large (24 shared layers, hidden 1024, 16 heads, FFN 4096, embeddings 128, vocab 30000), sequences of 512
tokens, 15 % masked, LAMB lr 1.76e-3 with linear warm-up, per-GPU micro-batch 32, target_batch_size 4096, gradients
averaged with Uniform8Bit compression, delayed optimizer step and delayed gradient averaging; every GPU is one peer.

One benchmark *step* is one collaborative optimizer step (an epoch of ``target_batch_size`` samples across the
swarm): it contains every micro-batch forward/backward of that epoch, gradient accumulation, the gradient
averaging round and the LAMB update. ``value`` is samples per second over all GPUs, timed with CUDA events on the
device (max over ranks); ``e2e`` repeats the measurement with every micro-batch copied from pinned host memory and
every loss read back to the host.

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        bench.py --gpus 8 --steps 3 --warmup 3
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

# stdout carries exactly one JSON line. Libraries write to file descriptor 1 as they please (NCCL prints its version
# banner there when NCCL_DEBUG=VERSION, whatever NCCL_DEBUG_FILE says), so descriptor 1 is pointed at stderr for the
# whole run and the result line goes out through a private duplicate of the original stdout.
_RESULT_FD = None


def _claim_stdout() -> None:
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def _emit(result: dict) -> None:
    _claim_stdout()
    os.write(_RESULT_FD, (json.dumps(result) + "\n").encode())


BASELINE_SAMPLES_PER_SEC = 20.924  # the only Optimizer throughput in the reference tree: examples/albert/README.md:96


def _reference_arm(args) -> None:
    reason = ("the reference cannot be installed offline: its build downloads the Go p2pd binary "
              "(setup.py:126-162, urlopen fails without network) and needs grpc_tools to compile protos")
    if int(os.environ.get("RANK", "0")) == 0:
        _emit({"impl": "reference", "unavailable": reason})


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.proc, self.path = gpu_index, None, None

    def start(self) -> None:
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(5)
        except Exception:
            self.proc.kill()
        try:
            rows = [line.strip().split(", ") for line in open(self.path) if line.strip()]
            clocks = [float(r[0]) for r in rows if r and r[0].replace(".", "").isdigit()]
            if clocks:
                busy = sorted(clocks)[len(clocks) // 4:]  # ignore idle samples at the edges
                out["sm_mhz"] = statistics.median(busy)
                out["sm_max_mhz"] = float(rows[0][1])
                out["power_w_max"] = max(float(r[2]) for r in rows if len(r) > 2 and r[2].replace(".", "").isdigit())
                names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
                for k, name in enumerate(names):
                    if any(len(r) > 4 + k and r[4 + k].strip().lower() == "active" for r in rows):
                        out["reasons"].append(name)
            os.unlink(self.path)
        except Exception:
            pass
        return out


def main() -> None:
    _claim_stdout()
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=3, help="timed collaborative optimizer steps (epochs)")
    parser.add_argument("--warmup", type=int, default=3, help="untimed warm-up epochs")
    parser.add_argument("--impl", default="ours", choices=["ours", "reference", "torch_nccl"],
                        help="ours: this framework; reference: the unmodified reference (unavailable offline); "
                             "torch_nccl: plain PyTorch + NCCL baseline of the same workload")
    parser.add_argument("--context-steps", type=int, default=1,
                        help="with --impl ours: collaborative steps of the plain PyTorch + NCCL baseline to time "
                             "afterwards for context (0 = skip)")
    parser.add_argument("--micro-batch", type=int, default=32)
    parser.add_argument("--seq-len", type=int, default=512)
    parser.add_argument("--target-batch-size", type=int, default=4096)
    parser.add_argument("--model", default="large", choices=["large", "tiny"])
    parser.add_argument("--no-e2e", action="store_true")
    args = parser.parse_args()
    if args.impl == "reference":
        return _reference_arm(args)

    import torch
    import torch.distributed as dist

    import hivemind_b200 as hivemind
    from hivemind_b200.models.albert import AlbertConfig, AlbertForMaskedLM, make_mlm_batch
    from hivemind_b200.ops import _lib
    from hivemind_b200.ops.gemm import check_kernel_errors
    from hivemind_b200.optim.fused import FusedLAMB

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"launched with WORLD_SIZE={world} but --gpus {args.gpus}"
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    host_group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
        # barriers and the final reductions of the timing go over a host-side group: a NCCL barrier would put a
        # kernel that waits for every rank into the stream that the background averaging rounds synchronise with
        host_group = dist.new_group(backend="gloo")
    warmup = args.warmup

    torch.manual_seed(1234)  # identical initial weights on every peer
    cfg = AlbertConfig.large() if args.model == "large" else AlbertConfig.tiny()
    seq_len = min(args.seq_len, cfg.max_position_embeddings)

    def baseline(steps: int, warmup_steps: int, end_to_end: bool = False) -> dict:
        sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "benchmarks"))
        import torch_albert_baseline

        gen_b = torch.Generator().manual_seed(2000 + rank)
        return torch_albert_baseline.run(
            device=device, world=world, rank=rank, host_group=host_group, micro_batch=args.micro_batch, seq_len=seq_len,
            target_batch_size=args.target_batch_size, steps=steps, warmup_steps=warmup_steps, end_to_end=end_to_end,
            make_batch=lambda i: make_mlm_batch(AlbertConfig.large(), args.micro_batch, seq_len, generator=gen_b, pin=True))

    if args.impl == "torch_nccl":
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        res = baseline(args.steps, warmup)
        clocks = sampler.stop() if rank == 0 else {}
        e2e = baseline(args.steps, 1, end_to_end=True) if not args.no_e2e else None
        if rank == 0:
            _emit({
                "metric": "Optimizer samples/s (ALBERT-large)", "value": res["value"], "unit": "samples/s",
                "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": res["ms_per_step"],
                "higher_is_better": True, "scaling": "strong", "vs_baseline": res["value"] / BASELINE_SAMPLES_PER_SEC,
                "dtype": "bf16", "data": "synthetic", "impl": "torch_nccl", "clocks": clocks,
                "e2e": None if e2e is None else {"value": e2e["value"], "unit": "samples/s"},
                "config": {"model": "albert-large, plain PyTorch modules", "global_batch": args.target_batch_size,
                           "micro_batch_per_gpu": args.micro_batch, "seq_len": seq_len, "parallelism": f"dp{world}",
                           "what": res["what"]}})
        if world > 1:
            dist.destroy_process_group()
        return

    model = AlbertForMaskedLM(cfg).to(device)

    # one DHT per peer; rank 0 bootstraps the others
    if rank == 0:
        dht = hivemind.DHT(start=True)
        maddrs = [str(m) for m in dht.get_visible_maddrs()]
    else:
        maddrs = None
    if world > 1:
        box = [maddrs]
        dist.broadcast_object_list(box, src=0, group=host_group)
        maddrs = box[0]
        if rank != 0:
            dht = hivemind.DHT(initial_peers=maddrs, start=True)

    total_steps, warmup_steps = 125000, 5000
    opt = hivemind.Optimizer(
        dht=dht, run_id="albert_bench", target_batch_size=args.target_batch_size, batch_size_per_step=args.micro_batch,
        # biases and LayerNorm weights are not decayed (examples/albert/run_trainer.py:250-260)
        params=[dict(params=[p for p in model.parameters() if p.ndim > 1], weight_decay=0.01),
                dict(params=[p for p in model.parameters() if p.ndim <= 1], weight_decay=0.0)],
        optimizer=lambda params: FusedLAMB(params, lr=1.76e-3, betas=(0.9, 0.999), eps=1e-6, weight_decay=0.01,
                                           clamp_value=10000.0, debias=True),
        scheduler=lambda o: torch.optim.lr_scheduler.LambdaLR(
            o, lambda step: min((step + 1) / warmup_steps, max(0.0, (total_steps - step) / (total_steps - warmup_steps)))),
        grad_compression=hivemind.Uniform8BitQuantization(), state_averaging_compression=hivemind.Float16Compression(),
        reuse_grad_buffers=True, offload_optimizer=True, delay_optimizer_step=True, delay_grad_averaging=True,
        matchmaking_time=1.0, averaging_timeout=30.0, next_chunk_timeout=5.0, average_state_every=1,
        averager_opts=dict(request_timeout=0.5, target_group_size=world if world > 1 else None),
        tracker_opts=dict(min_refresh_period=0.02, default_refresh_period=0.05, max_refresh_period=0.2),
        verbose=False)

    gen = torch.Generator().manual_seed(1000 + rank)
    host_pool = [make_mlm_batch(cfg, args.micro_batch, seq_len, generator=gen, pin=True) for _ in range(8)]
    device_pool = [{k: v.to(device) for k, v in b.items()} for b in host_pool]
    h2d_bytes = sum(v.numel() * v.element_size() for v in host_pool[0].values())

    def micro_step(i: int, end_to_end: bool):
        if end_to_end:
            batch = {k: v.to(device, non_blocking=True) for k, v in host_pool[i % len(host_pool)].items()}
        else:
            batch = device_pool[i % len(device_pool)]
        loss = model(batch["input_ids"], batch["labels"], masked_positions=batch["masked_positions"])
        loss.backward()
        opt.step()
        return float(loss.item()) if end_to_end else loss

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier(group=host_group)

    def run_epochs(num_epochs: int, end_to_end: bool):
        """Run micro-steps until this peer has finished ``num_epochs`` more collaborative steps."""
        target_epoch, steps, last = opt.local_epoch + num_epochs, 0, None
        while opt.local_epoch < target_epoch:
            last = micro_step(steps, end_to_end)
            steps += 1
        return steps, last

    def timed(num_epochs: int, end_to_end: bool):
        barrier()
        launches0 = _lib.launch_count()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        steps, last = run_epochs(num_epochs, end_to_end)
        end.record()
        barrier()
        ms = torch.tensor([start.elapsed_time(end)], dtype=torch.float64)
        samples = torch.tensor([float(steps * args.micro_batch)], dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX, group=host_group)
            dist.all_reduce(samples, op=dist.ReduceOp.SUM, group=host_group)
        return float(ms.item()), float(samples.item()), _lib.launch_count() - launches0, last

    run_epochs(warmup, end_to_end=False)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms, samples, launches, _ = timed(args.steps, end_to_end=False)
    clocks = sampler.stop() if rank == 0 else {}
    e2e = None
    if not args.no_e2e:
        run_epochs(1, end_to_end=True)
        e2e_ms, e2e_samples, _, last_loss = timed(args.steps, end_to_end=True)
        micro_per_step = e2e_samples / args.micro_batch / args.steps  # forward/backward passes per step, all GPUs
        e2e = {"value": e2e_samples / (e2e_ms / 1e3), "unit": "samples/s",
               "h2d_bytes_per_step": int(h2d_bytes * micro_per_step), "d2h_bytes_per_step": int(4 * micro_per_step),
               "note": f"every forward/backward pass copies its batch from pinned host memory ({h2d_bytes} B) and reads "
                       f"its loss back (4 B); a collaborative step has {micro_per_step:.0f} such passes over all GPUs",
               "last_loss": last_loss}
    check_kernel_errors()
    value = samples / (ms / 1e3)
    # for context only: the same workload built from stock PyTorch + NCCL, timed after this framework's run is over
    opt.shutdown()
    dht.shutdown()
    del opt, model
    torch.cuda.empty_cache()
    torch_nccl = None
    if args.context_steps > 0 and args.model == "large":
        try:
            torch_nccl = baseline(args.context_steps, 1)
        except Exception as e:  # the context number must never cost the headline number
            torch_nccl = {"error": repr(e)}
    if rank == 0:
        _emit({
            "metric": "Optimizer samples/s (ALBERT-large)", "value": value, "unit": "samples/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": value / BASELINE_SAMPLES_PER_SEC, "dtype": "bf16", "data": "synthetic",
            "impl": "ours", "gpu_launches": launches, "clocks": clocks, "e2e": e2e, "torch_nccl_same_box": torch_nccl,
            "config": {"model": f"albert-{args.model} (24 shared layers, hidden 1024, ffn 4096, vocab 30000)",
                       "global_batch": args.target_batch_size, "micro_batch_per_gpu": args.micro_batch,
                       "seq_len": seq_len, "parallelism": f"dp{world}", "optimizer": "LAMB lr 1.76e-3",
                       "grad_compression": "Uniform8Bit", "delay_optimizer_step": True, "delay_grad_averaging": True,
                       "state_averaging": "every epoch, Float16, device butterfly (delayed)",
                       "weight_decay": "0.01 on matrices, 0 on biases and LayerNorm weights",
                       "step_definition": "one collaborative optimizer step = target_batch_size samples over all GPUs",
                       "samples_in_timed_region": samples,
                       "l2": "activations of one micro-batch (>2 GB) exceed the 126 MB L2; no explicit flush",
                       "baseline_note": "vs_baseline divides by the only Optimizer throughput printed in the "
                                        "reference tree (20.924 samples/s, one trainer, unspecified GPU)"}})
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

"""A few forward/backward/optimizer steps of the ALBERT-shaped model without any networking, for kernel profiling.

    python benchmarks/profile_albert_step.py --batch 32 --steps 2 --warmup 2
    ncu --metrics gpu__time_duration.sum --clock-control none -c 1500 --csv --log-file launches.csv \
        python benchmarks/profile_albert_step.py --batch 32 --steps 1 --warmup 1
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from hivemind_b200.models.albert import AlbertConfig, AlbertForMaskedLM, make_mlm_batch
from hivemind_b200.optim.fused import FusedLAMB


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--batch", type=int, default=32)
    parser.add_argument("--seq", type=int, default=512)
    parser.add_argument("--steps", type=int, default=2)
    parser.add_argument("--warmup", type=int, default=2)
    parser.add_argument("--model", default="large")
    args = parser.parse_args()
    device = torch.device("cuda", 0)
    cfg = AlbertConfig.large() if args.model == "large" else AlbertConfig.tiny()
    model = AlbertForMaskedLM(cfg).to(device)
    opt = FusedLAMB(model.parameters(), lr=1.76e-3, eps=1e-6, weight_decay=0.01, clamp_value=10000.0, debias=True)
    batch = {k: v.to(device) for k, v in make_mlm_batch(cfg, args.batch, min(args.seq, cfg.max_position_embeddings)).items()}

    def step():
        loss = model(batch["input_ids"], batch["labels"], masked_positions=batch["masked_positions"])
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=False)
        return loss

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        loss = step()
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / args.steps
    print(f"batch {args.batch} x seq {args.seq}: {ms:.2f} ms/step, {args.batch / ms * 1e3:.1f} samples/s, loss {loss.item():.4f}")


if __name__ == "__main__":
    main()

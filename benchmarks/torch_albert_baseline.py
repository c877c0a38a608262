"""Plain-PyTorch baseline of the headline workload: the same ALBERT-large-shaped masked LM, built only from library
kernels (cuBLAS through ``nn.Linear`` under bf16 autocast, ``scaled_dot_product_attention``, ``F.layer_norm``,
``F.gelu``), fp32 master weights, gradients accumulated over micro-batches, summed across ranks with one NCCL
all-reduce per collaborative step, and a LAMB update written with ``torch._foreach`` operations.

It exists so that the numbers of ``bench.py`` have a same-box anchor made of stock components; nothing of this
package's kernels or averaging runs in it. ``run(...)`` returns samples per second over all ranks, timed on the
device like ``bench.py`` times its own arm.
"""
from __future__ import annotations

from typing import Dict, List

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


class TorchAlbertLayer(nn.Module):
    def __init__(self, hidden: int, heads: int, ffn: int, eps: float):
        super().__init__()
        self.heads, self.eps = heads, eps
        self.qkv = nn.Linear(hidden, 3 * hidden)
        self.attn_out = nn.Linear(hidden, hidden)
        self.attn_ln = nn.LayerNorm(hidden, eps=eps)
        self.ffn = nn.Linear(hidden, ffn)
        self.ffn_out = nn.Linear(ffn, hidden)
        self.ffn_ln = nn.LayerNorm(hidden, eps=eps)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        b, s, h = x.shape
        q, k, v = (t.transpose(1, 2) for t in self.qkv(x).view(b, s, 3, self.heads, h // self.heads).unbind(2))
        ctx = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(b, s, h)
        x = self.attn_ln(x + self.attn_out(ctx))
        return self.ffn_ln(x + self.ffn_out(F.gelu(self.ffn(x), approximate="tanh")))


class TorchAlbertForMaskedLM(nn.Module):
    """Same shapes as ``hivemind_b200.models.albert.AlbertForMaskedLM`` (one layer applied ``num_layers`` times)."""

    def __init__(self, vocab: int = 30000, emb: int = 128, hidden: int = 1024, layers: int = 24, heads: int = 16,
                 ffn: int = 4096, positions: int = 512, eps: float = 1e-12):
        super().__init__()
        self.layers = layers
        self.word = nn.Embedding(vocab, emb)
        self.pos = nn.Embedding(positions, emb)
        self.token_type = nn.Embedding(2, emb)
        self.emb_ln = nn.LayerNorm(emb, eps=eps)
        self.emb_proj = nn.Linear(emb, hidden)
        self.layer = TorchAlbertLayer(hidden, heads, ffn, eps)
        self.head_dense = nn.Linear(hidden, emb)
        self.head_ln = nn.LayerNorm(emb, eps=eps)
        self.decoder_bias = nn.Parameter(torch.zeros(vocab))

    def forward(self, input_ids: torch.Tensor, labels: torch.Tensor, masked_positions: torch.Tensor) -> torch.Tensor:
        b, s = input_ids.shape
        x = self.word(input_ids) + self.pos.weight[:s] + self.token_type.weight[0]
        x = self.emb_proj(self.emb_ln(x))
        for _ in range(self.layers):
            x = self.layer(x)
        rows = (masked_positions + torch.arange(b, device=input_ids.device).unsqueeze(1) * s).reshape(-1)
        picked = x.reshape(b * s, -1).index_select(0, rows)
        target = labels.reshape(-1).index_select(0, rows)
        z = self.head_ln(F.gelu(self.head_dense(picked), approximate="tanh"))
        logits = F.linear(z, self.word.weight, self.decoder_bias)
        return F.cross_entropy(logits.float(), target)


class ForeachLAMB(torch.optim.Optimizer):
    """LAMB (You et al., 2019) with bias correction and a clamped trust ratio, written with multi-tensor torch ops."""

    def __init__(self, params, lr: float, betas=(0.9, 0.999), eps: float = 1e-6, weight_decay: float = 0.01,
                 clamp_value: float = 10000.0):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, clamp_value=clamp_value))

    @torch.no_grad()
    def step(self):
        for group in self.param_groups:
            params = [p for p in group["params"] if p.grad is not None]
            if not params:
                continue
            grads = [p.grad for p in params]
            for p in params:
                if not self.state[p]:
                    self.state[p].update(step=0, exp_avg=torch.zeros_like(p), exp_avg_sq=torch.zeros_like(p))
            m = [self.state[p]["exp_avg"] for p in params]
            v = [self.state[p]["exp_avg_sq"] for p in params]
            b1, b2 = group["betas"]
            for p in params:
                self.state[p]["step"] += 1
            step = self.state[params[0]]["step"]
            torch._foreach_mul_(m, b1)
            torch._foreach_add_(m, grads, alpha=1 - b1)
            torch._foreach_mul_(v, b2)
            torch._foreach_addcmul_(v, grads, grads, value=1 - b2)
            denom = torch._foreach_sqrt(torch._foreach_div(v, 1 - b2 ** step))
            torch._foreach_add_(denom, group["eps"])
            update = torch._foreach_div(torch._foreach_div(m, 1 - b1 ** step), denom)
            if group["weight_decay"]:
                torch._foreach_add_(update, params, alpha=group["weight_decay"])
            w_norm = torch._foreach_norm(params)
            u_norm = torch._foreach_norm(update)
            for p, u, wn, un in zip(params, update, w_norm, u_norm):
                trust = torch.where((wn > 0) & (un > 0), wn.clamp(max=group["clamp_value"]) / un, torch.ones_like(wn))
                p.add_(u * trust, alpha=-group["lr"])


def split_decay_groups(named_parameters, weight_decay: float = 0.01) -> List[Dict]:
    """Biases and LayerNorm weights are not decayed (examples/albert/run_trainer.py:250-260)."""
    decay, no_decay = [], []
    for name, p in named_parameters:
        (no_decay if p.ndim == 1 else decay).append(p)
    return [dict(params=decay, weight_decay=weight_decay), dict(params=no_decay, weight_decay=0.0)]


def run(*, device: torch.device, world: int, rank: int, host_group, micro_batch: int, seq_len: int,
        target_batch_size: int, steps: int, warmup_steps: int, make_batch, end_to_end: bool = False) -> Dict:
    """Train ``steps`` collaborative steps (each ``target_batch_size`` samples over all ranks) after ``warmup_steps``.

    ``make_batch(i)`` returns the i-th pinned host batch (dict of tensors); with ``end_to_end`` every micro-batch is
    copied from the host and its loss read back, otherwise batches are pre-loaded on the device.
    """
    torch.manual_seed(1234)
    model = TorchAlbertForMaskedLM(positions=max(seq_len, 512)).to(device)
    opt = ForeachLAMB(split_decay_groups(model.named_parameters()), lr=1.76e-3)
    per_rank = max(target_batch_size // world // micro_batch, 1)
    pool = [make_batch(i) for i in range(8)]
    device_pool = [{k: v.to(device) for k, v in b.items()} for b in pool]

    def one_step(k: int):
        for i in range(per_rank):
            idx = (k * per_rank + i) % len(pool)
            batch = ({key: v.to(device, non_blocking=True) for key, v in pool[idx].items()} if end_to_end
                     else device_pool[idx])
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = model(batch["input_ids"], batch["labels"], batch["masked_positions"])
            (loss / per_rank).backward()
            if end_to_end:
                loss.item()
        if world > 1:
            flat = [p.grad for p in model.parameters() if p.grad is not None]
            bucket = torch.cat([g.reshape(-1) for g in flat])
            dist.all_reduce(bucket)
            bucket.div_(world)
            offset = 0
            for g in flat:
                g.copy_(bucket[offset:offset + g.numel()].view_as(g))
                offset += g.numel()
        opt.step()
        opt.zero_grad(set_to_none=False)

    for k in range(warmup_steps):
        one_step(k)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier(group=host_group)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for k in range(steps):
        one_step(warmup_steps + k)
    end.record()
    torch.cuda.synchronize()
    ms = torch.tensor([start.elapsed_time(end)], dtype=torch.float64)
    if world > 1:
        dist.barrier(group=host_group)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX, group=host_group)
    samples = float(steps * per_rank * micro_batch * world)
    del model, opt
    torch.cuda.empty_cache()
    return {"value": samples / (float(ms.item()) / 1e3), "unit": "samples/s", "ms_per_step": float(ms.item()) / steps,
            "steps": steps, "warmup": warmup_steps,
            "what": "plain PyTorch (cuBLAS, scaled_dot_product_attention, foreach LAMB) + one NCCL all-reduce per step"}

"""GPT-2-shaped causal language model built on the package's sm_100a kernels.

The reference library never looks inside the user's model; its PowerSGD averager
(hivemind/optim/power_sgd_averager.py:28-222) is exercised on generic 2-D weight gradients. This module provides the
decoder-only transformer on which the framework measures that averager: pre-LayerNorm blocks, learned position
embeddings, tanh-GELU, the output projection tied to the token embedding. Dense layers run on the tcgen05 GEMM with
fused bias/GELU epilogues; every ``residual add + LayerNorm`` pair is one kernel pass that also emits the updated
residual stream; weight gradients accumulate in fp32 straight into ``.grad``.

The vocabulary dimension of the embedding matrix is padded to a multiple of 128 rows (50257 -> 50304 for GPT-2) so
that the logits are an aligned GEMM output; the padded columns get a constant -1e4 logit offset and therefore
neither probability mass nor gradient.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from hivemind_b200.models.albert import _LowPrecisionCache
from hivemind_b200.ops.attention import attention
from hivemind_b200.ops.gemm import feed_forward, linear
from hivemind_b200.ops.norm_act import layer_norm


@dataclass
class GPT2Config:
    vocab_size: int = 50257
    n_positions: int = 1024
    n_embd: int = 1024
    n_layer: int = 24
    n_head: int = 16
    n_inner: int = 4096
    layer_norm_eps: float = 1e-5
    initializer_range: float = 0.02

    @classmethod
    def medium(cls) -> "GPT2Config":
        return cls()

    @classmethod
    def small(cls) -> "GPT2Config":
        return cls(n_embd=768, n_layer=12, n_head=12, n_inner=3072)

    @classmethod
    def tiny(cls) -> "GPT2Config":
        return cls(vocab_size=509, n_positions=64, n_embd=128, n_layer=2, n_head=2, n_inner=256)

    @property
    def padded_vocab_size(self) -> int:
        return (self.vocab_size + 127) // 128 * 128


class GPT2Block(nn.Module):
    """One decoder block. ``forward`` receives the block's already-normalised input and the residual stream, and
    returns the *next* block's normalised input (using the next LayerNorm's parameters) with the updated stream."""

    def __init__(self, cfg: GPT2Config):
        super().__init__()
        h, f = cfg.n_embd, cfg.n_inner
        self.num_heads, self.eps = cfg.n_head, cfg.layer_norm_eps
        self.ln_1_weight = nn.Parameter(torch.ones(h))
        self.ln_1_bias = nn.Parameter(torch.zeros(h))
        self.qkv_weight = nn.Parameter(torch.empty(3 * h, h))
        self.qkv_bias = nn.Parameter(torch.zeros(3 * h))
        self.attn_out_weight = nn.Parameter(torch.empty(h, h))
        self.attn_out_bias = nn.Parameter(torch.zeros(h))
        self.ln_2_weight = nn.Parameter(torch.ones(h))
        self.ln_2_bias = nn.Parameter(torch.zeros(h))
        self.ffn_weight = nn.Parameter(torch.empty(f, h))
        self.ffn_bias = nn.Parameter(torch.zeros(f))
        self.ffn_out_weight = nn.Parameter(torch.empty(h, f))
        self.ffn_out_bias = nn.Parameter(torch.zeros(h))
        nn.init.normal_(self.qkv_weight, std=cfg.initializer_range)
        nn.init.normal_(self.ffn_weight, std=cfg.initializer_range)
        # projections into the residual stream are scaled down by the depth, as in GPT-2
        for w in (self.attn_out_weight, self.ffn_out_weight):
            nn.init.normal_(w, std=cfg.initializer_range / (2 * cfg.n_layer) ** 0.5)

    def forward(self, normed, stream, next_ln_weight, next_ln_bias, lp: _LowPrecisionCache):
        b, s, h = normed.shape
        nh = self.num_heads
        qkv = linear(normed, self.qkv_weight, self.qkv_bias, weight_lp=lp.get(self.qkv_weight))
        ctx = attention(qkv, nh, causal=True)
        attn = linear(ctx, self.attn_out_weight, self.attn_out_bias, weight_lp=lp.get(self.attn_out_weight))
        normed, stream = layer_norm(attn, self.ln_2_weight, self.ln_2_bias, self.eps, residual=stream, return_sum=True)
        out = feed_forward(normed, self.ffn_weight, self.ffn_bias, self.ffn_out_weight, self.ffn_out_bias,
                           w1_lp=lp.get(self.ffn_weight), w2_lp=lp.get(self.ffn_out_weight))
        return layer_norm(out, next_ln_weight, next_ln_bias, self.eps, residual=stream, return_sum=True)


class GPT2LMHeadModel(nn.Module):
    """Decoder-only transformer with a tied output projection; ``forward`` returns the mean next-token loss."""

    def __init__(self, cfg: GPT2Config):
        super().__init__()
        self.cfg = cfg
        self.wte = nn.Parameter(torch.empty(cfg.padded_vocab_size, cfg.n_embd))
        self.wpe = nn.Parameter(torch.empty(cfg.n_positions, cfg.n_embd))
        self.blocks = nn.ModuleList([GPT2Block(cfg) for _ in range(cfg.n_layer)])
        self.ln_f_weight = nn.Parameter(torch.ones(cfg.n_embd))
        self.ln_f_bias = nn.Parameter(torch.zeros(cfg.n_embd))
        nn.init.normal_(self.wte, std=cfg.initializer_range)
        nn.init.normal_(self.wpe, std=cfg.initializer_range)
        with torch.no_grad():
            self.wte[cfg.vocab_size:].zero_()
        offset = torch.zeros(cfg.padded_vocab_size)
        offset[cfg.vocab_size:] = -1e4
        self.register_buffer("logit_offset", offset, persistent=False)
        self._lp = _LowPrecisionCache()

    def hidden_states(self, input_ids: torch.Tensor) -> torch.Tensor:
        b, s = input_ids.shape
        compute_dtype = torch.bfloat16 if input_ids.is_cuda else torch.float32
        stream = (F.embedding(input_ids, self.wte) + self.wpe[:s]).to(compute_dtype)
        first = self.blocks[0]
        normed = layer_norm(stream, first.ln_1_weight, first.ln_1_bias, self.cfg.layer_norm_eps)
        for i, block in enumerate(self.blocks):
            if i + 1 < len(self.blocks):
                nxt = self.blocks[i + 1]
                next_weight, next_bias = nxt.ln_1_weight, nxt.ln_1_bias
            else:
                next_weight, next_bias = self.ln_f_weight, self.ln_f_bias
            normed, stream = block(normed, stream, next_weight, next_bias, self._lp)
        return normed  # = ln_f(stream) after the last block

    def logits(self, input_ids: torch.Tensor) -> torch.Tensor:
        hidden = self.hidden_states(input_ids)
        out = linear(hidden, self.wte, self.logit_offset, weight_lp=self._lp.get(self.wte))
        return out[..., :self.cfg.vocab_size]

    def forward(self, input_ids: torch.Tensor, labels: Optional[torch.Tensor] = None) -> torch.Tensor:
        """
        :param input_ids: ``[batch, seq]`` token ids
        :param labels: ``[batch, seq]`` targets already aligned with the positions that predict them (``-100`` =
          not scored); by default position ``t`` predicts ``input_ids[:, t + 1]``
        """
        b, s = input_ids.shape
        hidden = self.hidden_states(input_ids)
        if labels is None:
            hidden, target = hidden[:, :-1], input_ids[:, 1:]
        else:
            target = labels
        hidden = hidden.reshape(-1, hidden.shape[-1])
        logits = linear(hidden, self.wte, self.logit_offset, weight_lp=self._lp.get(self.wte))
        return F.cross_entropy(logits.float(), target.reshape(-1), ignore_index=-100)

    def flops_per_token(self, seq_len: Optional[int] = None) -> float:
        """Forward+backward matmul FLOPs per token, causal attention counted at half of the full square."""
        c = self.cfg
        s = seq_len or c.n_positions
        per_layer = 2 * (4 * c.n_embd * c.n_embd + 2 * c.n_embd * c.n_inner) + 2 * s * c.n_embd
        return 3.0 * (c.n_layer * per_layer + 2 * c.n_embd * c.padded_vocab_size)


def make_lm_batch(cfg: GPT2Config, batch: int, seq: int, generator: Optional[torch.Generator] = None,
                  pin: bool = False) -> Dict[str, torch.Tensor]:
    """Synthetic causal-LM batch on the host: ids uniform over the vocabulary, labels = ids shifted by one."""
    ids = torch.randint(0, cfg.vocab_size, (batch, seq), generator=generator, dtype=torch.int64)
    labels = torch.full((batch, seq), -100, dtype=torch.int64)
    labels[:, :-1] = ids[:, 1:]
    out = {"input_ids": ids, "labels": labels}
    if pin and torch.cuda.is_available():
        out = {k: v.pin_memory() for k, v in out.items()}
    return out

"""Built-in expert modules, registered by name for ``Server.create(expert_cls=...)``.

``ffn``: ``LayerNorm(x + W2 gelu_tanh(W1 x + b1) + b2)`` with eps 1e-12 — the block of the reference
(hivemind/moe/server/layers/common.py:11-30). Here both matrix products run on the tcgen05 GEMM (bias and GELU in
the first product's epilogue) and the residual + LayerNorm is one kernel; on CPU the same formula runs in PyTorch.
``transformer``: one encoder layer over [batch, 128, hid]; ``nop`` / ``nop_delay``: identity experts for tests;
``det_dropout``: dropout with a caller-supplied mask.
"""
from __future__ import annotations

import time

import torch
from torch import nn

from hivemind_b200.moe.server.layers.custom_experts import register_expert_class
from hivemind_b200.ops.gemm import linear
from hivemind_b200.ops.norm_act import layer_norm

ffn_sample_input = lambda batch_size, hid_dim: torch.empty((batch_size, hid_dim))


@register_expert_class("ffn", ffn_sample_input)
class FeedforwardBlock(nn.Module):
    def __init__(self, hid_dim: int):
        super().__init__()
        self.ffn = nn.Linear(hid_dim, 4 * hid_dim)
        self.ffn_output = nn.Linear(4 * hid_dim, hid_dim)
        self.layer_norm = nn.LayerNorm(hid_dim, eps=1e-12)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        hidden = linear(x, self.ffn.weight, self.ffn.bias, activation="gelu")
        out = linear(hidden, self.ffn_output.weight, self.ffn_output.bias)
        return layer_norm(out.to(x.dtype), self.layer_norm.weight, self.layer_norm.bias, 1e-12, residual=x)


class TransformerEncoderLayer(nn.Module):
    """Post-norm encoder layer (self-attention + ffn) with tanh-GELU."""

    def __init__(self, d_model: int, nhead: int, dim_feedforward: int = 2048, dropout: float = 0.1):
        super().__init__()
        self.self_attn = nn.MultiheadAttention(d_model, nhead, dropout=dropout)
        self.linear1 = nn.Linear(d_model, dim_feedforward)
        self.dropout = nn.Dropout(dropout)
        self.linear2 = nn.Linear(dim_feedforward, d_model)
        self.norm1 = nn.LayerNorm(d_model)
        self.norm2 = nn.LayerNorm(d_model)
        self.dropout1 = nn.Dropout(dropout)
        self.dropout2 = nn.Dropout(dropout)

    def forward(self, src: torch.Tensor) -> torch.Tensor:
        src = src.transpose(0, 1)  # [seq, batch, hid]
        attended = self.self_attn(src, src, src)[0]
        src = self.norm1(src + self.dropout1(attended))
        hidden = self.dropout(linear(src, self.linear1.weight, self.linear1.bias, activation="gelu").to(src.dtype))
        src = self.norm2(src + self.dropout2(linear(hidden, self.linear2.weight, self.linear2.bias).to(src.dtype)))
        return src.transpose(0, 1)


transformer_sample_input = lambda batch_size, hid_dim: torch.empty((batch_size, 128, hid_dim))


@register_expert_class("transformer", transformer_sample_input)
class TunedTransformer(TransformerEncoderLayer):
    def __init__(self, hid_dim: int):
        super().__init__(hid_dim, dim_feedforward=4 * hid_dim, nhead=16)


nop_sample_input = lambda batch_size, hid_dim: torch.empty((batch_size, hid_dim))


@register_expert_class("nop", nop_sample_input)
class NopExpert(nn.Sequential):
    def __init__(self, hid_dim: int):
        super().__init__()
        self.w = nn.Parameter(torch.zeros(0), requires_grad=True)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x.clone()


@register_expert_class("nop_delay", nop_sample_input)
class DelayedNopExpert(nn.Sequential):
    """Identity that sleeps first; used to exercise client-side timeouts."""

    def __init__(self, hid_dim: int, delay: float = 0.5):
        super().__init__()
        self.w = nn.Parameter(torch.zeros(0), requires_grad=True)
        self.delay = delay

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        time.sleep(self.delay)
        return x.clone()

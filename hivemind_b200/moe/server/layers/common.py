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
from hivemind_b200.ops.gemm import feed_forward, linear
from hivemind_b200.ops.norm_act import layer_norm


def _rows(batch_size: int, hid_dim: int) -> torch.Tensor:
    """Schema input of experts that map [batch, hid] rows."""
    return torch.empty((batch_size, hid_dim))


def _sequences(batch_size: int, hid_dim: int, length: int = 128) -> torch.Tensor:
    """Schema input of experts that map [batch, length, hid] sequences."""
    return torch.empty((batch_size, length, hid_dim))


def gelu_fast(x: torch.Tensor) -> torch.Tensor:
    """The tanh approximation of GELU that the ``ffn`` and ``transformer`` experts use
    (hivemind/moe/server/layers/common.py:12-14 writes the formula out)."""
    return torch.nn.functional.gelu(x, approximate="tanh")


ffn_sample_input = nop_sample_input = _rows
transformer_sample_input = _sequences


@register_expert_class("ffn", _rows)
class FeedforwardBlock(nn.Module):
    """``LayerNorm(x + W2 gelu(W1 x + b1) + b2)``; parameter names match the reference's checkpoints."""

    expansion = 4

    def __init__(self, hid_dim: int):
        super().__init__()
        self.ffn = nn.Linear(hid_dim, self.expansion * hid_dim)
        self.ffn_output = nn.Linear(self.expansion * hid_dim, hid_dim)
        self.layer_norm = nn.LayerNorm(hid_dim, eps=1e-12)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        up, down, norm = self.ffn, self.ffn_output, self.layer_norm
        # one autograd node for both products; the residual's gradient joins the input gradient inside a GEMM and the
        # output bias gets its gradient from the LayerNorm's backward pass
        update, skip = feed_forward(x, up.weight, up.bias, down.weight, down.bias, skip_out_bias_grad=True, passthrough=True)
        return layer_norm(update.to(x.dtype), norm.weight, norm.bias, norm.eps, residual=skip, producer_bias=down.bias)


class TransformerEncoderLayer(nn.Module):
    """Post-norm encoder layer over batch-first input: self-attention, then a tanh-GELU feed-forward pair."""

    def __init__(self, d_model: int, nhead: int, dim_feedforward: int = 2048, dropout: float = 0.1):
        super().__init__()
        self.self_attn = nn.MultiheadAttention(d_model, nhead, dropout=dropout)
        self.linear1, self.linear2 = nn.Linear(d_model, dim_feedforward), nn.Linear(dim_feedforward, d_model)
        self.norm1, self.norm2 = nn.LayerNorm(d_model), nn.LayerNorm(d_model)
        self.dropout, self.dropout1, self.dropout2 = nn.Dropout(dropout), nn.Dropout(dropout), nn.Dropout(dropout)

    def _feed_forward(self, x: torch.Tensor) -> torch.Tensor:
        inner = linear(x, self.linear1.weight, self.linear1.bias, activation="gelu").to(x.dtype)
        return linear(self.dropout(inner), self.linear2.weight, self.linear2.bias).to(x.dtype)

    def forward(self, src: torch.Tensor) -> torch.Tensor:
        x = src.transpose(0, 1)  # the attention module wants [seq, batch, hid]
        x = self.norm1(x + self.dropout1(self.self_attn(x, x, x, need_weights=False)[0]))
        x = self.norm2(x + self.dropout2(self._feed_forward(x)))
        return x.transpose(0, 1)


@register_expert_class("transformer", _sequences)
class TunedTransformer(TransformerEncoderLayer):
    def __init__(self, hid_dim: int):
        super().__init__(hid_dim, nhead=16, dim_feedforward=4 * hid_dim)


class _Identity(nn.Sequential):
    """An expert that returns its input; the empty parameter keeps optimizers and checkpoints happy."""

    delay = 0.0

    def __init__(self, hid_dim: int):
        super().__init__()
        self.w = nn.Parameter(torch.zeros(0), requires_grad=True)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.delay > 0:
            time.sleep(self.delay)
        return x.clone()


@register_expert_class("nop", _rows)
class NopExpert(_Identity):
    pass


@register_expert_class("nop_delay", _rows)
class DelayedNopExpert(_Identity):
    """Identity that sleeps first; used to exercise client-side timeouts."""

    def __init__(self, hid_dim: int, delay: float = 0.5):
        super().__init__(hid_dim)
        self.delay = delay

"""ALBERT-shaped masked language model built on the package's sm_100a kernels.

The reference trains ``transformers``' ALBERT-large through ``hivemind.Optimizer``
(examples/albert/run_trainer.py:204-227, config ``albert-large-v2``); the library itself never looks inside the
model. This module provides the same architecture (factorised embeddings, one transformer layer whose weights are
shared by all ``num_hidden_layers`` applications, tanh-GELU, post-LayerNorm, tied MLM decoder) so that the framework
has a flagship model whose dense layers run on the tcgen05 GEMM with fused bias/GELU epilogues, whose
residual+LayerNorm is one kernel, and whose weight gradients are accumulated in fp32 straight into ``.grad``.

Parameters are fp32 (the master copy that the optimizer and the averagers see); matrix multiplies run in bf16 with
fp32 accumulation; bf16 copies of the weights are refreshed lazily when a parameter's version changes.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from hivemind_b200.ops.attention import attention
from hivemind_b200.ops.gemm import feed_forward, linear
from hivemind_b200.ops.norm_act import layer_norm

# HIVEMIND_B200_FUSE_EPILOGUES=0 runs the encoder with one autograd node per layer (no epilogue fusion across layers)
_FUSE_EPILOGUES = os.environ.get("HIVEMIND_B200_FUSE_EPILOGUES", "1") != "0"


@dataclass
class AlbertConfig:
    vocab_size: int = 30000
    embedding_size: int = 128
    hidden_size: int = 1024
    num_hidden_layers: int = 24
    num_attention_heads: int = 16
    intermediate_size: int = 4096
    max_position_embeddings: int = 512
    type_vocab_size: int = 2
    layer_norm_eps: float = 1e-12
    initializer_range: float = 0.02
    mask_token_id: int = 4

    @classmethod
    def large(cls) -> "AlbertConfig":
        return cls()

    @classmethod
    def tiny(cls) -> "AlbertConfig":
        return cls(vocab_size=512, embedding_size=64, hidden_size=128, num_hidden_layers=2, num_attention_heads=2,
                   intermediate_size=256, max_position_embeddings=64)


class _LowPrecisionCache:
    """bf16 copies of fp32 parameters, re-cast only when the parameter has been modified."""

    def __init__(self):
        self._copies: Dict[int, Tuple[int, int, torch.Tensor]] = {}

    def get(self, p: torch.Tensor) -> Optional[torch.Tensor]:
        if p.dtype == torch.bfloat16 or not p.is_cuda:
            return None
        entry = self._copies.get(id(p))
        if entry is not None and entry[0] == p._version and entry[1] == p.data_ptr():
            return entry[2]
        lp = p.detach().to(torch.bfloat16)
        self._copies[id(p)] = (p._version, p.data_ptr(), lp)
        return lp


class AlbertLayer(nn.Module):
    """Self-attention + FFN block; applied ``num_hidden_layers`` times with the same weights."""

    def __init__(self, cfg: AlbertConfig):
        super().__init__()
        h, f = cfg.hidden_size, cfg.intermediate_size
        self.num_heads = cfg.num_attention_heads
        self.eps = cfg.layer_norm_eps
        self.qkv_weight = nn.Parameter(torch.empty(3 * h, h))
        self.qkv_bias = nn.Parameter(torch.zeros(3 * h))
        self.attn_out_weight = nn.Parameter(torch.empty(h, h))
        self.attn_out_bias = nn.Parameter(torch.zeros(h))
        self.attn_ln_weight = nn.Parameter(torch.ones(h))
        self.attn_ln_bias = nn.Parameter(torch.zeros(h))
        self.ffn_weight = nn.Parameter(torch.empty(f, h))
        self.ffn_bias = nn.Parameter(torch.zeros(f))
        self.ffn_out_weight = nn.Parameter(torch.empty(h, f))
        self.ffn_out_bias = nn.Parameter(torch.zeros(h))
        self.ffn_ln_weight = nn.Parameter(torch.ones(h))
        self.ffn_ln_bias = nn.Parameter(torch.zeros(h))
        for w in (self.qkv_weight, self.attn_out_weight, self.ffn_weight, self.ffn_out_weight):
            nn.init.normal_(w, std=cfg.initializer_range)

    def forward(self, x: torch.Tensor, lp: _LowPrecisionCache) -> torch.Tensor:
        nh = self.num_heads
        if not _FUSE_EPILOGUES:  # every layer its own autograd node (kept for ablation runs)
            qkv = linear(x, self.qkv_weight, self.qkv_bias, weight_lp=lp.get(self.qkv_weight))
            attn = linear(attention(qkv, nh), self.attn_out_weight, self.attn_out_bias, weight_lp=lp.get(self.attn_out_weight))
            x = layer_norm(attn, self.attn_ln_weight, self.attn_ln_bias, self.eps, residual=x)
            inter = linear(x, self.ffn_weight, self.ffn_bias, activation="gelu", weight_lp=lp.get(self.ffn_weight))
            out = linear(inter, self.ffn_out_weight, self.ffn_out_bias, weight_lp=lp.get(self.ffn_out_weight))
            return layer_norm(out, self.ffn_ln_weight, self.ffn_ln_bias, self.eps, residual=x)
        # passthrough: the residual branch's gradient joins the projection's input gradient in that GEMM's epilogue
        qkv, x = linear(x, self.qkv_weight, self.qkv_bias, weight_lp=lp.get(self.qkv_weight), passthrough=True)
        ctx = attention(qkv, nh)  # reads the packed projections, writes [b, s, h]: no transposes around it
        # the biases in front of the two LayerNorms get their gradients from the LayerNorm backward pass
        attn = linear(ctx, self.attn_out_weight, self.attn_out_bias, weight_lp=lp.get(self.attn_out_weight),
                      skip_bias_grad=True)
        x = layer_norm(attn, self.attn_ln_weight, self.attn_ln_bias, self.eps, residual=x,
                       producer_bias=self.attn_out_bias)
        out, x = feed_forward(x, self.ffn_weight, self.ffn_bias, self.ffn_out_weight, self.ffn_out_bias,
                              w1_lp=lp.get(self.ffn_weight), w2_lp=lp.get(self.ffn_out_weight),
                              skip_out_bias_grad=True, passthrough=True)
        return layer_norm(out, self.ffn_ln_weight, self.ffn_ln_bias, self.eps, residual=x,
                          producer_bias=self.ffn_out_bias)


class AlbertForMaskedLM(nn.Module):
    """ALBERT encoder with the masked-LM head; ``forward`` returns the mean cross-entropy over labelled positions."""

    def __init__(self, cfg: AlbertConfig):
        super().__init__()
        self.cfg = cfg
        e, h = cfg.embedding_size, cfg.hidden_size
        self.word_embeddings = nn.Parameter(torch.empty(cfg.vocab_size, e))
        self.position_embeddings = nn.Parameter(torch.empty(cfg.max_position_embeddings, e))
        self.token_type_embeddings = nn.Parameter(torch.empty(cfg.type_vocab_size, e))
        self.emb_ln_weight = nn.Parameter(torch.ones(e))
        self.emb_ln_bias = nn.Parameter(torch.zeros(e))
        self.emb_proj_weight = nn.Parameter(torch.empty(h, e))
        self.emb_proj_bias = nn.Parameter(torch.zeros(h))
        self.layer = AlbertLayer(cfg)
        self.head_dense_weight = nn.Parameter(torch.empty(e, h))
        self.head_dense_bias = nn.Parameter(torch.zeros(e))
        self.head_ln_weight = nn.Parameter(torch.ones(e))
        self.head_ln_bias = nn.Parameter(torch.zeros(e))
        self.decoder_bias = nn.Parameter(torch.zeros(cfg.vocab_size))
        for w in (self.word_embeddings, self.position_embeddings, self.token_type_embeddings, self.emb_proj_weight,
                  self.head_dense_weight):
            nn.init.normal_(w, std=cfg.initializer_range)
        self._lp = _LowPrecisionCache()

    def encode(self, input_ids: torch.Tensor, token_type_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        b, s = input_ids.shape
        compute_dtype = torch.bfloat16 if input_ids.is_cuda else torch.float32
        emb = F.embedding(input_ids, self.word_embeddings) + self.position_embeddings[:s]
        if token_type_ids is None:
            emb = emb + self.token_type_embeddings[0]
        else:
            emb = emb + F.embedding(token_type_ids, self.token_type_embeddings)
        emb = layer_norm(emb.to(compute_dtype), self.emb_ln_weight, self.emb_ln_bias, self.cfg.layer_norm_eps)
        x = linear(emb, self.emb_proj_weight, self.emb_proj_bias, weight_lp=self._lp.get(self.emb_proj_weight))
        for _ in range(self.cfg.num_hidden_layers):
            x = self.layer(x, self._lp)
        return x

    def forward(self, input_ids: torch.Tensor, labels: torch.Tensor,
                masked_positions: Optional[torch.Tensor] = None,
                token_type_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        """
        :param input_ids: ``[batch, seq]`` token ids (masked positions already replaced by the mask token)
        :param labels: ``[batch, seq]`` target ids, ``-100`` where no prediction is scored
        :param masked_positions: optional ``[batch, n]`` indices of the scored positions of each sequence; passing
          them avoids a device-to-host synchronisation to find the labelled rows
        """
        return self.masked_lm_loss(self.encode(input_ids, token_type_ids), labels, masked_positions)

    def masked_lm_loss(self, hidden: torch.Tensor, labels: torch.Tensor,
                       masked_positions: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Mean cross-entropy of the tied decoder over the scored positions of ``hidden`` (``[batch, seq, hidden]``)."""
        b, s = labels.shape
        hidden = hidden.reshape(b * s, -1)
        if masked_positions is not None:
            rows = (masked_positions + torch.arange(b, device=labels.device).unsqueeze(1) * s).reshape(-1)
        else:
            rows = (labels.reshape(-1) != -100).nonzero(as_tuple=True)[0]
        picked = hidden.index_select(0, rows)
        target = labels.reshape(-1).index_select(0, rows)
        z = linear(picked, self.head_dense_weight, self.head_dense_bias, activation="gelu",
                   weight_lp=self._lp.get(self.head_dense_weight))
        z = layer_norm(z, self.head_ln_weight, self.head_ln_bias, self.cfg.layer_norm_eps)
        logits = linear(z, self.word_embeddings, self.decoder_bias, weight_lp=self._lp.get(self.word_embeddings))
        return F.cross_entropy(logits.float(), target, ignore_index=-100)

    def flops_per_token(self) -> float:
        """Forward+backward matmul FLOPs per token (6 x parameters touched per token, plus attention)."""
        c = self.cfg
        h, f, L, s = c.hidden_size, c.intermediate_size, c.num_hidden_layers, c.max_position_embeddings
        per_layer = 2 * (4 * h * h + 2 * h * f) + 4 * s * h
        return 3.0 * (L * per_layer + 2 * c.embedding_size * h)


class AlbertForPreTraining(AlbertForMaskedLM):
    """The two pre-training objectives of ALBERT: masked LM plus sentence-order prediction, a two-way classifier on the
    ``tanh``-pooled first token that tells whether two consecutive segments come in their original order (the model
    that the reference's example trains, examples/albert/run_trainer.py:204-227, there taken from ``transformers``)."""

    def __init__(self, cfg: AlbertConfig):
        super().__init__(cfg)
        h = cfg.hidden_size
        self.pooler_weight = nn.Parameter(torch.empty(h, h))
        self.pooler_bias = nn.Parameter(torch.zeros(h))
        self.sop_weight = nn.Parameter(torch.empty(2, h))
        self.sop_bias = nn.Parameter(torch.zeros(2))
        for w in (self.pooler_weight, self.sop_weight):
            nn.init.normal_(w, std=cfg.initializer_range)

    def sentence_order_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        pooled = torch.tanh(linear(hidden[:, 0].contiguous(), self.pooler_weight, self.pooler_bias,
                                   weight_lp=self._lp.get(self.pooler_weight)).float())
        # two output columns are no work for a tensor-core tile: this product stays a plain matmul
        return pooled @ self.sop_weight.float().t() + self.sop_bias.float()

    def forward(self, input_ids: torch.Tensor, labels: torch.Tensor, masked_positions: Optional[torch.Tensor] = None,
                token_type_ids: Optional[torch.Tensor] = None,
                sentence_order_label: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Masked-LM loss, plus the sentence-order loss when ``sentence_order_label`` (``[batch]``, 0 = original order,
        1 = swapped) is given."""
        hidden = self.encode(input_ids, token_type_ids)
        loss = self.masked_lm_loss(hidden, labels, masked_positions)
        if sentence_order_label is not None:
            loss = loss + F.cross_entropy(self.sentence_order_logits(hidden), sentence_order_label)
        return loss


def make_mlm_batch(cfg: AlbertConfig, batch: int, seq: int, generator: Optional[torch.Generator] = None,
                   mask_fraction: float = 0.15, pin: bool = False) -> Dict[str, torch.Tensor]:
    """Synthetic MLM batch on the host: ids uniform in [5, vocab), a fixed count of masked positions per sequence."""
    n_mask = max(1, int(round(mask_fraction * seq)))
    ids = torch.randint(5, cfg.vocab_size, (batch, seq), generator=generator, dtype=torch.int64)
    pos = torch.rand(batch, seq, generator=generator).argsort(dim=1)[:, :n_mask].contiguous()
    labels = torch.full((batch, seq), -100, dtype=torch.int64)
    labels.scatter_(1, pos, ids.gather(1, pos))
    ids.scatter_(1, pos, cfg.mask_token_id)
    out = {"input_ids": ids, "labels": labels, "masked_positions": pos}
    if pin and torch.cuda.is_available():
        out = {k: v.pin_memory() for k, v in out.items()}
    return out

"""Fused multi-head self-attention on the package's tcgen05 kernels (``csrc/attention.cu``).

``attention(qkv, num_heads, causal)`` takes the packed projection output ``[batch, seq, 3 * hidden]`` (q, k and v
thirds, each split into heads of 64 channels) and returns the context ``[batch, seq, hidden]`` — the layouts that
the surrounding linear layers produce and consume, so no transposes or copies surround the kernels, and the backward
pass writes one packed ``d(qkv)`` tensor. The same computation in the reference's ``transformer`` expert goes through
``nn.MultiheadAttention`` (hivemind/moe/server/layers/common.py:33-62).

On CPU tensors, or for head sizes other than 64, the function evaluates the PyTorch formula
(``reference_attention``), which is also what the GPU tests compare the kernels against.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch

from hivemind_b200.ops import _lib
from hivemind_b200.ops.gemm import _err_flag

KERNEL_HEAD_DIM = 64


def reference_attention(qkv: torch.Tensor, num_heads: int, causal: bool = False,
                        scale: Optional[float] = None) -> torch.Tensor:
    """Plain PyTorch attention over a packed ``[batch, seq, 3 * hidden]`` tensor, in the tensor's own dtype."""
    b, s, three_h = qkv.shape
    hidden = three_h // 3
    d = hidden // num_heads
    q, k, v = (t.transpose(1, 2) for t in qkv.view(b, s, 3, num_heads, d).unbind(2))  # [b, nh, s, d]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    scores = torch.matmul(q, k.transpose(-1, -2)) * scale
    if causal:
        mask = torch.ones(s, s, dtype=torch.bool, device=qkv.device).tril()
        scores = scores.masked_fill(~mask, float("-inf"))
    ctx = torch.matmul(torch.softmax(scores, dim=-1), v)
    return ctx.transpose(1, 2).reshape(b, s, hidden)


class _AttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv: torch.Tensor, num_heads: int, causal: bool, scale: float):
        b, s, three_h = qkv.shape
        hidden = three_h // 3
        lib = _lib.load_library()
        dev = qkv.device
        out = torch.empty((b, s, hidden), dtype=torch.bfloat16, device=dev)
        lse = torch.empty((b, num_heads, s), dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            code = lib.hm_attn_fwd(_lib.ptr(qkv), _lib.ptr(out), _lib.ptr(lse), b, s, num_heads, KERNEL_HEAD_DIM,
                                   int(causal), ctypes.c_float(scale), _lib.ptr(_err_flag(dev)), _lib.stream_ptr(dev))
        _lib.check(code, "hm_attn_fwd")
        ctx.save_for_backward(qkv, out, lse)
        ctx.num_heads, ctx.causal, ctx.scale = num_heads, causal, scale
        return out

    @staticmethod
    def backward(ctx, dout: torch.Tensor):
        qkv, out, lse = ctx.saved_tensors
        b, s, three_h = qkv.shape
        hidden = three_h // 3
        dev = qkv.device
        if dout.dtype != torch.bfloat16:
            dout = dout.to(torch.bfloat16)
        if not dout.is_contiguous():
            dout = dout.contiguous()
        lib = _lib.load_library()
        dqkv = torch.empty_like(qkv)
        delta = torch.empty_like(lse)
        dq_acc = torch.empty((b, s, hidden), dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            code = lib.hm_attn_bwd(_lib.ptr(qkv), _lib.ptr(out), _lib.ptr(dout), _lib.ptr(lse), _lib.ptr(dqkv),
                                   _lib.ptr(delta), _lib.ptr(dq_acc), b, s, ctx.num_heads, KERNEL_HEAD_DIM,
                                   int(ctx.causal), ctypes.c_float(ctx.scale), _lib.ptr(_err_flag(dev)),
                                   _lib.stream_ptr(dev))
        _lib.check(code, "hm_attn_bwd", kernels=3)
        return dqkv, None, None, None


def kernel_supports(qkv: torch.Tensor, num_heads: int) -> bool:
    """True if the tensor-core kernels cover this call: CUDA, bf16, heads of 64 channels."""
    if not qkv.is_cuda or qkv.dim() != 3 or qkv.shape[-1] % (3 * num_heads) != 0:
        return False
    return qkv.dtype == torch.bfloat16 and qkv.shape[-1] // (3 * num_heads) == KERNEL_HEAD_DIM


def attention(qkv: torch.Tensor, num_heads: int, causal: bool = False, scale: Optional[float] = None) -> torch.Tensor:
    """Multi-head self-attention over packed projections.

    :param qkv: ``[batch, seq, 3 * hidden]``: the q, k and v thirds, each ``num_heads`` heads of ``hidden / num_heads``
    :param causal: position i attends to positions <= i only
    :param scale: softmax scale, ``1 / sqrt(head_dim)`` by default
    :returns: ``[batch, seq, hidden]`` in the dtype of ``qkv``
    """
    assert qkv.dim() == 3 and qkv.shape[-1] % (3 * num_heads) == 0
    head_dim = qkv.shape[-1] // (3 * num_heads)
    scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
    if kernel_supports(qkv, num_heads) and _lib.use_kernels(qkv):
        return _AttentionFn.apply(qkv.contiguous(), num_heads, bool(causal), scale)
    return reference_attention(qkv, num_heads, causal, scale)

"""LayerNorm (optionally fused with a residual add) and bias + tanh-GELU as autograd functions.

CUDA tensors run the sm_100a kernels of ``csrc/norm_act.cu``; CPU tensors run the PyTorch formulas below, which
double as the fp32 oracle of the GPU tests. The tanh form of GELU is the one the reference's ``ffn`` expert uses
(hivemind/moe/server/layers/common.py:11-12).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.nn.functional as F

from hivemind_b200.ops import _lib

_MAX_H = 8 * 32 * 8


def _kernel_ok(x: torch.Tensor, h: int) -> bool:
    return _lib.use_kernels(x) and x.dtype in (torch.bfloat16, torch.float32) and h % 8 == 0 and h <= _MAX_H


def gelu_tanh_reference(x: torch.Tensor) -> torch.Tensor:
    return F.gelu(x, approximate="tanh")


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, gamma, beta, eps, return_sum=False, producer_bias=None):
        ctx.set_materialize_grads(False)
        ctx.return_sum = return_sum
        ctx.producer_bias = producer_bias
        h = x.shape[-1]
        x2 = x.reshape(-1, h).contiguous()
        r2 = residual.reshape(-1, h).contiguous() if residual is not None else None
        rows = x2.shape[0]
        lib = _lib.load_library()
        y = torch.empty_like(x2)
        z = torch.empty_like(x2) if r2 is not None else None
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        g32 = gamma.detach().to(torch.float32).contiguous()
        b32 = beta.detach().to(torch.float32).contiguous()
        with torch.cuda.device(x.device):
            code = lib.hm_layernorm_fwd(_lib.ptr(x2), _lib.ptr(r2), _lib.ptr(g32), _lib.ptr(b32), _lib.ptr(y),
                                        _lib.ptr(z), _lib.ptr(mean), _lib.ptr(rstd), rows, h, ctypes.c_float(eps),
                                        _lib.dtype_code(x.dtype), _lib.sm_count(x.device), _lib.stream_ptr(x.device))
        _lib.check(code, "hm_layernorm_fwd")
        ctx.save_for_backward(z if z is not None else x2, g32, mean, rstd)
        ctx.has_residual = r2 is not None
        ctx.shape = x.shape
        ctx.param_dtype = (gamma.dtype, beta.dtype)
        ctx.params = (gamma, beta)
        if return_sum:
            return y.view(x.shape), (z if z is not None else x2).view(x.shape)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy, dz=None):
        zin, g32, mean, rstd = ctx.saved_tensors
        h = zin.shape[-1]
        rows = zin.shape[0]
        if dy is None:  # only the sum was used downstream
            dz = dz if dz is not None else torch.zeros(ctx.shape, dtype=zin.dtype, device=zin.device)
            pb = ctx.producer_bias
            db = None if pb is None else dz.reshape(-1, h).sum(0, dtype=torch.float32).to(pb.dtype)
            return dz, (dz if ctx.has_residual else None), None, None, None, None, db
        dy2 = dy.reshape(-1, h).contiguous()
        if dy2.dtype != zin.dtype:
            dy2 = dy2.to(zin.dtype)
        lib = _lib.load_library()
        dx = torch.empty_like(zin)
        gamma, beta = ctx.params
        # the kernel adds its column sums with atomics: when fp32 .grad buffers exist they are the target
        # (no zero-fill, cast and add per call); otherwise fresh buffers are returned to autograd
        direct = all(p.grad is not None and p.grad.dtype == torch.float32 and p.grad.is_contiguous()
                     and p.requires_grad for p in (gamma, beta))
        if direct:
            dgamma, dbeta = gamma.grad, beta.grad
        else:
            dgb = torch.zeros(2, h, dtype=torch.float32, device=zin.device)
            dgamma, dbeta = dgb[0], dgb[1]
        # the bias of the layer that produced the normalised tensor (if the caller named it): its gradient is the
        # column sum of dx, which the one-pass kernel takes along the way
        pb = ctx.producer_bias
        pb_direct = pb is not None and dz is None and pb.grad is not None and pb.grad.dtype == torch.float32 \
            and pb.grad.is_contiguous()
        dxsum = None
        if pb is not None and dz is None:
            dxsum = pb.grad if pb_direct else torch.zeros(h, dtype=torch.float32, device=zin.device)
        with torch.cuda.device(zin.device):
            code = lib.hm_layernorm_bwd_fused(_lib.ptr(dy2), _lib.ptr(zin), _lib.ptr(g32), _lib.ptr(mean),
                                              _lib.ptr(rstd), _lib.ptr(dx), _lib.ptr(dgamma), _lib.ptr(dbeta),
                                              _lib.ptr(dxsum), rows, h, _lib.dtype_code(zin.dtype),
                                              _lib.sm_count(zin.device), _lib.stream_ptr(zin.device))
            if code == -1:  # shape or dtype outside the one-pass kernel: row pass + column-strip pass
                code = lib.hm_layernorm_bwd(_lib.ptr(dy2), _lib.ptr(zin), _lib.ptr(g32), _lib.ptr(mean),
                                            _lib.ptr(rstd), _lib.ptr(dx), _lib.ptr(dgamma), _lib.ptr(dbeta), rows, h,
                                            _lib.dtype_code(zin.dtype), _lib.sm_count(zin.device),
                                            _lib.stream_ptr(zin.device))
                if dxsum is not None:
                    from hivemind_b200.ops.gemm import colsum_
                    colsum_(dxsum, dx)
        _lib.check(code, "hm_layernorm_bwd")
        dx = dx.view(ctx.shape)
        if dz is not None:
            dx.add_(dz.reshape(ctx.shape))
        grad_pb = None
        if pb is not None and not pb_direct:
            grad_pb = (dxsum if dxsum is not None else dx.reshape(-1, h).sum(0, dtype=torch.float32)).to(pb.dtype)
        if direct:
            return dx, (dx if ctx.has_residual else None), None, None, None, None, grad_pb
        return (dx, (dx if ctx.has_residual else None), dgamma.to(ctx.param_dtype[0]), dbeta.to(ctx.param_dtype[1]),
                None, None, grad_pb)


def layer_norm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, eps: float = 1e-5,
               residual: Optional[torch.Tensor] = None, return_sum: bool = False,
               producer_bias: Optional[torch.Tensor] = None):
    """``LayerNorm(x + residual)`` over the last dimension (``residual`` optional), statistics in fp32.

    With ``return_sum`` the result is ``(LayerNorm(x + residual), x + residual)``: the second tensor is the updated
    residual stream of a pre-LayerNorm transformer, produced by the same kernel pass.

    ``producer_bias``: the bias parameter of the linear layer whose output is ``x``, when that layer was called with
    ``skip_bias_grad=True``. The gradient of that bias is the column sum of this function's input gradient, which the
    backward kernel computes in the pass that produces the input gradient; it is delivered to the parameter from here.
    """
    h = x.shape[-1]
    if _kernel_ok(x, h):
        return _LayerNormFn.apply(x, residual, gamma, beta, eps, return_sum, producer_bias)
    if producer_bias is not None:
        x = _ColumnSumTap.apply(x, producer_bias)
    z = x if residual is None else x + residual
    y = F.layer_norm(z.to(torch.float32), (h,), gamma.to(torch.float32), beta.to(torch.float32), eps).to(x.dtype)
    return (y, z) if return_sum else y


class _ColumnSumTap(torch.autograd.Function):
    """Identity on ``x`` whose backward also hands the column sums of the gradient to ``bias`` (PyTorch path of
    ``layer_norm(..., producer_bias=...)``)."""

    @staticmethod
    def forward(ctx, x, bias):
        ctx.bias_dtype = bias.dtype
        return x.view_as(x)

    @staticmethod
    def backward(ctx, dx):
        return dx, dx.reshape(-1, dx.shape[-1]).sum(0, dtype=torch.float32).to(ctx.bias_dtype)


class _BiasGeluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias):
        h = x.shape[-1]
        x2 = x.reshape(-1, h).contiguous()
        rows = x2.shape[0]
        lib = _lib.load_library()
        y = torch.empty_like(x2)
        b32 = bias.detach().to(torch.float32).contiguous() if bias is not None else None
        with torch.cuda.device(x.device):
            code = lib.hm_bias_gelu_fwd(_lib.ptr(x2), _lib.ptr(b32), _lib.ptr(y), ctypes.c_longlong(rows), h,
                                        _lib.dtype_code(x.dtype), _lib.sm_count(x.device), _lib.stream_ptr(x.device))
        _lib.check(code, "hm_bias_gelu_fwd")
        ctx.save_for_backward(x2, b32)
        ctx.shape = x.shape
        ctx.bias_dtype = bias.dtype if bias is not None else None
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, b32 = ctx.saved_tensors
        h = x2.shape[-1]
        rows = x2.shape[0]
        dy2 = dy.reshape(-1, h).contiguous()
        if dy2.dtype != x2.dtype:
            dy2 = dy2.to(x2.dtype)
        lib = _lib.load_library()
        dx = torch.empty_like(x2)
        db = torch.zeros(h, dtype=torch.float32, device=x2.device) if b32 is not None else None
        with torch.cuda.device(x2.device):
            code = lib.hm_bias_gelu_bwd(_lib.ptr(dy2), _lib.ptr(x2), _lib.ptr(b32), _lib.ptr(dx), _lib.ptr(db),
                                        ctypes.c_longlong(rows), h, _lib.dtype_code(x2.dtype),
                                        _lib.sm_count(x2.device), _lib.stream_ptr(x2.device))
        _lib.check(code, "hm_bias_gelu_bwd")
        return dx.view(ctx.shape), (db.to(ctx.bias_dtype) if db is not None else None)


def bias_gelu(x: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``gelu_tanh(x + bias)`` over the last dimension."""
    h = x.shape[-1]
    if _lib.use_kernels(x) and x.dtype in (torch.bfloat16, torch.float32) and h % 8 == 0:
        return _BiasGeluFn.apply(x, bias)
    z = x if bias is None else x + bias.to(x.dtype)
    return gelu_tanh_reference(z)

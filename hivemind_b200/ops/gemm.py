"""tcgen05 tensor-core GEMM with fused epilogues, and the autograd ``linear`` built on it.

``tc_gemm`` drives ``csrc/tc_gemm.cu`` (TMA-fed ``tcgen05.mma`` with TMEM accumulators). On CPU tensors the same
function evaluates the PyTorch formula, which is what the GPU tests compare against.

``linear(x, weight, bias, activation)`` is the building block of the expert FFN
(hivemind/moe/server/layers/common.py:17-30) and of the ALBERT / GPT-2 shaped models: forward, input-gradient and
weight-gradient GEMMs all run on the kernel without transposed copies, the bias and tanh-GELU are fused in the forward
epilogue, and weight gradients are accumulated in fp32 by TMA reduce-add (directly into ``weight.grad`` when that
buffer already exists, which also sums the uses of a shared weight and successive micro-batches).
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional

import torch
import torch.nn.functional as F

from hivemind_b200.ops import _lib

EPI_NONE, EPI_BIAS, EPI_BIAS_GELU = 0, 1, 2
_err_flags: Dict[int, torch.Tensor] = {}


def _err_flag(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    flag = _err_flags.get(idx)
    if flag is None:
        flag = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _err_flags[idx] = flag
    return flag


def check_kernel_errors() -> None:
    """Raise if any tensor-core kernel of this process recorded a bounded wait that ran out (synchronises)."""
    for idx, flag in _err_flags.items():
        code = int(flag.item())
        if code:
            flag.zero_()
            raise RuntimeError(f"tc_gemm on cuda:{idx}: a bounded wait ran out (role code {code}); results are invalid")


_PAIR_DEFAULT = os.environ.get("HIVEMIND_B200_GEMM_PAIR", "0") == "1"  # opt-in until validated everywhere


def _pick_block_n(n: int, m: int, tf32: bool, sms: int) -> int:
    options = (128, 64, 32) if tf32 else (256, 128, 64)
    for bn in options:
        if n >= bn and ((m + 127) // 128) * ((n + bn - 1) // bn) >= sms:
            return bn
    for bn in options:  # few tiles: take the largest tile that N fills
        if n >= bn:
            return bn
    return options[-1]


def tc_gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
            out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
            bias: Optional[torch.Tensor] = None, gelu: bool = False, aux: Optional[torch.Tensor] = None,
            reduce_add: bool = False, splits: int = 1, alpha: float = 1.0,
            block_n: Optional[int] = None, pair: Optional[bool] = None) -> torch.Tensor:
    """``D[M,N] = epi(alpha * sum_k A(m,k) B(n,k))``.

    :param a: ``[M, K]`` (or ``[K, M]`` when ``a_mn``), bf16 or fp32 (fp32 is multiplied as tf32)
    :param b: ``[N, K]`` (or ``[K, N]`` when ``b_mn``), same dtype as ``a``
    :param out: destination ``[M, N]`` (bf16 or fp32); with ``reduce_add`` the result is added to it (fp32 only)
    :param bias: fp32 ``[N]`` added before the optional tanh-GELU; ``aux`` (bf16) receives the pre-GELU values
    :param splits: split-K factor (needs ``reduce_add``)
    :param pair: use the two-CTA kernel (one 256x256 tile per pair of SMs, bf16 only); default: when the problem
      has at least one full 256x256 tile and ``HIVEMIND_B200_GEMM_PAIR`` is not ``0``
    """
    assert a.dim() == 2 and b.dim() == 2 and a.dtype == b.dtype
    m, k = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    n, kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    assert k == kb, f"contraction mismatch: {k} vs {kb}"
    if out is None:
        out_dtype = out_dtype or (torch.float32 if (reduce_add or a.dtype == torch.float32) else torch.bfloat16)
        out = (torch.zeros if reduce_add else torch.empty)((m, n), dtype=out_dtype, device=a.device)
    assert out.shape == (m, n)
    if not _lib.use_kernels(a, b, out):
        af = (a.t() if a_mn else a).to(torch.float32)
        bf = (b.t() if b_mn else b).to(torch.float32)
        res = alpha * (af @ bf.t())
        if bias is not None:
            res = res + bias.to(torch.float32)
        if aux is not None:
            aux.copy_(res)
        if gelu:
            res = F.gelu(res, approximate="tanh")
        if reduce_add:
            out.add_(res.to(out.dtype))
        else:
            out.copy_(res)
        return out

    tf32 = a.dtype == torch.float32
    assert a.dtype in (torch.float32, torch.bfloat16), "tc_gemm operands must be bf16 or fp32"
    assert out.dtype in (torch.float32, torch.bfloat16)
    assert a.stride(1) == 1 and b.stride(1) == 1 and out.stride(1) == 1, "innermost dimension must be contiguous"
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == n
    if aux is not None:
        assert aux.dtype == torch.bfloat16 and aux.shape == (m, n) and aux.stride(1) == 1
    lib = _lib.load_library()
    sms = _lib.sm_count(a.device)
    if block_n is None:
        block_n = _pick_block_n(n, m, tf32, sms)
    epi = EPI_BIAS_GELU if gelu else (EPI_BIAS if bias is not None else EPI_NONE)
    if pair is None:
        pair = _PAIR_DEFAULT and not tf32 and m >= 256 and n >= 256 and block_n == 256
    if pair:
        assert not tf32, "the two-CTA kernel multiplies bf16 operands"
        with torch.cuda.device(a.device):
            code = lib.hm_tc_gemm_pair(
                _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.ptr(aux), _lib.ptr(bias), m, n, k,
                ctypes.c_longlong(a.stride(0)), ctypes.c_longlong(b.stride(0)), ctypes.c_longlong(out.stride(0)),
                ctypes.c_longlong(aux.stride(0) if aux is not None else 0), int(a_mn), int(b_mn),
                int(out.dtype == torch.float32), epi, int(reduce_add), splits, ctypes.c_float(alpha),
                _lib.ptr(_err_flag(a.device)), sms, _lib.stream_ptr(a.device))
        _lib.check(code, "hm_tc_gemm_pair")
        return out
    with torch.cuda.device(a.device):
        code = lib.hm_tc_gemm(
            _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.ptr(aux), _lib.ptr(bias), m, n, k,
            ctypes.c_longlong(a.stride(0)), ctypes.c_longlong(b.stride(0)), ctypes.c_longlong(out.stride(0)),
            ctypes.c_longlong(aux.stride(0) if aux is not None else 0), int(a_mn), int(b_mn), int(tf32),
            int(out.dtype == torch.float32), epi, int(reduce_add), splits, ctypes.c_float(alpha), block_n,
            _lib.ptr(_err_flag(a.device)), sms, _lib.stream_ptr(a.device))
    _lib.check(code, "hm_tc_gemm")
    return out


def colsum_(out: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """``out[c] += sum_r x[r, c]`` (fp32 ``out``; ``x`` bf16 or fp32 with contiguous rows)."""
    assert x.dim() == 2 and out.dtype == torch.float32
    if not _lib.use_kernels(x, out):
        out.add_(x.to(torch.float32).sum(0))
        return out
    assert x.stride(1) == 1
    lib = _lib.load_library()
    with torch.cuda.device(x.device):
        code = lib.hm_colsum(_lib.ptr(x), _lib.ptr(out), ctypes.c_longlong(x.shape[0]), x.shape[1],
                             ctypes.c_longlong(x.stride(0)), _lib.dtype_code(x.dtype), _lib.sm_count(x.device),
                             _lib.stream_ptr(x.device))
    _lib.check(code, "hm_colsum")
    return out


def _split_k_for(m: int, n: int, k: int, sms: int, pair: bool = False) -> int:
    """
    Split factor of a weight-gradient GEMM's contraction. Work items (tiles x splits) run in waves of ``sms``; an item
    costs its share of K plus a fixed epilogue (an fp32 128x256 reduce-add, about as long as 1024 elements of K).
    Picks the factor with the shortest estimated time, e.g. 3 for 96 tiles on 148 SMs (two full waves instead of
    one wave that leaves a third of the GPU idle).
    """
    if pair:  # the two-CTA kernel works on 256x256 tiles, one per pair of SMs
        tiles, sms = ((m + 255) // 256) * ((n + 255) // 256), max(sms // 2, 1)
    else:
        tiles = ((m + 127) // 128) * ((n + 255) // 256 if n >= 256 else 1)
    if tiles <= 0:
        return 1
    epilogue, best, best_cost = 1024.0, 1, None
    for splits in range(1, 17):
        if splits > 1 and k // splits < 512:
            break
        waves = -(-tiles * splits // sms)
        cost = waves * (k / splits + epilogue)
        if best_cost is None or cost < best_cost * 0.97:  # prefer fewer splits unless the gain is clear
            best, best_cost = splits, cost
    return best


class _LinearFn(torch.autograd.Function):
    """y = act(x W^T + b) with bf16 tensor-core GEMMs and fp32 weight-gradient accumulation."""

    @staticmethod
    def forward(ctx, x, weight, bias, weight_lp, activation, skip_bias_grad=False):
        ctx.skip_bias_grad = skip_bias_grad
        in_f = x.shape[-1]
        x2 = x.reshape(-1, in_f)
        if x2.dtype != torch.bfloat16:
            x2 = x2.to(torch.bfloat16)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        w = weight_lp if weight_lp is not None else weight.detach().to(torch.bfloat16)
        b32 = None
        if bias is not None:
            b32 = bias.detach() if bias.dtype == torch.float32 else bias.detach().to(torch.float32)
        gelu = activation == "gelu"
        need_grad = any(ctx.needs_input_grad[:3])
        pre = torch.empty((x2.shape[0], w.shape[0]), dtype=torch.bfloat16, device=x.device) if (gelu and need_grad) else None
        y = tc_gemm(x2, w, bias=b32, gelu=gelu, aux=pre, out_dtype=torch.bfloat16)
        ctx.save_for_backward(x2, w, pre)
        ctx.weight = weight
        ctx.bias = bias
        ctx.x_shape = x.shape
        ctx.x_dtype = x.dtype
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from hivemind_b200.ops.norm_act import _BiasGeluFn  # noqa: F401  (kernel shared with bias_gelu)
        x2, w, pre = ctx.saved_tensors
        weight, bias = ctx.weight, ctx.bias
        out_f = w.shape[0]
        dy2 = dy.reshape(-1, out_f)
        if dy2.dtype != torch.bfloat16:
            dy2 = dy2.to(torch.bfloat16)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        lib = _lib.load_library()
        dev = x2.device
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        need_b = bias is not None and ctx.needs_input_grad[2] and not ctx.skip_bias_grad
        grad_b = None
        if need_b:
            use_b_buf = bias.grad is not None and bias.grad.dtype == torch.float32 and bias.grad.is_contiguous()
            gb = bias.grad if use_b_buf else torch.zeros(out_f, dtype=torch.float32, device=dev)
        if pre is not None:
            # d(pre) = dy * gelu'(pre); the same kernel also accumulates the bias gradient column sums
            dpre = torch.empty_like(pre)
            with torch.cuda.device(dev):
                code = lib.hm_bias_gelu_bwd(_lib.ptr(dy2), _lib.ptr(pre), _lib.ptr(None), _lib.ptr(dpre),
                                            _lib.ptr(gb if need_b else None), ctypes.c_longlong(pre.shape[0]), out_f,
                                            _lib.HM_BF16, _lib.sm_count(dev), _lib.stream_ptr(dev))
            _lib.check(code, "hm_bias_gelu_bwd")
            dy2 = dpre
        elif need_b:
            colsum_(gb, dy2)
        if need_b:
            grad_b = None if use_b_buf else gb.to(bias.dtype)
        grad_x = None
        if need_x:
            grad_x = tc_gemm(dy2, w, b_mn=True, out_dtype=torch.bfloat16).view(ctx.x_shape)
            if grad_x.dtype != ctx.x_dtype:
                grad_x = grad_x.to(ctx.x_dtype)
        grad_w = None
        if need_w:
            tokens = dy2.shape[0]
            # weight gradients contract over all tokens with both operands MN-major: the two-CTA kernel is about
            # 1.5x faster than the one-CTA kernel on these (1280 vs 800 TFLOP/s for 4096 x 1024 x 16384)
            use_pair = out_f >= 256 and x2.shape[1] >= 256
            splits = _split_k_for(out_f, x2.shape[1], tokens, _lib.sm_count(dev), pair=use_pair)
            use_w_buf = weight.grad is not None and weight.grad.dtype == torch.float32 and weight.grad.is_contiguous()
            gw = weight.grad if use_w_buf else torch.zeros(weight.shape, dtype=torch.float32, device=dev)
            tc_gemm(dy2, x2, a_mn=True, b_mn=True, out=gw, reduce_add=True, splits=splits, pair=use_pair)
            grad_w = None if use_w_buf else gw.to(weight.dtype)
        return grad_x, grad_w, grad_b, None, None, None


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           activation: Optional[str] = None, weight_lp: Optional[torch.Tensor] = None,
           skip_bias_grad: bool = False) -> torch.Tensor:
    """``act(x @ weight.T + bias)`` with ``activation`` in (None, "gelu") (tanh-GELU).

    ``weight`` is the (fp32 or bf16) parameter that receives the gradient; ``weight_lp`` is an optional
    up-to-date bf16 copy of it, which saves the cast. CUDA inputs run on the tcgen05 kernel in bf16 with fp32
    accumulation; CPU inputs run the PyTorch formula in the input dtype.

    ``skip_bias_grad``: the caller obtains the bias gradient elsewhere (``layer_norm(..., producer_bias=bias)`` takes
    it in the pass that produces this layer's output gradient), so this call leaves ``bias.grad`` alone.
    """
    in_f, out_f = weight.shape[1], weight.shape[0]
    if _lib.use_kernels(x, weight) and in_f % 8 == 0 and out_f % 8 == 0:
        return _LinearFn.apply(x, weight, bias, weight_lp, activation, skip_bias_grad)
    if bias is not None and skip_bias_grad:
        bias = bias.detach()
    y = F.linear(x, weight.to(x.dtype), None if bias is None else bias.to(x.dtype))
    return F.gelu(y, approximate="tanh") if activation == "gelu" else y

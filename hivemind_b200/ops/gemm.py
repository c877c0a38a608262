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
            block_n: Optional[int] = None, pair: Optional[bool] = None, add: Optional[torch.Tensor] = None,
            add_is_gelu_input: bool = False) -> torch.Tensor:
    """``D[M,N] = epi(alpha * sum_k A(m,k) B(n,k))``.

    :param a: ``[M, K]`` (or ``[K, M]`` when ``a_mn``), bf16 or fp32 (fp32 is multiplied as tf32)
    :param b: ``[N, K]`` (or ``[K, N]`` when ``b_mn``), same dtype as ``a``
    :param out: destination ``[M, N]`` (bf16 or fp32); with ``reduce_add`` the result is added to it (fp32 only)
    :param bias: fp32 ``[N]`` added before the optional tanh-GELU; ``aux`` (bf16) receives the pre-GELU values
    :param add: bf16 ``[M, N]`` added to the result in the epilogue (bf16 output, no GELU, one-CTA kernel); with
      ``add_is_gelu_input`` the result is instead multiplied by ``gelu_tanh'(add)`` (backward through a GELU)
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
        if add is not None and add_is_gelu_input:
            z = add.to(torch.float32).requires_grad_()
            with torch.enable_grad():
                (dz,) = torch.autograd.grad(F.gelu(z, approximate="tanh").sum(), z)
            res = res * dz
        elif add is not None:
            res = res + add.to(torch.float32)
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
    if add is not None:
        assert not tf32 and not gelu and aux is None and not reduce_add and out.dtype == torch.bfloat16 and not pair
        assert add.dtype == torch.bfloat16 and add.shape == (m, n) and add.stride(1) == 1
        with torch.cuda.device(a.device):
            code = lib.hm_tc_gemm_add(
                _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.ptr(add), _lib.ptr(bias), m, n, k,
                ctypes.c_longlong(a.stride(0)), ctypes.c_longlong(b.stride(0)), ctypes.c_longlong(out.stride(0)),
                ctypes.c_longlong(add.stride(0)), int(a_mn), int(b_mn), epi, int(add_is_gelu_input),
                ctypes.c_float(alpha), block_n,
                _lib.ptr(_err_flag(a.device)), sms, _lib.stream_ptr(a.device))
        _lib.check(code, "hm_tc_gemm_add")
        return out
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


def _as_rows(t: torch.Tensor, width: int) -> torch.Tensor:
    """``t`` as a contiguous bf16 matrix with ``width`` columns."""
    t2 = t.reshape(-1, width)
    if t2.dtype != torch.bfloat16:
        t2 = t2.to(torch.bfloat16)
    return t2 if t2.is_contiguous() else t2.contiguous()


def _weight_grad(weight: torch.Tensor, dy2: torch.Tensor, x2: torch.Tensor) -> Optional[torch.Tensor]:
    """``dW = dy2^T x2`` accumulated in fp32. With an fp32 ``weight.grad`` in place the GEMM adds straight into it and
    None is returned (nothing is left for autograd to accumulate); otherwise the gradient is returned."""
    out_f, in_f, tokens = dy2.shape[1], x2.shape[1], dy2.shape[0]
    # weight gradients contract over all tokens with both operands MN-major: the two-CTA kernel is about
    # 1.5x faster than the one-CTA kernel on these (1280 vs 800 TFLOP/s for 4096 x 1024 x 16384)
    use_pair = out_f >= 256 and in_f >= 256
    splits = _split_k_for(out_f, in_f, tokens, _lib.sm_count(dy2.device), pair=use_pair)
    in_place = weight.grad is not None and weight.grad.dtype == torch.float32 and weight.grad.is_contiguous()
    gw = weight.grad if in_place else torch.zeros(weight.shape, dtype=torch.float32, device=dy2.device)
    tc_gemm(dy2, x2, a_mn=True, b_mn=True, out=gw, reduce_add=True, splits=splits, pair=use_pair)
    return None if in_place else gw.to(weight.dtype)


def _bias_grad_buffer(bias: torch.Tensor, width: int, device: torch.device):
    """fp32 buffer that column-sum kernels add the bias gradient to, and whether it is ``bias.grad`` itself."""
    in_place = bias.grad is not None and bias.grad.dtype == torch.float32 and bias.grad.is_contiguous()
    return (bias.grad if in_place else torch.zeros(width, dtype=torch.float32, device=device)), in_place


def _skip_rows(dskip: Optional[torch.Tensor], width: int) -> Optional[torch.Tensor]:
    """The gradient that came back through a passed-through input, as the bf16 matrix the GEMM epilogue adds."""
    if dskip is None:
        return None
    skip2 = dskip.reshape(-1, width)
    if skip2.dtype != torch.bfloat16 or skip2.stride(1) != 1 or skip2.stride(0) % 8 != 0:
        skip2 = skip2.to(torch.bfloat16).contiguous()
    return skip2


class _LinearFn(torch.autograd.Function):
    """y = act(x W^T + b) with bf16 tensor-core GEMMs and fp32 weight-gradient accumulation."""

    @staticmethod
    def forward(ctx, x, weight, bias, weight_lp, activation, skip_bias_grad=False, passthrough=False):
        ctx.skip_bias_grad = skip_bias_grad
        ctx.set_materialize_grads(False)
        x2 = _as_rows(x, x.shape[-1])
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
        y = y.view(*x.shape[:-1], w.shape[0])
        return (y, x.view_as(x)) if passthrough else y

    @staticmethod
    def backward(ctx, dy, dskip=None):
        if dy is None:  # only the passed-through input was used downstream
            return dskip, None, None, None, None, None, None
        x2, w, pre = ctx.saved_tensors
        weight, bias = ctx.weight, ctx.bias
        out_f = w.shape[0]
        dy2 = _as_rows(dy, out_f)
        lib = _lib.load_library()
        dev = x2.device
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        need_b = bias is not None and ctx.needs_input_grad[2] and not ctx.skip_bias_grad
        grad_b = None
        if need_b:
            gb, b_in_place = _bias_grad_buffer(bias, out_f, dev)
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
            grad_b = None if b_in_place else gb.to(bias.dtype)
        grad_x = None
        if need_x:
            # the gradient that arrived through the passed-through input is added in the GEMM's epilogue
            skip2 = _skip_rows(dskip, x2.shape[1])
            grad_x = tc_gemm(dy2, w, b_mn=True, out_dtype=torch.bfloat16, add=skip2, pair=False if skip2 is not None else None)
            grad_x = grad_x.view(ctx.x_shape)
            if grad_x.dtype != ctx.x_dtype:
                grad_x = grad_x.to(ctx.x_dtype)
        elif dskip is not None:
            grad_x = dskip
        grad_w = _weight_grad(weight, dy2, x2) if need_w else None
        return grad_x, grad_w, grad_b, None, None, None, None


class _FeedForwardFn(torch.autograd.Function):
    """``gelu(x W1^T + b1) W2^T + b2`` as ONE autograd node: the backward pass applies the GELU derivative in place on
    the hidden gradient (one pass that also yields ``b1``'s gradient), adds the gradient of a passed-through input in
    the epilogue of the input-gradient GEMM, and leaves ``b2``'s gradient to the LayerNorm behind the block."""

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, w1_lp, w2_lp, skip_out_bias_grad, passthrough):
        ctx.set_materialize_grads(False)
        ctx.skip_out_bias_grad = skip_out_bias_grad
        x2 = _as_rows(x, x.shape[-1])
        w1b = w1_lp if w1_lp is not None else w1.detach().to(torch.bfloat16)
        w2b = w2_lp if w2_lp is not None else w2.detach().to(torch.bfloat16)
        pre = torch.empty((x2.shape[0], w1b.shape[0]), dtype=torch.bfloat16, device=x.device)
        inter = tc_gemm(x2, w1b, bias=b1.detach().to(torch.float32), gelu=True, aux=pre, out_dtype=torch.bfloat16)
        out = tc_gemm(inter, w2b, bias=b2.detach().to(torch.float32), out_dtype=torch.bfloat16)
        ctx.save_for_backward(x2, w1b, w2b, pre, inter)
        ctx.params = (w1, b1, w2, b2)
        ctx.x_shape, ctx.x_dtype = x.shape, x.dtype
        out = out.view(*x.shape[:-1], w2b.shape[0])
        return (out, x.view_as(x)) if passthrough else out

    @staticmethod
    def backward(ctx, dout, dskip=None):
        if dout is None:
            return (dskip,) + (None,) * 8
        x2, w1b, w2b, pre, inter = ctx.saved_tensors
        w1, b1, w2, b2 = ctx.params
        need = ctx.needs_input_grad
        dev = x2.device
        dout2 = _as_rows(dout, w2b.shape[0])
        grad_b2 = None
        if need[4] and not ctx.skip_out_bias_grad:
            gb2, in_place = _bias_grad_buffer(b2, w2b.shape[0], dev)
            colsum_(gb2, dout2)
            grad_b2 = None if in_place else gb2.to(b2.dtype)
        # gradient of the pre-activations: (dout W2) * gelu'(pre). The derivative runs as its own pass over the GEMM's
        # output (in place, with the column sums for b1 taken along the way): applied in the GEMM's epilogue it made
        # that epilogue longer than the tile's MMAs (0.21 ms instead of 0.11 + 0.04 ms on 16384 x 4096 x 1024)
        dpre = tc_gemm(dout2, w2b, b_mn=True, out_dtype=torch.bfloat16)
        grad_w2 = _weight_grad(w2, dout2, inter) if need[3] else None
        grad_b1, gb1, in_place = None, None, False
        if need[2]:
            gb1, in_place = _bias_grad_buffer(b1, w1b.shape[0], dev)
        lib = _lib.load_library()
        with torch.cuda.device(dev):
            code = lib.hm_bias_gelu_bwd(_lib.ptr(dpre), _lib.ptr(pre), _lib.ptr(None), _lib.ptr(dpre), _lib.ptr(gb1),
                                        ctypes.c_longlong(pre.shape[0]), w1b.shape[0], _lib.HM_BF16,
                                        _lib.sm_count(dev), _lib.stream_ptr(dev))
        _lib.check(code, "hm_bias_gelu_bwd")
        if need[2]:
            grad_b1 = None if in_place else gb1.to(b1.dtype)
        grad_x = None
        if need[0]:
            skip2 = _skip_rows(dskip, x2.shape[1])
            grad_x = tc_gemm(dpre, w1b, b_mn=True, out_dtype=torch.bfloat16, add=skip2,
                             pair=False if skip2 is not None else None).view(ctx.x_shape)
            if grad_x.dtype != ctx.x_dtype:
                grad_x = grad_x.to(ctx.x_dtype)
        elif dskip is not None:
            grad_x = dskip
        grad_w1 = _weight_grad(w1, dpre, x2) if need[1] else None
        return grad_x, grad_w1, grad_b1, grad_w2, grad_b2, None, None, None, None


def feed_forward(x: torch.Tensor, w1: torch.Tensor, b1: torch.Tensor, w2: torch.Tensor, b2: torch.Tensor, *,
                 w1_lp: Optional[torch.Tensor] = None, w2_lp: Optional[torch.Tensor] = None,
                 skip_out_bias_grad: bool = False, passthrough: bool = False):
    """``gelu_tanh(x @ w1.T + b1) @ w2.T + b2``. On CUDA this is one autograd node (four GEMMs forward and backward
    plus two column sums); elsewhere it is two ``linear`` calls. ``skip_out_bias_grad`` and ``passthrough`` mean what
    they mean for ``linear``: ``b2``'s gradient is taken by the LayerNorm that follows, and the returned copy of ``x``
    carries the residual connection's gradient into the input-gradient GEMM."""
    if _lib.use_kernels(x, w1, w2) and all(d % 8 == 0 for d in (*w1.shape, *w2.shape)):
        return _FeedForwardFn.apply(x, w1, b1, w2, b2, w1_lp, w2_lp, skip_out_bias_grad, passthrough)
    inter = linear(x, w1, b1, activation="gelu", weight_lp=w1_lp)
    out = linear(inter, w2, b2, weight_lp=w2_lp, skip_bias_grad=skip_out_bias_grad)
    return (out, x) if passthrough else out


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           activation: Optional[str] = None, weight_lp: Optional[torch.Tensor] = None,
           skip_bias_grad: bool = False, passthrough: bool = False):
    """``act(x @ weight.T + bias)`` with ``activation`` in (None, "gelu") (tanh-GELU).

    ``weight`` is the (fp32 or bf16) parameter that receives the gradient; ``weight_lp`` is an optional
    up-to-date bf16 copy of it, which saves the cast. CUDA inputs run on the tcgen05 kernel in bf16 with fp32
    accumulation; CPU inputs run the PyTorch formula in the input dtype.

    ``skip_bias_grad``: the caller obtains the bias gradient elsewhere (``layer_norm(..., producer_bias=bias)`` takes
    it in the pass that produces this layer's output gradient), so this call leaves ``bias.grad`` alone.

    ``passthrough``: return ``(y, x)``. Use the returned ``x`` for the residual connection around the layer: the
    gradient that comes back through it is then added inside the input-gradient GEMM instead of by a separate pass.
    """
    in_f, out_f = weight.shape[1], weight.shape[0]
    if _lib.use_kernels(x, weight) and in_f % 8 == 0 and out_f % 8 == 0:
        return _LinearFn.apply(x, weight, bias, weight_lp, activation, skip_bias_grad, passthrough)
    if bias is not None and skip_bias_grad:
        bias = bias.detach()
    y = F.linear(x, weight.to(x.dtype), None if bias is None else bias.to(x.dtype))
    y = F.gelu(y, approximate="tanh") if activation == "gelu" else y
    return (y, x) if passthrough else y

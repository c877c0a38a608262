"""Many ``ffn`` experts in a handful of launches: ``LayerNorm(x + W2_e gelu_tanh(W1_e x + b1_e) + b2_e)`` for the
rows of every expert ``e`` of an aligned ``ops.moe.dispatch`` (each expert owns whole 128-row tiles).

The block is the reference's ``ffn`` expert (hivemind/moe/server/layers/common.py:11-30) and its training step is
what the reference's ``ModuleBackend.backward`` does per expert (hivemind/moe/server/module_backend.py:106-154).
On CUDA the two products of all experts run as ONE grouped tcgen05 GEMM each (the M-tile table selects the
expert's weights; bias + GELU in the first epilogue), residual + LayerNorm is one grouped kernel, and the backward
pass is five grouped launches (LayerNorm backward with the bias-2 column sums, two data-gradient GEMMs, GELU
backward with the bias-1 column sums, two weight-gradient GEMMs that add straight into the fp32 ``.grad``).
Nothing here reads a row count on the host: rows of tiles that no expert owns are skipped on the device.
On CPU the same math runs per expert in PyTorch (the oracle of the GPU tests).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from hivemind_b200.ops import _lib
from hivemind_b200.ops.gemm import EPI_BIAS, EPI_BIAS_GELU, EPI_NONE, _err_flag

LN_EPS = 1e-12


def tc_gemm_grouped(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, table: torch.Tensor, *, mode: int,
                    num_groups: int, m: int, n: int, k: int, a_mn: bool = False, b_mn: bool = False,
                    bias: Optional[torch.Tensor] = None, gelu: bool = False, aux: Optional[torch.Tensor] = None,
                    reduce_add: bool = False, block_n: Optional[int] = None) -> torch.Tensor:
    """
    Grouped bf16 GEMM on the tcgen05 kernel.

    mode 1 (rows grouped): ``a`` is ``[m, k]``, ``out`` ``[m, n]``, ``table[m // 128]`` names the group of each
    M tile (-1 = skip) and ``b`` stacks the groups' ``[n, k]`` (or, with ``b_mn``, ``[k, n]``) matrices.
    mode 2 (K grouped): ``a`` is ``[k, m]`` and ``b`` ``[k, n]`` (both MN-major), group ``g`` contracts rows
    ``table[g]:table[g+1]`` and writes (or adds to) ``out[g*m:(g+1)*m]``.
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and table.dtype == torch.int32
    assert a.stride(-1) == 1 and b.stride(-1) == 1 and out.stride(-1) == 1
    lib = _lib.load_library()
    sms = _lib.sm_count(a.device)
    if mode == 2 and a_mn and b_mn and bias is None and aux is None and m % 256 == 0 and n >= 256:
        # weight gradients: the two-CTA kernel is about 1.5x faster on MN-major x MN-major products
        out2 = out.view(-1, out.shape[-1])
        with torch.cuda.device(a.device):
            code = lib.hm_tc_gemm_pair_grouped_k(
                _lib.ptr(a), _lib.ptr(b), _lib.ptr(out2), m, n, k, ctypes.c_longlong(a.stride(-2)),
                ctypes.c_longlong(b.stride(-2)), ctypes.c_longlong(out2.stride(0)), int(out.dtype == torch.float32),
                int(reduce_add), ctypes.c_float(1.0), _lib.ptr(_err_flag(a.device)), sms, num_groups, _lib.ptr(table),
                _lib.stream_ptr(a.device))
        _lib.check(code, "hm_tc_gemm_pair_grouped_k")
        return out
    if block_n is None:
        block_n = 256 if n >= 256 else (128 if n >= 128 else 64)
    epi = EPI_BIAS_GELU if gelu else (EPI_BIAS if bias is not None else EPI_NONE)
    out2 = out.view(-1, out.shape[-1])
    with torch.cuda.device(a.device):
        code = lib.hm_tc_gemm_grouped(
            _lib.ptr(a), _lib.ptr(b), _lib.ptr(out2), _lib.ptr(aux), _lib.ptr(bias), m, n, k,
            ctypes.c_longlong(a.stride(-2)), ctypes.c_longlong(b.stride(-2)), ctypes.c_longlong(out2.stride(0)),
            ctypes.c_longlong(aux.stride(0) if aux is not None else 0), int(a_mn), int(b_mn),
            int(out.dtype == torch.float32), epi, int(reduce_add), ctypes.c_float(1.0), block_n,
            _lib.ptr(_err_flag(a.device)), sms, mode, num_groups, _lib.ptr(table), _lib.stream_ptr(a.device))
    _lib.check(code, "hm_tc_gemm_grouped")
    return out


def _grad_buffer(p: torch.Tensor) -> torch.Tensor:
    """The fp32 ``.grad`` of a parameter, created as zeros if absent: gradients are accumulated into it in place."""
    if p.grad is None:
        p.grad = torch.zeros_like(p, dtype=torch.float32)
    assert p.grad.dtype == torch.float32 and p.grad.is_contiguous()
    return p.grad


class _GroupedFFNFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tile_group, offsets, module):
        rows, hidden = x.shape
        experts, inner = module.w1.shape[0], module.w1.shape[1]
        w1, w2 = module.low_precision_weights()
        lib = _lib.load_library()
        dev = x.device
        need_grad = ctx.needs_input_grad[0] or module.w1.requires_grad  # pre-GELU values are kept for backward
        pre = torch.empty(rows, inner, dtype=torch.bfloat16, device=dev) if need_grad else None
        act = torch.empty(rows, inner, dtype=torch.bfloat16, device=dev)
        tc_gemm_grouped(x, w1.view(experts * inner, hidden), act, tile_group, mode=1, num_groups=experts, m=rows,
                        n=inner, k=hidden, bias=module.b1.detach(), gelu=True, aux=pre)
        proj = torch.empty(rows, hidden, dtype=torch.bfloat16, device=dev)
        tc_gemm_grouped(act, w2.view(experts * hidden, inner), proj, tile_group, mode=1, num_groups=experts, m=rows,
                        n=hidden, k=inner, bias=module.b2.detach())
        y = torch.zeros_like(x)  # rows of unowned tiles stay zero
        z = torch.empty_like(x)
        mean = torch.empty(rows, dtype=torch.float32, device=dev)
        rstd = torch.empty(rows, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            code = lib.hm_layernorm_fwd_grouped(_lib.ptr(proj), _lib.ptr(x), _lib.ptr(module.gamma.detach()),
                                                _lib.ptr(module.beta.detach()), _lib.ptr(y), _lib.ptr(z),
                                                _lib.ptr(mean), _lib.ptr(rstd), rows, hidden, ctypes.c_float(LN_EPS),
                                                _lib.HM_BF16, _lib.ptr(tile_group), _lib.sm_count(dev),
                                                _lib.stream_ptr(dev))
        _lib.check(code, "hm_layernorm_fwd_grouped")
        ctx.save_for_backward(x, pre, act, z, mean, rstd, tile_group, offsets, w1, w2)
        ctx.module = module
        return y

    @staticmethod
    def backward(ctx, dy):
        x, pre, act, z, mean, rstd, tile_group, offsets, w1, w2 = ctx.saved_tensors
        module = ctx.module
        rows, hidden = x.shape
        experts, inner = module.w1.shape[0], module.w1.shape[1]
        lib = _lib.load_library()
        dev = x.device
        dy = dy.contiguous()
        train = module.w1.requires_grad
        g_w1, g_b1, g_w2, g_b2 = (_grad_buffer(p) if train else None for p in (module.w1, module.b1, module.w2, module.b2))
        g_gamma, g_beta = (_grad_buffer(p) if train else None for p in (module.gamma, module.beta))
        dz = torch.zeros_like(x)
        with torch.cuda.device(dev):
            code = lib.hm_layernorm_bwd_grouped(_lib.ptr(dy), _lib.ptr(z), _lib.ptr(module.gamma.detach()),
                                                _lib.ptr(mean), _lib.ptr(rstd), _lib.ptr(dz), _lib.ptr(g_gamma),
                                                _lib.ptr(g_beta), _lib.ptr(g_b2), rows, hidden, _lib.HM_BF16,
                                                _lib.ptr(tile_group), _lib.sm_count(dev), _lib.stream_ptr(dev))
        _lib.check(code, "hm_layernorm_bwd_grouped")
        if train:  # dW2[e] += dz_e^T act_e
            tc_gemm_grouped(dz, act, g_w2, offsets, mode=2, num_groups=experts, m=hidden, n=inner, k=rows,
                            a_mn=True, b_mn=True, reduce_add=True)
        dact = torch.empty(rows, inner, dtype=torch.bfloat16, device=dev)  # dz W2
        tc_gemm_grouped(dz, w2.view(experts * hidden, inner), dact, tile_group, mode=1, num_groups=experts, m=rows,
                        n=inner, k=hidden, b_mn=True)
        dpre = dact  # in place: the kernel reads and writes the same element
        with torch.cuda.device(dev):
            code = lib.hm_gelu_bwd_grouped(_lib.ptr(dact), _lib.ptr(pre), _lib.ptr(dpre), _lib.ptr(g_b1),
                                           ctypes.c_longlong(rows), inner, _lib.HM_BF16, _lib.ptr(tile_group),
                                           _lib.stream_ptr(dev))
        _lib.check(code, "hm_gelu_bwd_grouped")
        if train:  # dW1[e] += dpre_e^T x_e
            tc_gemm_grouped(dpre, x, g_w1, offsets, mode=2, num_groups=experts, m=inner, n=hidden, k=rows,
                            a_mn=True, b_mn=True, reduce_add=True)
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.zeros_like(x)
            tc_gemm_grouped(dpre, w1.view(experts * inner, hidden), dx, tile_group, mode=1, num_groups=experts,
                            m=rows, n=hidden, k=inner, b_mn=True)
            dx.add_(dz)  # the residual branch
        return dx, None, None, None


class GroupedFeedforward(nn.Module):
    """
    ``num_experts`` independent ``ffn`` experts with stacked parameters. ``forward(x, routed)`` takes the packed rows
    of an aligned dispatch (``ops.moe.dispatch(..., align=128)``) and returns the experts' outputs in the same layout.

    Parameters are fp32 (what optimizers and averagers see); products run in bf16 with fp32 accumulation on bf16
    copies refreshed when a parameter changes. On CUDA, parameter gradients are accumulated directly into ``.grad``
    during ``backward`` (they do not flow through autograd's return values).
    """

    def __init__(self, num_experts: int, hid_dim: int, inner_dim: Optional[int] = None):
        super().__init__()
        inner_dim = inner_dim or 4 * hid_dim
        self.num_experts, self.hid_dim, self.inner_dim = num_experts, hid_dim, inner_dim
        self.w1 = nn.Parameter(torch.empty(num_experts, inner_dim, hid_dim))
        self.b1 = nn.Parameter(torch.empty(num_experts, inner_dim))
        self.w2 = nn.Parameter(torch.empty(num_experts, hid_dim, inner_dim))
        self.b2 = nn.Parameter(torch.empty(num_experts, hid_dim))
        self.gamma = nn.Parameter(torch.ones(num_experts, hid_dim))
        self.beta = nn.Parameter(torch.zeros(num_experts, hid_dim))
        for e in range(num_experts):  # the initialisation of nn.Linear, expert by expert
            for w, b in ((self.w1, self.b1), (self.w2, self.b2)):
                nn.init.kaiming_uniform_(w.data[e], a=5 ** 0.5)
                bound = 1 / w.shape[2] ** 0.5
                nn.init.uniform_(b.data[e], -bound, bound)
        self._lp = {}

    def low_precision_weights(self):
        out = []
        for name in ("w1", "w2"):
            p = getattr(self, name)
            cached = self._lp.get(name)
            if cached is None or cached[0] != p._version or cached[1] != p.data_ptr():
                cached = (p._version, p.data_ptr(), p.detach().to(torch.bfloat16))
                self._lp[name] = cached
            out.append(cached[2])
        return out

    def load_expert(self, index: int, block: nn.Module) -> None:
        """Copy the weights of a ``FeedforwardBlock`` (the single-expert ``ffn`` class) into slot ``index``."""
        with torch.no_grad():
            self.w1[index].copy_(block.ffn.weight)
            self.b1[index].copy_(block.ffn.bias)
            self.w2[index].copy_(block.ffn_output.weight)
            self.b2[index].copy_(block.ffn_output.bias)
            self.gamma[index].copy_(block.layer_norm.weight)
            self.beta[index].copy_(block.layer_norm.bias)

    def supports_kernels(self, x: torch.Tensor) -> bool:
        return (x.is_cuda and x.dtype == torch.bfloat16 and self.hid_dim % 128 == 0 and self.inner_dim % 128 == 0
                and self.hid_dim <= 1024)

    def forward(self, x: torch.Tensor, routed) -> torch.Tensor:
        assert routed.tile_group is not None, "GroupedFeedforward needs an aligned dispatch (align=128)"
        if self.supports_kernels(x):
            _lib.use_kernels(x)
            return _GroupedFFNFn.apply(x, routed.tile_group, routed.offsets, self)
        return self._forward_reference(x, routed)

    def _forward_reference(self, x: torch.Tensor, routed) -> torch.Tensor:
        bounds = routed.offsets.tolist()
        pieces = []
        for e in range(self.num_experts):
            rows = x[bounds[e]:bounds[e + 1]]
            if rows.shape[0] == 0:
                continue
            compute = rows.to(self.w1.dtype)
            hidden = F.gelu(F.linear(compute, self.w1[e], self.b1[e]), approximate="tanh")
            out = F.linear(hidden, self.w2[e], self.b2[e])
            out = F.layer_norm(compute + out, (self.hid_dim,), self.gamma[e], self.beta[e], LN_EPS)
            pieces.append(out.to(x.dtype))
        tail = x.shape[0] - bounds[self.num_experts]
        if tail > 0:
            pieces.append(torch.zeros(tail, x.shape[1], dtype=x.dtype, device=x.device))
        return torch.cat(pieces, 0) if pieces else torch.zeros_like(x)

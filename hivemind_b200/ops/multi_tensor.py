"""Multi-tensor elementwise ops and optimizer updates (one kernel launch for any number of tensors).

On CUDA tensors these call the hand-written sm_100a kernels of ``csrc/multi_tensor.cu``; on CPU tensors they run
the equivalent PyTorch code, which is also the oracle of the GPU tests.

They stand in for the per-parameter ATen loops of the reference: gradient accumulation and scaling
(hivemind/optim/grad_averager.py:130-148,204-219), AMP unscale + finite check (hivemind/optim/grad_scaler.py:59-74),
the delta rule of state averaging (hivemind/optim/state_averager.py:617-621) and the optimizer step itself
(hivemind/optim/state_averager.py:515-523).
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from hivemind_b200.ops import _lib
from hivemind_b200.utils.profiling import traced

MT_AXPY, MT_SCALE_COPY, MT_ZERO, MT_SCALE_CHECK, MT_DELTA, MT_COPY2 = range(6)
NUM_SLOTS = 6


class _OptArgs(ctypes.Structure):
    _fields_ = [
        ("lr", ctypes.c_float), ("beta1", ctypes.c_float), ("beta2", ctypes.c_float), ("eps", ctypes.c_float),
        ("weight_decay", ctypes.c_float), ("bias1", ctypes.c_float), ("bias2", ctypes.c_float),
        ("grad_scale", ctypes.c_float), ("momentum", ctypes.c_float), ("dampening", ctypes.c_float),
        ("clamp_value", ctypes.c_float), ("decoupled_wd", ctypes.c_int), ("nesterov", ctypes.c_int),
        ("first_step", ctypes.c_int), ("debias", ctypes.c_int),
    ]


@dataclass
class TensorTable:
    """Device-side description of parallel lists of tensors (up to six pointer slots per entry)."""

    slots: List[Optional[List[torch.Tensor]]]
    device: torch.device
    num_tensors: int
    num_chunks: int
    tensors_dev: Optional[torch.Tensor]
    chunks_dev: Optional[torch.Tensor]
    key: Tuple

    @property
    def on_cuda(self) -> bool:
        return self.device.type == "cuda"


_table_cache: Dict[Tuple, TensorTable] = {}
_TABLE_CACHE_LIMIT = 256


def make_table(*slots: Optional[Sequence[torch.Tensor]]) -> TensorTable:
    """Build (or fetch from cache) the table for parallel tensor lists. ``None`` leaves a slot empty."""
    slots = list(slots) + [None] * (NUM_SLOTS - len(slots))
    present = [list(s) for s in slots if s is not None]
    assert present, "at least one slot is required"
    n = len(present[0])
    assert all(len(s) == n for s in present), "all slots must list the same number of tensors"
    key = tuple(None if s is None else tuple((t.data_ptr(), t.numel(), t.dtype) for t in s) for s in slots)
    cached = _table_cache.get(key)
    if cached is not None:
        return cached
    ref = present[0]
    device = ref[0].device if n else torch.device("cpu")
    norm_slots: List[Optional[List[torch.Tensor]]] = []
    for s in slots:
        if s is None:
            norm_slots.append(None)
            continue
        s = list(s)
        for t, r in zip(s, ref):
            assert t.numel() == r.numel(), "tensors in one row must have equal numel"
            assert t.is_contiguous(), "multi-tensor ops need contiguous tensors"
            assert t.device == device
        norm_slots.append(s)
    tensors_dev = chunks_dev = None
    num_chunks = 0
    if device.type == "cuda" and n:
        lib = _lib.load_library()
        chunk = lib.hm_mt_chunk_size()
        rows, chunks = [], []
        for i in range(n):
            row = [0] * 8
            dt = 0
            for si, s in enumerate(norm_slots):
                if s is not None:
                    row[si] = s[i].data_ptr()
                    dt |= _lib.dtype_code(s[i].dtype) << (4 * si)
            row[6] = ref[i].numel()
            row[7] = dt
            rows.append(row)
            for c in range((ref[i].numel() + chunk - 1) // chunk):
                chunks.append((i, c))
        num_chunks = len(chunks)
        tensors_dev = torch.tensor(rows, dtype=torch.int64).to(device)
        chunks_dev = torch.tensor(chunks if chunks else [(0, 0)], dtype=torch.int32).to(device)
    table = TensorTable([], device, n, num_chunks, tensors_dev, chunks_dev, key)  # holds no tensor references
    if len(_table_cache) >= _TABLE_CACHE_LIMIT:
        _table_cache.pop(next(iter(_table_cache)))
    _table_cache[key] = table
    return table


def _elementwise(table: TensorTable, op: int, alpha: float, flag: Optional[torch.Tensor] = None) -> None:
    lib = _lib.load_library()
    with torch.cuda.device(table.device):
        code = lib.hm_mt_elementwise(_lib.ptr(table.tensors_dev), _lib.ptr(table.chunks_dev), table.num_chunks, op,
                                     ctypes.c_float(alpha), _lib.ptr(flag), _lib.stream_ptr(table.device))
    _lib.check(code, "hm_mt_elementwise")


@traced("grads.axpy")
def axpy_(dst: Sequence[torch.Tensor], src: Sequence[torch.Tensor], alpha: float = 1.0) -> None:
    """dst[i] += alpha * src[i] (dst fp32 accumulators, src of any float dtype)."""
    if not len(dst):
        return
    table = make_table(dst, src)
    if table.on_cuda:
        _elementwise(table, MT_AXPY, alpha)
    else:
        for d, s in zip(dst, src):
            d.add_(s.to(d.dtype), alpha=alpha)


@traced("grads.scale_copy")
def scale_copy_(dst: Sequence[torch.Tensor], src: Sequence[torch.Tensor], alpha: float = 1.0) -> None:
    """dst[i] = alpha * src[i] (dtype conversion included)."""
    if not len(dst):
        return
    table = make_table(dst, src)
    if table.on_cuda:
        _elementwise(table, MT_SCALE_COPY, alpha)
    else:
        for d, s in zip(dst, src):
            d.copy_(s.to(torch.float32) * alpha if alpha != 1.0 else s)


def zero_(dst: Sequence[torch.Tensor]) -> None:
    if not len(dst):
        return
    table = make_table(dst)
    if table.on_cuda:
        _elementwise(table, MT_ZERO, 0.0)
    else:
        for d in dst:
            d.zero_()


def copy2_(src: Sequence[torch.Tensor], dst_a: Sequence[torch.Tensor], dst_b: Optional[Sequence[torch.Tensor]] = None) -> None:
    """dst_a[i] = dst_b[i] = src[i] in one pass (e.g. fp32 master and bf16 compute copy)."""
    if not len(src):
        return
    table = make_table(dst_a, src, dst_b)
    if table.on_cuda:
        _elementwise(table, MT_COPY2, 1.0)
    else:
        for i, s in enumerate(src):
            dst_a[i].copy_(s)
            if dst_b is not None:
                dst_b[i].copy_(s)


def delta_update_(local: Sequence[torch.Tensor], new: Sequence[torch.Tensor], old: Sequence[torch.Tensor],
                  alpha: float = 1.0) -> None:
    """local[i] += alpha * (new[i] - old[i]) — the delta rule used when averaging ran in the background."""
    if not len(local):
        return
    table = make_table(local, new, old)
    if table.on_cuda:
        _elementwise(table, MT_DELTA, alpha)
    else:
        for l, n, o in zip(local, new, old):
            l.add_((n.to(torch.float32) - o.to(torch.float32)).to(l.dtype), alpha=alpha)


def unscale_and_check_(tensors: Sequence[torch.Tensor], inv_scale: float = 1.0,
                       found_inf: Optional[torch.Tensor] = None) -> torch.Tensor:
    """tensors[i] *= inv_scale; returns an int32 device scalar that is non-zero if any input was inf/nan."""
    device = tensors[0].device if len(tensors) else torch.device("cpu")
    if found_inf is None:
        found_inf = torch.zeros(1, dtype=torch.int32, device=device)
    if not len(tensors):
        return found_inf
    table = make_table(tensors)
    if table.on_cuda:
        _elementwise(table, MT_SCALE_CHECK, inv_scale, found_inf)
    else:
        for t in tensors:
            if not torch.isfinite(t).all():
                found_inf.fill_(1)
            if inv_scale != 1.0:
                t.mul_(inv_scale)
    return found_inf


def all_finite(tensors: Sequence[torch.Tensor]) -> bool:
    """Host-visible finite check over a list of tensors (one kernel + one 4-byte read)."""
    return int(unscale_and_check_(tensors, 1.0).item()) == 0


def sumsq(tensors: Sequence[torch.Tensor]) -> torch.Tensor:
    """fp32[len+1]: per-tensor sums of squares, and their total in the last entry."""
    n = len(tensors)
    device = tensors[0].device if n else torch.device("cpu")
    out = torch.zeros(n + 1, dtype=torch.float32, device=device)
    if not n:
        return out
    table = make_table(tensors)
    if table.on_cuda:
        lib = _lib.load_library()
        with torch.cuda.device(device):
            code = lib.hm_mt_sumsq(_lib.ptr(table.tensors_dev), _lib.ptr(table.chunks_dev), table.num_chunks, 0, n,
                                   _lib.ptr(out), _lib.stream_ptr(device))
        _lib.check(code, "hm_mt_sumsq")
    else:
        for i, t in enumerate(tensors):
            out[i] = t.to(torch.float32).pow(2).sum()
        out[n] = out[:n].sum()
    return out


@traced("grads.clip_norm")
def clip_grad_norm_(tensors: Sequence[torch.Tensor], max_norm: float) -> torch.Tensor:
    """Scale all tensors so that their global L2 norm is at most ``max_norm``; returns the norm before clipping."""
    n = len(tensors)
    sq = sumsq(tensors)
    if not n:
        return sq[0]
    table = make_table(tensors)
    if table.on_cuda:
        lib = _lib.load_library()
        with torch.cuda.device(table.device):
            code = lib.hm_mt_clip(_lib.ptr(table.tensors_dev), _lib.ptr(table.chunks_dev), table.num_chunks,
                                  _lib.ptr(sq), n, ctypes.c_float(max_norm), _lib.stream_ptr(table.device))
        _lib.check(code, "hm_mt_clip")
    else:
        coef = max_norm / (float(sq[n].sqrt()) + 1e-6)
        if coef < 1:
            for t in tensors:
                t.mul_(coef)
    return sq[n].sqrt()


# ------------------------------------------------------------------------------------------------------------------
def _opt_args(**kw) -> _OptArgs:
    a = _OptArgs()
    defaults = dict(lr=0.0, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, bias1=1.0, bias2=1.0, grad_scale=1.0,
                    momentum=0.0, dampening=0.0, clamp_value=1e4, decoupled_wd=0, nesterov=0, first_step=0, debias=1)
    defaults.update(kw)
    for k, v in defaults.items():
        setattr(a, k, v)
    return a


@traced("optimizer.adam")
def adam_step_(params, grads, exp_avgs, exp_avg_sqs, *, step: int, lr: float, betas=(0.9, 0.999), eps: float = 1e-8,
               weight_decay: float = 0.0, decoupled: bool = False, grad_scale: float = 1.0,
               model_copies: Optional[Sequence[torch.Tensor]] = None) -> None:
    """One Adam (``decoupled=False``) or AdamW (``decoupled=True``) step with torch.optim semantics."""
    if not len(params):
        return
    beta1, beta2 = betas
    bias1, bias2 = 1 - beta1 ** step, 1 - beta2 ** step
    table = make_table(params, grads, exp_avgs, exp_avg_sqs, model_copies)
    if table.on_cuda:
        lib = _lib.load_library()
        h = _opt_args(lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay, bias1=bias1, bias2=bias2,
                      grad_scale=grad_scale, decoupled_wd=int(decoupled))
        with torch.cuda.device(table.device):
            code = lib.hm_mt_adam(_lib.ptr(table.tensors_dev), _lib.ptr(table.chunks_dev), table.num_chunks,
                                  ctypes.byref(h), _lib.stream_ptr(table.device))
        _lib.check(code, "hm_mt_adam")
        return
    for i, p in enumerate(params):
        g = grads[i].to(torch.float32) * grad_scale
        if decoupled:
            p.mul_(1 - lr * weight_decay)
        else:
            g = g + weight_decay * p
        exp_avgs[i].mul_(beta1).add_(g, alpha=1 - beta1)
        exp_avg_sqs[i].mul_(beta2).addcmul_(g, g, value=1 - beta2)
        denom = exp_avg_sqs[i].sqrt() / math.sqrt(bias2) + eps
        p.addcdiv_(exp_avgs[i], denom, value=-lr / bias1)
        if model_copies is not None:
            model_copies[i].copy_(p)


@traced("optimizer.sgd")
def sgd_step_(params, grads, momentum_bufs=None, *, lr: float, momentum: float = 0.0, dampening: float = 0.0,
              weight_decay: float = 0.0, nesterov: bool = False, first_step: bool = False, grad_scale: float = 1.0,
              model_copies: Optional[Sequence[torch.Tensor]] = None) -> None:
    """One SGD step with torch.optim.SGD semantics."""
    if not len(params):
        return
    table = make_table(params, grads, momentum_bufs, None, model_copies)
    if table.on_cuda:
        lib = _lib.load_library()
        h = _opt_args(lr=lr, momentum=momentum if momentum_bufs is not None else 0.0, dampening=dampening,
                      weight_decay=weight_decay, nesterov=int(nesterov), first_step=int(first_step),
                      grad_scale=grad_scale)
        with torch.cuda.device(table.device):
            code = lib.hm_mt_sgd(_lib.ptr(table.tensors_dev), _lib.ptr(table.chunks_dev), table.num_chunks,
                                 ctypes.byref(h), _lib.stream_ptr(table.device))
        _lib.check(code, "hm_mt_sgd")
        return
    for i, p in enumerate(params):
        g = grads[i].to(torch.float32) * grad_scale + weight_decay * p
        if momentum and momentum_bufs is not None:
            buf = momentum_bufs[i]
            if first_step:
                buf.copy_(g)
            else:
                buf.mul_(momentum).add_(g, alpha=1 - dampening)
            g = g + momentum * buf if nesterov else buf
        p.add_(g, alpha=-lr)
        if model_copies is not None:
            model_copies[i].copy_(p)


@traced("optimizer.lamb")
def lamb_step_(params, grads, exp_avgs, exp_avg_sqs, update_scratch, *, step: int, lr: float, betas=(0.9, 0.999),
               eps: float = 1e-6, weight_decay: float = 0.0, clamp_value: float = 1e4, debias: bool = True,
               grad_scale: float = 1.0, model_copies: Optional[Sequence[torch.Tensor]] = None,
               norms_scratch: Optional[torch.Tensor] = None) -> None:
    """One LAMB step (trust ratio per tensor, weight norm clamped to ``clamp_value``, optional debiasing).

    ``update_scratch`` holds one fp32 tensor per parameter for the intermediate Adam step; ``norms_scratch`` is an
    fp32 buffer of ``2 * len(params)`` entries (allocated when not given).
    """
    if not len(params):
        return
    beta1, beta2 = betas
    bias1, bias2 = 1 - beta1 ** step, 1 - beta2 ** step
    table = make_table(params, grads, exp_avgs, exp_avg_sqs, model_copies, update_scratch)
    if table.on_cuda:
        lib = _lib.load_library()
        if norms_scratch is None:
            norms_scratch = torch.empty(2 * len(params), dtype=torch.float32, device=table.device)
        h = _opt_args(lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay, bias1=bias1, bias2=bias2,
                      grad_scale=grad_scale, clamp_value=clamp_value, debias=int(debias))
        with torch.cuda.device(table.device):
            code = lib.hm_mt_lamb(_lib.ptr(table.tensors_dev), _lib.ptr(table.chunks_dev), table.num_chunks,
                                  len(params), ctypes.byref(h), _lib.ptr(norms_scratch), _lib.stream_ptr(table.device))
        _lib.check(code, "hm_mt_lamb", kernels=2)
        return
    bc = math.sqrt(bias2) / bias1 if debias else 1.0
    for i, p in enumerate(params):
        g = grads[i].to(torch.float32) * grad_scale
        exp_avgs[i].mul_(beta1).add_(g, alpha=1 - beta1)
        exp_avg_sqs[i].mul_(beta2).addcmul_(g, g, value=1 - beta2)
        u = exp_avgs[i] / (exp_avg_sqs[i].sqrt() + eps) + weight_decay * p
        wn = float(p.norm().clamp(0, clamp_value))
        un = float(u.norm())
        trust = 1.0 if wn == 0 or un == 0 else wn / un
        p.add_(u, alpha=-lr * bc * trust)
        if model_copies is not None:
            model_copies[i].copy_(p)

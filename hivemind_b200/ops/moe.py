"""Mixture-of-experts routing ops: gate top-k, dispatch (sort rows by expert), combine (weighted mixture) + autograd.

CUDA tensors run the kernels of ``csrc/moe.cu``; CPU tensors run the PyTorch formulas in this file, which are also
the oracles of the GPU tests. The math is that of the reference's client layers: expert logit = sum of grid scores,
mixture weights = softmax over the experts that answered (hivemind/moe/client/moe.py:95-137); Switch multiplies
per-dimension softmax probabilities (hivemind/moe/client/switch_moe.py:78-145).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence, Tuple

import torch

from hivemind_b200.ops import _lib

MAX_K = 8
MODE_SOFTMAX, MODE_PROB, MODE_SUM = 0, 1, 2


def _check(code: int, what: str, kernels: int = 1) -> None:
    _lib.check(code, what, kernels)


# ---------------------------------------------------------------------------------------------------------- gate


def expert_coordinates(idx: torch.Tensor, grid_size: Sequence[int]) -> torch.Tensor:
    """Expert ids (row-major over the grid) -> coordinates ``[..., ndim]``; ids < 0 map to coordinate 0."""
    rem = idx.clamp(min=0).to(torch.int64)
    coords = []
    for size in reversed(tuple(grid_size)):
        coords.append(rem % size)
        rem = rem // size
    return torch.stack(coords[::-1], dim=-1)


def expert_values(scores: torch.Tensor, idx: torch.Tensor, grid_size: Sequence[int], mode: str = "sum") -> torch.Tensor:
    """
    Differentiable value of the chosen experts: the sum of their coordinates' scores (``mode="sum"``) or the
    product of per-dimension softmax probabilities (``mode="prob"``). Slots with ``idx < 0`` get -inf / 0.
    """
    coords = expert_coordinates(idx, grid_size)
    parts = scores.split_with_sizes(tuple(grid_size), dim=-1)
    value = None
    for d, part in enumerate(parts):
        if mode == "prob":
            part = torch.softmax(part.float(), dim=-1)
        picked = part.float().gather(1, coords[..., d])
        value = picked if value is None else (value * picked if mode == "prob" else value + picked)
    empty = torch.full_like(value, 0.0 if mode == "prob" else float("-inf"))
    return torch.where(idx >= 0, value, empty)


def gate_topk_reference(scores: torch.Tensor, grid_size: Sequence[int], k: int, alive: Optional[torch.Tensor] = None,
                        mode: str = "sum") -> Tuple[torch.Tensor, torch.Tensor]:
    grid_size = tuple(grid_size)
    parts = scores.float().split_with_sizes(grid_size, dim=-1)
    if mode == "prob":
        parts = [torch.softmax(p, dim=-1) for p in parts]
    total = None
    for d, part in enumerate(parts):
        shape = [part.shape[0]] + [1] * len(grid_size)
        shape[d + 1] = grid_size[d]
        part = part.reshape(shape)
        total = part if total is None else (total * part if mode == "prob" else total + part)
    flat = total.reshape(total.shape[0], -1).clone()
    invalid = ~(flat > 0) if mode == "prob" else flat == float("-inf")
    if alive is not None:
        invalid = invalid | ~alive.to(torch.bool).reshape(1, -1)
    flat[invalid] = float("-inf")
    kk = min(k, flat.shape[1])
    # stable order: larger value first, smaller id on ties
    order = torch.argsort(flat, dim=1, descending=True, stable=True)[:, :kk]
    val = flat.gather(1, order)
    idx = torch.where(val == float("-inf"), torch.full_like(order, -1), order).to(torch.int32)
    if mode == "prob":
        val = torch.where(idx >= 0, val, torch.zeros_like(val))
    if kk < k:
        pad = k - kk
        idx = torch.cat([idx, torch.full((idx.shape[0], pad), -1, dtype=idx.dtype, device=idx.device)], 1)
        val = torch.cat([val, torch.full((val.shape[0], pad), 0.0 if mode == "prob" else float("-inf"),
                                         device=val.device)], 1)
    return idx, val


def gate_topk(scores: torch.Tensor, grid_size: Sequence[int], k: int, alive: Optional[torch.Tensor] = None,
              mode: str = "sum") -> Tuple[torch.Tensor, torch.Tensor]:
    """
    Choose the ``k`` best live experts of every token (no gradient; see ``expert_values`` for the differentiable part).

    :param scores: ``[tokens, sum(grid_size)]`` per-dimension gate scores (``-inf`` drops a coordinate)
    :param alive: optional ``uint8/bool [prod(grid_size)]`` mask of experts that exist
    :param mode: ``"sum"`` (logits add up) or ``"prob"`` (per-dimension softmax probabilities multiply)
    :returns: ``idx int32 [tokens, k]`` (-1 = no expert) and ``val float32 [tokens, k]``
    """
    assert 1 <= k <= MAX_K and mode in ("sum", "prob")
    scores = scores.detach()
    if not _lib.use_kernels(scores):
        return gate_topk_reference(scores, grid_size, k, alive, mode)
    grid_size = tuple(int(g) for g in grid_size)
    scores = scores.float().contiguous()
    tokens = scores.shape[0]
    idx = torch.empty(tokens, k, dtype=torch.int32, device=scores.device)
    val = torch.empty(tokens, k, dtype=torch.float32, device=scores.device)
    alive_u8 = None if alive is None else alive.to(device=scores.device, dtype=torch.uint8).contiguous()
    dims = (ctypes.c_int * len(grid_size))(*grid_size)
    lib = _lib.load_library()
    with torch.cuda.device(scores.device):
        code = lib.hm_moe_gate_topk(_lib.ptr(scores), tokens, scores.stride(0), len(grid_size), dims,
                                    _lib.ptr(alive_u8), k, 1 if mode == "prob" else 0, _lib.ptr(idx), _lib.ptr(val),
                                    _lib.stream_ptr(scores.device))
    _check(code, "hm_moe_gate_topk")
    return idx, val


# ------------------------------------------------------------------------------------------------------ dispatch


TILE_ROWS = 128  # M tile of the grouped GEMM; aligned dispatch pads every expert's rows to a multiple of it


class Dispatch:
    """
    Result of ``dispatch``: rows sorted by expert. Expert ``e`` owns ``packed[offsets[e]:offsets[e+1]]``, of which
    the first ``counts[e]`` rows hold tokens (with ``align=1`` that is all of them; with ``align=128`` the rest is
    zero padding). ``tile_group[m]`` (aligned dispatch only) is the expert that owns rows ``128*m .. 128*m+127``.
    """
    __slots__ = ("packed", "pos", "counts", "offsets", "src", "num_experts", "tile_group")

    def __init__(self, packed, pos, counts, offsets, src, num_experts, tile_group=None):
        self.packed, self.pos, self.counts, self.offsets, self.src = packed, pos, counts, offsets, src
        self.num_experts, self.tile_group = num_experts, tile_group


def packed_capacity(tokens: int, k: int, num_experts: int, align: int) -> int:
    """Rows to allocate for the packed buffer (an upper bound that needs no knowledge of the routing)."""
    if align == 1:
        return tokens * k
    worst = tokens * k + num_experts * (align - 1)
    return (worst + align - 1) // align * align


def _dispatch_reference(x: torch.Tensor, idx: torch.Tensor, num_experts: int, align: int = 1):
    tokens, k = idx.shape
    device = x.device
    flat = idx.reshape(-1).to(torch.int64)
    routed = flat >= 0
    key = torch.where(routed, flat, torch.full_like(flat, num_experts))
    order = torch.argsort(key, stable=True)
    n_routed = int(routed.sum())
    src = order[:n_routed]
    counts = torch.bincount(flat[routed], minlength=num_experts).to(torch.int32)
    padded = (counts + align - 1) // align * align
    offsets = torch.zeros(num_experts + 1, dtype=torch.int32, device=device)
    offsets[1:] = torch.cumsum(padded, 0)
    dense_start = torch.zeros(num_experts, dtype=torch.int64, device=device)
    dense_start[1:] = torch.cumsum(counts, 0)[:-1]
    expert_of = flat[src]
    row = offsets[:-1].to(torch.int64)[expert_of] + (torch.arange(n_routed, device=device) - dense_start[expert_of])
    capacity = packed_capacity(tokens, k, num_experts, align)
    pos = torch.full((tokens * k,), -1, dtype=torch.int32, device=device)
    pos[src] = row.to(torch.int32)
    packed = torch.zeros(capacity, x.shape[1], dtype=x.dtype, device=device)
    packed[row] = x[src // k]
    src_full = torch.full((capacity,), -1, dtype=torch.int32, device=device)
    src_full[row] = src.to(torch.int32)
    tile_group = None
    if align > 1:
        tile_group = torch.full((capacity // TILE_ROWS,), -1, dtype=torch.int32, device=device)
        starts = torch.arange(capacity // TILE_ROWS, device=device) * TILE_ROWS
        owner = torch.searchsorted(offsets[1:].to(torch.int64), starts, right=True)
        valid = starts < int(offsets[-1])
        tile_group[valid] = owner[valid].to(torch.int32)
    return packed, pos.view(tokens, k), counts, offsets, src_full, tile_group


def _dispatch_raw(x: torch.Tensor, idx: torch.Tensor, num_experts: int, align: int = 1):
    if not _lib.use_kernels(x):
        return _dispatch_reference(x, idx, num_experts, align)
    tokens, k = idx.shape
    hidden = x.shape[1]
    assert x.stride(1) == 1 and idx.dtype == torch.int32 and idx.is_contiguous() and align in (1, TILE_ROWS)
    device = x.device
    capacity = packed_capacity(tokens, k, num_experts, align)
    max_tiles = capacity // TILE_ROWS if align > 1 else 0
    packed = torch.empty(capacity, hidden, dtype=x.dtype, device=device)
    meta = torch.empty(2 * tokens * k + capacity + 2 * num_experts + 1 + max_tiles, dtype=torch.int32, device=device)
    cursor = 0

    def take(n):
        nonlocal cursor
        part = meta[cursor:cursor + n]
        cursor += n
        return part

    pos, rank, src = take(tokens * k), take(tokens * k), take(capacity)
    counts, offsets, tile_group = take(num_experts), take(num_experts + 1), take(max_tiles)
    lib = _lib.load_library()
    with torch.cuda.device(device):
        code = lib.hm_moe_dispatch(_lib.ptr(x), ctypes.c_longlong(x.stride(0)), hidden, _lib.dtype_code(x.dtype),
                                   _lib.ptr(idx), tokens, k, num_experts, _lib.ptr(counts), _lib.ptr(offsets),
                                   _lib.ptr(rank), _lib.ptr(packed), ctypes.c_longlong(capacity), _lib.ptr(pos),
                                   _lib.ptr(src), align, _lib.ptr(tile_group if align > 1 else None), max_tiles,
                                   _lib.stream_ptr(device))
    _check(code, "hm_moe_dispatch", kernels=3)
    return packed, pos.view(tokens, k), counts, offsets, src, (tile_group if align > 1 else None)


class _DispatchFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, idx, num_experts, align):
        packed, pos, counts, offsets, src, tile_group = _dispatch_raw(x, idx, num_experts, align)
        ctx.save_for_backward(pos)
        if tile_group is None:
            tile_group = torch.empty(0, dtype=torch.int32, device=x.device)
        ctx.mark_non_differentiable(pos, counts, offsets, src, tile_group)
        return packed, pos, counts, offsets, src, tile_group

    @staticmethod
    def backward(ctx, grad_packed, *unused):
        (pos,) = ctx.saved_tensors
        grad_x = _combine_raw(grad_packed.contiguous(), pos, None, None, None, MODE_SUM)[0]
        return grad_x, None, None, None


def dispatch(x: torch.Tensor, idx: torch.Tensor, num_experts: int, align: int = 1) -> Dispatch:
    """
    Sort token rows by their chosen experts (each token appears once per routed slot).

    :param x: ``[tokens, hidden]`` (bf16 or fp32, rows 16-byte aligned)
    :param idx: ``int32 [tokens, k]`` expert ids, -1 for an empty slot
    :param align: 1 = dense rows; 128 = pad every expert to whole 128-row tiles (what ``grouped_ffn`` needs)
    :returns: a ``Dispatch``; gradient flows from ``packed`` back to ``x`` (sum over a token's slots)
    """
    packed, pos, counts, offsets, src, tile_group = _DispatchFn.apply(x, idx.contiguous(), num_experts, align)
    return Dispatch(packed, pos, counts, offsets, src, num_experts, tile_group if align > 1 else None)


# ------------------------------------------------------------------------------------------------------- combine


def _slot_weights_reference(pos, gate, keep, mode):
    on = pos >= 0
    if keep is not None:
        on = on & keep.to(torch.bool)
    if mode == MODE_SUM:
        return on.float()
    if mode == MODE_PROB:
        return torch.where(on, gate.float(), torch.zeros_like(gate, dtype=torch.float32))
    masked = torch.where(on, gate.float(), torch.full_like(gate, float("-inf"), dtype=torch.float32))
    weights = torch.softmax(masked, dim=1)
    return torch.where(on.any(1, keepdim=True), weights, torch.zeros_like(weights)).nan_to_num(0.0)


def _combine_reference(y, pos, gate, keep, residual, mode):
    w = _slot_weights_reference(pos, gate, keep, mode)
    rows = y.float()[pos.clamp(min=0).to(torch.int64)]  # [T, k, H]
    out = (w.unsqueeze(-1) * rows).sum(1)
    if residual is not None:
        out = out + residual.float()
    return out.to(y.dtype), w


def _combine_raw(y, pos, gate, keep, residual, mode):
    if not _lib.use_kernels(y):
        return _combine_reference(y, pos, gate, keep, residual, mode)
    tokens, k = pos.shape
    hidden = y.shape[1]
    out = torch.empty(tokens, hidden, dtype=y.dtype, device=y.device)
    w = torch.empty(tokens, k, dtype=torch.float32, device=y.device)
    gate32 = None if gate is None else gate.detach().float().contiguous()
    lib = _lib.load_library()
    with torch.cuda.device(y.device):
        code = lib.hm_moe_combine_fwd(_lib.ptr(y), hidden, _lib.dtype_code(y.dtype), _lib.ptr(pos), _lib.ptr(gate32),
                                      _lib.ptr(keep), _lib.ptr(residual), tokens, k, mode, _lib.ptr(out), _lib.ptr(w),
                                      _lib.stream_ptr(y.device))
    _check(code, "hm_moe_combine_fwd")
    return out, w


class _CombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, pos, gate, keep, residual, mode):
        y = y.contiguous()
        pos = pos.contiguous()
        keep = None if keep is None else keep.to(torch.uint8).contiguous()
        residual = None if residual is None else residual.to(y.dtype).contiguous()
        out, w = _combine_raw(y, pos, gate, keep, residual, mode)
        ctx.save_for_backward(y, pos, w, keep)
        ctx.mode = mode
        ctx.has_residual = residual is not None
        ctx.gate_dtype = None if gate is None else gate.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        y, pos, w, keep = ctx.saved_tensors
        mode = ctx.mode
        dout = dout.contiguous().to(y.dtype)
        tokens, k = pos.shape
        if not _lib.use_kernels(y):
            rows = y.float()[pos.clamp(min=0).to(torch.int64)]
            dots = (rows * dout.float().unsqueeze(1)).sum(-1)
            on = pos >= 0 if keep is None else (pos >= 0) & keep.to(torch.bool)
            dy = torch.zeros_like(y, dtype=torch.float32)
            sel = pos >= 0
            dy[pos[sel].to(torch.int64)] = (w.unsqueeze(-1) * dout.float().unsqueeze(1))[sel]
            if mode == MODE_SOFTMAX:
                dgate = w * (dots - (w * dots).sum(1, keepdim=True))
            else:
                dgate = dots
            dgate = torch.where(on, dgate, torch.zeros_like(dgate))
            dy = dy.to(y.dtype)
        else:
            dy = torch.zeros_like(y) if bool(ctx.needs_input_grad[0]) else torch.empty_like(y)
            dgate = torch.empty(tokens, k, dtype=torch.float32, device=y.device)
            lib = _lib.load_library()
            with torch.cuda.device(y.device):
                code = lib.hm_moe_combine_bwd(_lib.ptr(dout), _lib.ptr(y), y.shape[1], _lib.dtype_code(y.dtype),
                                              _lib.ptr(pos), _lib.ptr(w), _lib.ptr(keep), tokens, k, mode,
                                              _lib.ptr(dy), _lib.ptr(dgate), _lib.stream_ptr(y.device))
            _check(code, "hm_moe_combine_bwd")
        grad_gate = None
        if ctx.gate_dtype is not None and mode != MODE_SUM:
            grad_gate = dgate.to(ctx.gate_dtype)
        return dy, None, grad_gate, None, (dout if ctx.has_residual else None), None


def combine(y: torch.Tensor, pos: torch.Tensor, gate: Optional[torch.Tensor], mode: str = "softmax",
            keep: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """
    Mix the experts' answers: ``out[t] = residual[t] + sum_j w[t, j] * y[pos[t, j]]``.

    :param y: ``[rows, hidden]`` expert outputs in dispatch order
    :param pos: ``int32 [tokens, k]`` row of each slot in ``y`` (-1 = no expert)
    :param gate: ``[tokens, k]`` expert logits (``mode="softmax"``) or probabilities (``mode="prob"``)
    :param keep: optional ``[tokens, k]`` mask; slots with 0 are treated as experts that did not answer
    """
    mode_id = {"softmax": MODE_SOFTMAX, "prob": MODE_PROB, "sum": MODE_SUM}[mode]
    return _CombineFn.apply(y, pos, gate, keep, residual, mode_id)


def masked_softmax_combine(logits: torch.Tensor, mask: torch.Tensor, outputs: torch.Tensor) -> torch.Tensor:
    """
    ``softmax(logits over mask) @ outputs`` for ``outputs`` of shape ``[batch, k, ...]``: the mixture step of
    ``RemoteMixtureOfExperts``, fused into one kernel on CUDA. Falls back to the PyTorch formula for shapes the
    kernel does not take (k > 8, rows not a multiple of 16 bytes).
    """
    batch, k = outputs.shape[:2]
    feature_shape = outputs.shape[2:]
    hidden = int(torch.tensor(feature_shape).prod()) if len(feature_shape) else 1
    usable = (k <= MAX_K and (hidden * outputs.element_size()) % 16 == 0
              and outputs.dtype in (torch.float32, torch.bfloat16))
    if not usable:
        masked = logits.masked_fill(~mask, float("-inf"))
        weights = torch.softmax(masked, dim=1).nan_to_num(0.0)
        return (weights.view(batch, k, *([1] * len(feature_shape))) * outputs).sum(1)
    pos = torch.arange(batch * k, dtype=torch.int32, device=outputs.device).view(batch, k)
    flat = outputs.reshape(batch * k, hidden)
    out = combine(flat, pos, logits, "softmax", keep=mask)
    return out.view(batch, *feature_shape)

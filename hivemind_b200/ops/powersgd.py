"""PowerSGD device ops: batched orthogonalisation and the low-rank GEMMs on the tcgen05 kernel (tf32).

Reference math: hivemind/optim/power_sgd_averager.py:150-183 and hivemind/utils/math.py:6-14.
"""
from __future__ import annotations

import ctypes
from typing import Sequence

import numpy as np
import torch

from hivemind_b200.ops import _lib
from hivemind_b200.ops.gemm import tc_gemm

_PSMAT = np.dtype([("p", "<u8"), ("rows", "<i8"), ("gram", "<u8"), ("rinv", "<u8")])


def orthogonalize_batch_(matrices: Sequence[torch.Tensor], eps: float = 1e-8) -> None:
    """In-place thin-QR orthogonalisation of several [m_i, r] fp32 CUDA matrices with one launch per pass."""
    if not matrices:
        return
    r = matrices[0].shape[1]
    assert all(m.is_cuda and m.dtype == torch.float32 and m.dim() == 2 and m.shape[1] == r and m.is_contiguous()
               for m in matrices) and r <= 64
    device = matrices[0].device
    lib = _lib.load_library()
    rows_per_block = lib.hm_ps_rows_per_block()
    scratch = torch.zeros(len(matrices), 2, r * r, dtype=torch.float32, device=device)
    table = np.zeros(len(matrices), dtype=_PSMAT)
    items = []
    for i, m in enumerate(matrices):
        table[i] = (m.data_ptr(), m.shape[0], scratch[i, 0].data_ptr(), scratch[i, 1].data_ptr())
        items += [(i, b) for b in range((m.shape[0] + rows_per_block - 1) // rows_per_block)]
    table_dev = torch.from_numpy(table.view(np.uint8).copy()).to(device)
    items_dev = torch.tensor(items, dtype=torch.int32).to(device)
    with torch.cuda.device(device):
        for sweep in range(2):  # CholeskyQR2: the second sweep repairs the orthogonality lost to rounding in G
            if sweep:
                scratch[:, 0].zero_()
            code = lib.hm_ps_orthogonalize_sweep(_lib.ptr(table_dev), len(matrices), _lib.ptr(items_dev), len(items), r,
                                                 ctypes.c_float(eps), _lib.stream_ptr(device))
            _lib.check(code, "hm_ps_orthogonalize_sweep", kernels=3)


def orthogonalize_kernel_(matrix: torch.Tensor, eps: float = 1e-8) -> torch.Tensor:
    if not matrix.is_contiguous():
        tmp = matrix.contiguous()
        orthogonalize_batch_([tmp], eps)
        matrix.copy_(tmp)
    else:
        orthogonalize_batch_([matrix], eps)
    return matrix


def _tile_n(r: int) -> int:
    return 32 if r <= 32 else (64 if r <= 64 else 128)


def _can_use_tc(m2d: torch.Tensor, r: int) -> bool:
    rows, cols = m2d.shape
    return m2d.is_cuda and m2d.dtype == torch.float32 and r % 4 == 0 and r <= 128 and cols % 4 == 0 and m2d.is_contiguous()


def _splits(rows_out: int, contraction: int, sms: int) -> int:
    tiles = (rows_out + 127) // 128
    if tiles >= sms:
        return 1
    return max(1, min(sms // tiles, contraction // 256))


def compute_p_(p: torch.Tensor, m2d: torch.Tensor, q: torch.Tensor) -> None:
    """P[m, r] = M[m, n] @ Q[n, r]."""
    r = q.shape[1]
    if _can_use_tc(m2d, r):
        p.zero_()
        tc_gemm(m2d, q, b_mn=True, out=p, reduce_add=True, splits=_splits(m2d.shape[0], m2d.shape[1], _lib.sm_count(p.device)),
                block_n=_tile_n(r))
    else:
        torch.matmul(m2d, q, out=p)


def compute_q_(q: torch.Tensor, m2d: torch.Tensor, p: torch.Tensor) -> None:
    """Q[n, r] = M[m, n]^T @ P[m, r]."""
    r = p.shape[1]
    if _can_use_tc(m2d, r):
        q.zero_()
        tc_gemm(m2d, p, a_mn=True, b_mn=True, out=q, reduce_add=True,
                splits=_splits(m2d.shape[1], m2d.shape[0], _lib.sm_count(q.device)), block_n=_tile_n(r))
    else:
        torch.matmul(m2d.t(), p, out=q)


def reconstruct_(out2d: torch.Tensor, p: torch.Tensor, q: torch.Tensor) -> None:
    """out[m, n] = P[m, r] @ Q[n, r]^T."""
    r = p.shape[1]
    n = q.shape[0]
    if _can_use_tc(out2d, r) and n >= 32:
        tc_gemm(p, q, out=out2d, block_n=128 if n >= 128 else (64 if n >= 64 else 32))
    else:
        torch.matmul(p, q.t(), out=out2d)


# ---------------------------------------------------------------------------------------------------------------
# the same three products for a STACK of matrices of one shape, one launch each (grouped modes of the tcgen05 kernel)
_group_tables = {}


def _group_table(device: torch.device, groups: int, step: int, per_tile: bool) -> torch.Tensor:
    """Mode 1 (``per_tile``): the group of every 128-row tile of the stacked A / D; mode 2: row offsets of the groups
    along the shared contraction axis. Cached: the tables depend only on the shapes."""
    key = (device.index, groups, step, per_tile)
    table = _group_tables.get(key)
    if table is None:
        if per_tile:
            values = torch.arange(groups, dtype=torch.int32).repeat_interleave(step // 128)
        else:
            values = torch.arange(groups + 1, dtype=torch.int32) * step
        table = _group_tables[key] = values.to(device)
    return table


def can_stack(rows: int, cols: int, r: int) -> bool:
    """Whether matrices of this shape can go through the grouped launches (whole 128-row tiles in both directions)."""
    return rows % 128 == 0 and cols % 128 == 0 and r % 4 == 0 and r <= 128


def _grouped(a, b, d, m, n, k, a_mn, b_mn, mode, groups, table, reduce_add=False, alpha=1.0, block_n=None) -> None:
    from hivemind_b200.ops.gemm import _err_flag

    lib = _lib.load_library()
    dev = a.device
    with torch.cuda.device(dev):
        code = lib.hm_tc_gemm_grouped_tf32(
            _lib.ptr(a), _lib.ptr(b), _lib.ptr(d), m, n, k, ctypes.c_longlong(a.stride(0)), ctypes.c_longlong(b.stride(0)),
            ctypes.c_longlong(d.stride(0)), int(a_mn), int(b_mn), int(reduce_add), ctypes.c_float(alpha),
            block_n or _tile_n(n), _lib.ptr(_err_flag(dev)), _lib.sm_count(dev), mode, groups, _lib.ptr(table),
            _lib.stream_ptr(dev))
    _lib.check(code, "hm_tc_gemm_grouped_tf32")


def compute_p_stacked_(p: torch.Tensor, m: torch.Tensor, q: torch.Tensor) -> None:
    """``p[g] = m[g] @ q[g]`` for stacked ``m [G, rows, cols]``, ``q [G, cols, r]``, ``p [G, rows, r]`` (fp32, CUDA)."""
    groups, rows, cols = m.shape
    r = q.shape[2]
    _grouped(m.view(groups * rows, cols), q.view(groups * cols, r), p.view(groups * rows, r), groups * rows, r, cols,
             False, True, 1, groups, _group_table(m.device, groups, rows, True))


def compute_q_stacked_(q: torch.Tensor, m: torch.Tensor, p: torch.Tensor) -> None:
    """``q[g] = m[g].T @ p[g]`` for the same stacks: the contraction runs over each group's own rows."""
    groups, rows, cols = m.shape
    r = p.shape[2]
    _grouped(m.view(groups * rows, cols), p.view(groups * rows, r), q.view(groups * cols, r), cols, r, groups * rows,
             True, True, 2, groups, _group_table(m.device, groups, rows, False))


def reconstruct_stacked_(out: torch.Tensor, p: torch.Tensor, q: torch.Tensor) -> None:
    """``out[g] = p[g] @ q[g].T`` for ``out [G, rows, cols]``."""
    groups, rows, cols = out.shape
    r = p.shape[2]
    _grouped(p.view(groups * rows, r), q.view(groups * cols, r), out.view(groups * rows, cols), groups * rows, cols, r,
             False, False, 1, groups, _group_table(out.device, groups, rows, True), block_n=128)


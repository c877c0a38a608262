"""PowerSGD device ops: batched orthogonalisation and the low-rank GEMMs on the tcgen05 kernel (tf32).

Reference math: hivemind/optim/power_sgd_averager.py:150-183 and hivemind/utils/math.py:6-14.
"""
from __future__ import annotations

import ctypes
from typing import List, Sequence

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

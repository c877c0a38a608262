"""Small tensor helpers of the PowerSGD path (reference: hivemind/utils/math.py:6-24)."""
from __future__ import annotations

import torch


def orthogonalize_(matrix: torch.Tensor, eps: float = 1e-8) -> torch.Tensor:
    """Modified Gram–Schmidt over the columns of ``matrix`` ([m, r]), in place.

    CUDA fp32 matrices run the hand-written kernel of ``ops/csrc/powersgd.cu``; anything else runs the loop below,
    which is also the oracle of that kernel's test.
    """
    if matrix.is_cuda and matrix.dtype == torch.float32 and matrix.dim() == 2 and matrix.shape[1] <= 64:
        from hivemind_b200.ops.powersgd import orthogonalize_kernel_

        return orthogonalize_kernel_(matrix, eps)
    return orthogonalize_reference_(matrix, eps)


def orthogonalize_reference_(matrix: torch.Tensor, eps: float = 1e-8) -> torch.Tensor:
    n_cols = matrix.shape[1]
    for i in range(n_cols):
        col = matrix[:, i]
        col /= torch.linalg.norm(col) + eps
        if i + 1 < n_cols:
            rest = matrix[:, i + 1:]
            rest.addmm_(col[:, None], (col @ rest)[None, :], alpha=-1)
    return matrix


def get_flatten_greedy_dims(tensor: torch.Tensor, max_ndim: int = 2):
    """Merge the two smallest adjacent dimensions until at most ``max_ndim`` remain; returns the new shape."""
    dims = list(tensor.shape)
    while len(dims) > max_ndim:
        sizes = [dims[i] * dims[i + 1] for i in range(len(dims) - 1)]
        i = min(range(len(sizes)), key=sizes.__getitem__)
        dims[i:i + 2] = [sizes[i]]
    return dims

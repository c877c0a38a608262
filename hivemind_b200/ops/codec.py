"""Tensor codecs on the GPU: fp16, mean/std-scaled fp16, uniform / quantile / block-wise 8-bit.

These are the whole-tensor encode kernels of ``csrc/codec.cu`` driven as a one-rank "group" whose
outbox is a scratch buffer: the tensor (or each of its last-axis rows, for the scaled codec) is one part. They serve
the compression classes when those are handed CUDA tensors (state downloads, expert RPC payloads), so that only
compressed bytes cross PCIe. Math: hivemind/compression/floating.py:18-64, quantization.py:60-93,130-153.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Dict, List, Tuple

import numpy as np
import torch

from hivemind_b200.ops import _lib

_HALF_MIN, _HALF_MAX = -65504.0, 65504.0
_MAX_PEERS = 16
PH_STATS, PH_BORDERS, PH_ENCODE, PH_PUBLISH = range(4)


class _HbPeer(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("outbox", ctypes.c_void_p), ("deltabox", ctypes.c_void_p),
                ("ready", ctypes.c_void_p), ("delta_ready", ctypes.c_void_p), ("avg", ctypes.c_void_p)]


class _HbGroup(ctypes.Structure):
    """Mirror of ``HbGroup`` in ``csrc/codec.cu`` (a one-rank group whose outbox is the output buffer)."""

    _fields_ = [("n_peers", ctypes.c_int), ("n_parts", ctypes.c_int), ("me", ctypes.c_int),
                ("max_local_parts", ctypes.c_int), ("epoch", ctypes.c_uint), ("alpha", ctypes.c_float),
                ("sender_timeout_ns", ctypes.c_ulonglong), ("reducer_timeout_ns", ctypes.c_ulonglong),
                ("delta_stride", ctypes.c_ulonglong), ("weight", ctypes.c_float * _MAX_PEERS),
                ("sends", ctypes.c_int * _MAX_PEERS), ("peer", _HbPeer * _MAX_PEERS), ("parts", ctypes.c_void_p),
                ("part_stats", ctypes.c_void_p), ("dstats", ctypes.c_void_p), ("bins", ctypes.c_void_p),
                ("bin_cnt", ctypes.c_void_p), ("dbins", ctypes.c_void_p), ("dbin_cnt", ctypes.c_void_p),
                ("borders", ctypes.c_void_p), ("dborders", ctypes.c_void_p), ("include", ctypes.c_void_p),
                ("apply_decision", ctypes.c_void_p), ("ban", ctypes.c_void_p), ("t_start", ctypes.c_void_p),
                ("status", ctypes.c_void_p), ("avg", ctypes.c_void_p)]


_PART_DTYPE = np.dtype([("start", "<i8"), ("enc_off", "<i8"), ("span_off", "<i8"), ("avg_off", "<i8"), ("len", "<i4"),
                        ("owner", "<i4"), ("local_idx", "<i4"), ("codec", "<i4")])
_code_uploaded: Dict[int, bool] = {}
_code_lock = threading.Lock()


def _ensure_code_table(device_index: int) -> None:
    """Upload the block-wise code table into the library's constant memory of this device (once)."""
    from hivemind_b200.compression.quantization import dynamic_code_table

    with _code_lock:
        if _code_uploaded.get(device_index):
            return
        lib = _lib.load_library()
        assert lib.hm_bf_sizeof_group() == ctypes.sizeof(_HbGroup), "HbGroup layout mismatch between C and Python"
        assert lib.hm_bf_sizeof_part() == _PART_DTYPE.itemsize, "HbPart layout mismatch between C and Python"
        code = dynamic_code_table().numpy().astype(np.float32)
        with torch.cuda.device(device_index):
            _lib.check(lib.hm_bf_set_blockwise_code(code.ctypes.data_as(ctypes.c_void_p)), "hm_bf_set_blockwise_code", 0)
        _code_uploaded[device_index] = True


def record_bytes(codec: int, length: int) -> int:
    """Bytes of a whole-tensor record: header (statistics or codebook) + payload rounded up to 16 bytes."""
    header = {1: 16, 3: 1024, 4: 1024}.get(codec, 0)
    if codec == 5:
        header = ((length + 4095) // 4096 * 4 + 15) // 16 * 16
    elem = 4 if codec == 0 else (2 if codec in (1, 2) else 1)
    return header + (length * elem + 15) // 16 * 16


def _run_encode(flat: torch.Tensor, parts: List[Tuple[int, int]], codec: int) -> Tuple[torch.Tensor, List[int]]:
    """Encode ``flat[start:start+len]`` for every (start, len) into one byte buffer; returns it and record offsets."""
    device = flat.device
    lib = _lib.load_library()
    _ensure_code_table(device.index)
    chunk = lib.hm_bf_chunk()
    n_parts = len(parts)
    table = np.zeros(n_parts, dtype=_PART_DTYPE)
    offsets, cursor = [], 0
    for p, (start, length) in enumerate(parts):
        table[p] = (start, cursor, 0, start, length, 1, p, codec)  # owner 1 != me 0: "a part that I send"
        offsets.append(cursor)
        cursor += record_bytes(codec, length)
    outbox = torch.empty(max(cursor, 16), dtype=torch.uint8, device=device)
    parts_dev = torch.from_numpy(table.view(np.uint8).copy()).to(device)
    items = [(p, c, 0, 0) for p, (_, length) in enumerate(parts) for c in range((length + chunk - 1) // chunk)]
    per_part = [(p, 0, 0, 0) for p in range(n_parts)]
    items_dev = torch.tensor(items or [(0, 0, 0, 0)], dtype=torch.int32).to(device)
    per_part_dev = torch.tensor(per_part or [(0, 0, 0, 0)], dtype=torch.int32).to(device)
    scratch = torch.zeros(n_parts * (16 + 1024 * 3) + 64, dtype=torch.uint8, device=device)
    ready = torch.zeros(max(n_parts, 1), dtype=torch.int32, device=device)
    g = _HbGroup()
    g.n_peers, g.n_parts, g.me, g.max_local_parts, g.epoch, g.alpha = 2, n_parts, 0, 1, 1, 1.0
    g.sends[0] = 1
    g.peer[0].data = flat.data_ptr()
    g.peer[0].outbox = outbox.data_ptr()
    g.peer[0].ready = ready.data_ptr()
    g.parts = parts_dev.data_ptr()
    base = scratch.data_ptr()
    g.part_stats = base
    g.bins = base + n_parts * 16
    g.bin_cnt = g.bins + n_parts * 1024
    g.borders = g.bin_cnt + n_parts * 1024
    group_dev = torch.from_numpy(np.frombuffer(bytes(g), dtype=np.uint8).copy()).to(device)
    stream = _lib.stream_ptr(device)
    launches = []
    if codec in (1, 4):
        launches.append((PH_STATS, items_dev, len(items)))
    if codec == 3:
        launches.append((PH_BORDERS, per_part_dev, n_parts))
    launches += [(PH_ENCODE, items_dev, len(items)), (PH_PUBLISH, per_part_dev, n_parts)]
    with torch.cuda.device(device):
        for phase, it, count in launches:
            if count:
                _lib.check(lib.hm_bf_launch(phase, _lib.ptr(group_dev), _lib.ptr(it), count, 0, stream), "hm_bf_launch")
    return outbox, offsets


def _as_flat_f32(tensor: torch.Tensor) -> torch.Tensor:
    flat = tensor.detach().reshape(-1)
    if flat.dtype != torch.float32 or not flat.is_contiguous() or flat.data_ptr() % 16:
        flat = flat.to(torch.float32).contiguous().clone() if flat.data_ptr() % 16 else flat.to(torch.float32).contiguous()
    return flat


def encode_float16(tensor: torch.Tensor) -> torch.Tensor:
    flat = _as_flat_f32(tensor)
    if flat.numel() == 0:
        return torch.empty(tensor.shape, dtype=torch.float16, device=tensor.device)
    buf, _ = _run_encode(flat, [(0, flat.numel())], 2)
    return buf[:flat.numel() * 2].view(torch.float16).view(tensor.shape)


def encode_scaled_float16(tensor: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns (fp16 values, fp32 means, fp32 stds); statistics are per last-axis row, kept with ``keepdim``."""
    row = tensor.shape[-1] if tensor.dim() else 1
    rows = tensor.numel() // max(row, 1)
    stats_shape = (*tensor.shape[:-1], 1) if tensor.dim() else ()
    if row % 4 != 0 or rows > 65536:
        # rows that do not start on a 16-byte boundary (or very many tiny rows): the plain formula on the device
        work = tensor.detach().to(torch.float32)
        means = work.mean(dim=-1, keepdim=True)
        work = work - means
        stds = (work.norm(dim=-1, keepdim=True) / (row ** 0.5)).clamp_min(torch.finfo(torch.float32).eps)
        return (work / stds).clamp_(_HALF_MIN, _HALF_MAX).to(torch.float16), means, stds
    flat = _as_flat_f32(tensor)
    buf, offsets = _run_encode(flat, [(r * row, row) for r in range(rows)], 1)
    rec = 16 + (row * 2 + 15) // 16 * 16
    records = buf[:rows * rec].view(rows, rec)
    half = records[:, 16:16 + row * 2].contiguous().view(torch.float16).view(tensor.shape)
    header = records[:, :8].contiguous().view(torch.float32)
    return half, header[:, 0].reshape(stats_shape).clone(), header[:, 1].reshape(stats_shape).clone()


def _encode_codebook(tensor: torch.Tensor, codec: int) -> Tuple[torch.Tensor, torch.Tensor]:
    flat = _as_flat_f32(tensor)
    buf, _ = _run_encode(flat, [(0, flat.numel())], codec)
    codebook = buf[:1024].view(torch.float32).clone()
    indices = buf[1024:1024 + flat.numel()].view(tensor.shape)
    return indices, codebook


def encode_uniform8(tensor: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    return _encode_codebook(tensor, 4)


def encode_quantile8(tensor: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    return _encode_codebook(tensor, 3)


def encode_blockwise8(tensor: torch.Tensor, code: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns (uint8 indices, fp32 absmax per 4096 values). ``code`` must be the library's dynamic code table."""
    flat = _as_flat_f32(tensor)
    n = flat.numel()
    buf, _ = _run_encode(flat, [(0, n)], 5)
    n_blocks = (n + 4095) // 4096
    header = (n_blocks * 4 + 15) // 16 * 16
    return buf[header:header + n].view(tensor.shape), buf[:n_blocks * 4].view(torch.float32).clone()

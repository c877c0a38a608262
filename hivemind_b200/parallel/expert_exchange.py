"""``PeerExpertExchange``: mixture-of-experts dispatch / combine between the GPUs of one box over peer-mapped memory.

Each rank owns one arena (``cudaMalloc`` + CUDA IPC handle) with its client buffers (token rows sorted by global
expert, their per-expert offsets), its server buffers (expert outputs in the gathered layout, the layout table) and
four flag words. Ranks write only their own arena and pull from their peers' arenas with the kernels of
``ops/csrc/moe_exchange.cu``; flags carry the step number, every wait is bounded, and a peer that does not show up
in time is treated like an expert that did not answer (``ok`` rows are 0, the combine step masks them), which is
the failure semantics of ``RemoteMixtureOfExperts`` (hivemind/moe/client/moe.py:255-300) carried over to the device.

The exchange is written as four stages (client publish, server gather, server publish, client pull) so that a test
on a single GPU can run several ranks stage by stage; in normal operation ``exchange_and_run`` chains them.
"""
from __future__ import annotations

import ctypes
import os
from typing import Callable, List, Optional, Sequence, Tuple

import torch

from hivemind_b200.ops import _lib
from hivemind_b200.ops import moe as moe_ops

MAX_RANKS = 16
FORWARD, BACKWARD = 0, 1


class _MxPeers(ctypes.Structure):
    _fields_ = [("n_ranks", ctypes.c_int), ("me", ctypes.c_int), ("experts_per_rank", ctypes.c_int),
                ("hidden_bytes", ctypes.c_int), ("timeout_ns", ctypes.c_ulonglong),
                ("rows", ctypes.c_void_p * MAX_RANKS), ("offsets", ctypes.c_void_p * MAX_RANKS),
                ("answers", ctypes.c_void_p * MAX_RANKS), ("base_table", ctypes.c_void_p * MAX_RANKS),
                ("rows_flag", ctypes.c_void_p * MAX_RANKS), ("answers_flag", ctypes.c_void_p * MAX_RANKS),
                ("capacity", ctypes.c_int)]


class _RawCuda:
    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}
        self._owner = owner


class GatheredRows:
    """What the server side of a step hands to the experts (the fields ``GroupedFeedforward`` reads)."""

    def __init__(self, packed, tile_group, offsets, base_table, src_start, seg_count, status):
        self.packed, self.tile_group, self.offsets = packed, tile_group, offsets
        self.base_table, self.src_start, self.seg_count, self.status = base_table, src_start, seg_count, status


class PeerExpertExchange:
    """
    :param rank / world: this rank and the number of ranks sharing the experts
    :param experts_per_rank: experts hosted by every rank (global expert ``e`` lives on rank ``e // experts_per_rank``)
    :param hidden: row width in elements; :param dtype: row dtype (rows must be a multiple of 16 bytes)
    :param max_rows: most (token, slot) rows this rank will ever send in one step (tokens * k_best)
    :param exchange_descriptors: ``f(my_descriptor) -> [descriptor of rank 0, 1, ...]`` (e.g. an all_gather_object);
      if omitted, call ``connect(descriptors)`` before the first step
    :param timeout: seconds to wait for a peer's flag before treating it as absent
    """

    def __init__(self, *, rank: int, world: int, experts_per_rank: int, hidden: int, max_rows: int,
                 device: torch.device, exchange_descriptors: Optional[Callable[[dict], List[dict]]] = None,
                 dtype: torch.dtype = torch.bfloat16, timeout: float = 10.0):
        assert 1 <= world <= MAX_RANKS
        self.rank, self.world, self.experts_per_rank = rank, world, experts_per_rank
        self.num_experts = world * experts_per_rank
        self.hidden, self.dtype, self.device = hidden, dtype, torch.device(device)
        self.row_bytes = hidden * torch.empty(0, dtype=dtype).element_size()
        assert self.row_bytes % 16 == 0
        self.max_rows = max_rows
        worst = world * max_rows + experts_per_rank * (moe_ops.TILE_ROWS - 1)
        self.capacity = (worst + moe_ops.TILE_ROWS - 1) // moe_ops.TILE_ROWS * moe_ops.TILE_ROWS
        self.max_tiles = self.capacity // moe_ops.TILE_ROWS
        self.timeout_ns = int(timeout * 1e9)
        self.lib = _lib.load_library()
        self.layout, cursor = {}, 0
        for name, nbytes in (("fwd_rows", max_rows * self.row_bytes), ("bwd_rows", max_rows * self.row_bytes),
                             ("offsets", (self.num_experts + 1) * 4), ("fwd_answers", self.capacity * self.row_bytes),
                             ("bwd_answers", self.capacity * self.row_bytes),
                             ("base_table", 2 * experts_per_rank * world * 4), ("flags", 256)):
            self.layout[name] = cursor
            cursor += (nbytes + 255) // 256 * 256
        self.arena_bytes = cursor
        base = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(self.lib.hm_arena_alloc(ctypes.byref(base), ctypes.c_ulonglong(self.arena_bytes)), "hm_arena_alloc", 0)
            handle = (ctypes.c_ubyte * 64)()
            rc = self.lib.hm_ipc_export(base, handle)
        self.base = base.value
        self._bytes = torch.as_tensor(_RawCuda(self.base, self.arena_bytes, self), device=self.device)
        self.descriptor = dict(rank=rank, pid=os.getpid(), dev=self.device.index, ptr=self.base, layout=self.layout,
                               handle=bytes(handle) if rc == 0 else None, arena_bytes=self.arena_bytes)
        self.peer_base: List[int] = []
        self._opened: List[int] = []
        self.epoch = 0
        self.sms = _lib.sm_count(self.device)
        if exchange_descriptors is not None:
            self.connect(exchange_descriptors(self.descriptor))

    def connect(self, descriptors: Sequence[dict]) -> None:
        """Map the arenas of all ranks (``descriptors[r]`` is rank r's ``descriptor``)."""
        rank, world = self.rank, self.world
        self.descriptors = list(descriptors)
        assert len(self.descriptors) == world and all(d["layout"] == self.layout for d in self.descriptors), \
            "all ranks must build the exchange with the same sizes"
        for d in self.descriptors:
            if d["rank"] == rank:
                self.peer_base.append(self.base)
            elif d["pid"] == os.getpid():
                if d["dev"] != self.device.index:
                    rc = self.lib.hm_enable_peer_access(self.device.index, d["dev"])
                    if rc != 0:
                        raise RuntimeError(f"GPU {self.device.index} cannot access GPU {d['dev']} (code {rc})")
                self.peer_base.append(d["ptr"])
            else:
                out = ctypes.c_void_p()
                buf = (ctypes.c_ubyte * 64).from_buffer_copy(d["handle"])
                with torch.cuda.device(self.device):
                    _lib.check(self.lib.hm_ipc_open(buf, ctypes.byref(out)), "hm_ipc_open", 0)
                self.peer_base.append(out.value)
                self._opened.append(out.value)

    # ------------------------------------------------------------------------------------------------ plumbing
    def _view(self, name: str, nbytes: int) -> torch.Tensor:
        return self._bytes[self.layout[name]:self.layout[name] + nbytes]

    def _rows_view(self, name: str, rows: int) -> torch.Tensor:
        return self._view(name, rows * self.row_bytes).view(self.dtype).view(rows, self.hidden)

    def _flag_ptr(self, base: int, index: int) -> int:
        return base + self.layout["flags"] + 64 * index  # rows fwd, answers fwd, rows bwd, answers bwd

    def _peers(self, phase: int) -> _MxPeers:
        p = _MxPeers()
        p.n_ranks, p.me, p.experts_per_rank, p.hidden_bytes = self.world, self.rank, self.experts_per_rank, self.row_bytes
        p.timeout_ns, p.capacity = self.timeout_ns, self.capacity
        rows_name, answers_name = ("fwd_rows", "fwd_answers") if phase == FORWARD else ("bwd_rows", "bwd_answers")
        for r, base in enumerate(self.peer_base):
            p.rows[r] = base + self.layout[rows_name]
            p.offsets[r] = base + self.layout["offsets"]
            p.answers[r] = base + self.layout[answers_name]
            p.base_table[r] = base + self.layout["base_table"]
            p.rows_flag[r] = self._flag_ptr(base, 2 * phase)
            p.answers_flag[r] = self._flag_ptr(base, 2 * phase + 1)
        return p

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    # -------------------------------------------------------------------------------------------------- stages
    def client_publish(self, rows: torch.Tensor, offsets: Optional[torch.Tensor], phase: int, epoch: int) -> None:
        """Stage 1: put my rows (sorted by global expert) and, in the forward phase, their offsets into my arena."""
        n = rows.shape[0]
        assert n <= self.max_rows and rows.dtype == self.dtype and rows.shape[1] == self.hidden
        self._rows_view("fwd_rows" if phase == FORWARD else "bwd_rows", n).copy_(rows)
        if offsets is not None:
            self._view("offsets", (self.num_experts + 1) * 4).view(torch.int32).copy_(offsets)
        with torch.cuda.device(self.device):
            code = self.lib.hm_mx_publish(ctypes.c_void_p(self._flag_ptr(self.base, 2 * phase)), epoch,
                                          _lib.stream_ptr(self.device))
        _lib.check(code, "hm_mx_publish")

    def server_gather(self, phase: int, epoch: int) -> GatheredRows:
        """Stage 2: wait for the clients, lay their rows out by (expert, client) and pull them over NVLink."""
        el, r = self.experts_per_rank, self.world
        meta = torch.zeros(el * r + el + 1 + self.max_tiles, dtype=torch.int32, device=self.device)
        src_start = meta[:el * r]
        offs_pad = meta[el * r:el * r + el + 1]
        tile_group = meta[el * r + el + 1:]
        status = torch.zeros(1, dtype=torch.int64, device=self.device)  # own allocation: 8-byte aligned for atomics
        # first rows and lengths of the (expert, client) segments live in the arena: the clients read both
        tables = self._view("base_table", 2 * el * r * 4).view(torch.int32)
        base_table, seg_count = tables[:el * r], tables[el * r:]
        gathered = torch.zeros(self.capacity, self.hidden, dtype=self.dtype, device=self.device)
        peers = self._peers(phase)
        with torch.cuda.device(self.device):
            code = self.lib.hm_mx_layout(ctypes.byref(peers), epoch, _lib.ptr(base_table), _lib.ptr(src_start),
                                         _lib.ptr(seg_count), _lib.ptr(offs_pad), _lib.ptr(tile_group), self.max_tiles,
                                         _lib.ptr(status), _lib.stream_ptr(self.device))
            _lib.check(code, "hm_mx_layout")
            code = self.lib.hm_mx_gather(ctypes.byref(peers), _lib.ptr(base_table), _lib.ptr(src_start),
                                         _lib.ptr(seg_count), _lib.ptr(gathered), self.capacity, 4 * self.sms,
                                         _lib.stream_ptr(self.device))
            _lib.check(code, "hm_mx_gather")
        return GatheredRows(gathered, tile_group, offs_pad, base_table, src_start, seg_count, status)

    def server_publish(self, answers: torch.Tensor, phase: int, epoch: int) -> None:
        """Stage 3: expose my experts' outputs (gathered layout) and raise the flag."""
        assert answers.shape == (self.capacity, self.hidden)
        self._rows_view("fwd_answers" if phase == FORWARD else "bwd_answers", self.capacity).copy_(answers)
        with torch.cuda.device(self.device):
            code = self.lib.hm_mx_publish(ctypes.c_void_p(self._flag_ptr(self.base, 2 * phase + 1)), epoch,
                                          _lib.stream_ptr(self.device))
        _lib.check(code, "hm_mx_publish")

    def client_pull(self, my_offsets: torch.Tensor, rows: int, phase: int, epoch: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Stage 4: pull the answers of my ``rows`` rows; returns them with a per-row ok mask (0 = server absent)."""
        out = torch.empty(rows, self.hidden, dtype=self.dtype, device=self.device)
        ok = torch.zeros(rows, dtype=torch.uint8, device=self.device)
        server_state = torch.zeros(self.world, dtype=torch.int32, device=self.device)
        words = torch.zeros(2, dtype=torch.int64, device=self.device)  # [phase start time, status]; 8-byte aligned
        peers = self._peers(phase)
        with torch.cuda.device(self.device):
            code = self.lib.hm_mx_pull(ctypes.byref(peers), epoch, _lib.ptr(my_offsets), self.num_experts,
                                       _lib.ptr(out), _lib.ptr(ok), _lib.ptr(server_state), _lib.ptr(words[0:1]),
                                       _lib.ptr(words[1:2]), 4 * self.sms, _lib.stream_ptr(self.device))
        _lib.check(code, "hm_mx_pull")
        return out, ok

    def close(self) -> None:
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            for ptr in self._opened:
                self.lib.hm_ipc_close(ctypes.c_void_p(ptr))
        self._opened = []
        # the arena itself stays allocated until process exit: peers may still hold mappings of it


class PeerExchangeExperts(torch.autograd.Function):
    """Dispatch rows to the ranks that host their experts, run the experts, bring the answers back (and the reverse
    for gradients). ``packed`` / ``offsets`` come from ``ops.moe.dispatch(..., align=1)`` over the GLOBAL experts."""

    @staticmethod
    def forward(ctx, packed: torch.Tensor, offsets: torch.Tensor, exchange: PeerExpertExchange, run_experts):
        epoch = exchange.next_epoch()
        rows = packed.shape[0]
        exchange.client_publish(packed.detach(), offsets, FORWARD, epoch)
        gathered = exchange.server_gather(FORWARD, epoch)
        with torch.enable_grad():
            gathered.packed.requires_grad_(True)
            answers = run_experts(gathered.packed, gathered)
        exchange.server_publish(answers.detach(), FORWARD, epoch)
        out, ok = exchange.client_pull(offsets, rows, FORWARD, epoch)
        ctx.exchange, ctx.epoch, ctx.rows = exchange, epoch, rows
        ctx.graph = (gathered.packed, answers)
        ctx.save_for_backward(offsets)
        ctx.mark_non_differentiable(ok)
        return out, ok

    @staticmethod
    def backward(ctx, grad_out: torch.Tensor, _grad_ok):
        exchange, epoch = ctx.exchange, ctx.epoch
        (offsets,) = ctx.saved_tensors
        gathered_in, answers = ctx.graph
        exchange.client_publish(grad_out.contiguous().to(exchange.dtype), None, BACKWARD, epoch)
        grads = exchange.server_gather(BACKWARD, epoch)
        torch.autograd.backward(answers, grads.packed)
        grad_rows = gathered_in.grad if gathered_in.grad is not None else torch.zeros_like(gathered_in)
        exchange.server_publish(grad_rows, BACKWARD, epoch)
        grad_packed, _ = exchange.client_pull(offsets, ctx.rows, BACKWARD, epoch)
        ctx.graph = None
        return grad_packed, None, None, None

"""Host side of the device butterfly: arenas, handle exchange, part tables and kernel launches.

One ``DeviceEndpoint`` belongs to one averager (one GPU). It owns a single device allocation ("arena") that holds
the averaged tensors as one flat fp32 vector plus the staging areas that other GPUs read: the outbox with encoded
parts, the delta box with encoded averages-minus-input, and the flag pages. At group assembly every member's
``describe()`` blob travels in the matchmaking ``gather`` field; members map each other's arenas (CUDA IPC across
processes, peer access inside one process) and then each runs ``run_round``: a fixed sequence of kernel launches
(``ops/csrc/butterfly.cu``) on a private stream, with no host synchronisation until the end.

Division of labour with the reference: ``TensorPartContainer`` / ``TensorPartReducer`` / ``AllReduceRunner``
(hivemind/averaging/partition.py, allreduce.py) become a part table in device memory, bounded flag waits and
per-part inclusion decisions; load balancing, modes, weights and timeouts keep their meaning.
"""
from __future__ import annotations

import ctypes
import os
import time
import socket
import threading
import zlib
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from hivemind_b200.utils.profiling import device_range

from hivemind_b200.averaging.allreduce import AveragingMode
from hivemind_b200.averaging.partition import compute_part_layout
from hivemind_b200.compression import (BlockwiseQuantization, CompressionBase, CompressionInfo, Float16Compression,
                                       NoCompression, Quantile8BitQuantization, ScaledFloat16Compression,
                                       Uniform8BitQuantization)
from hivemind_b200.compression.adaptive import AdaptiveCompressionBase
from hivemind_b200.compression.quantization import dynamic_code_table
from hivemind_b200.ops import _lib
from hivemind_b200.utils.logging import get_logger

logger = get_logger(__name__)

GUARD_BYTES, GUARD_PATTERN = 256, 0xA5  # canary zones between the regions of an arena
DEBUG_CHECKS = os.environ.get("HIVEMIND_B200_DEBUG", "0") == "1"
EXIT_GRACE_SECONDS = 2.0  # how long after a round peers may still read this arena (see DeviceEndpoint.close)
MAX_PEERS = 16
ALIGN = 16  # elements: tensor starts and part boundaries are multiples of this, so every access is 16-byte aligned
PH_STATS, PH_BORDERS, PH_ENCODE, PH_PUBLISH, PH_REDUCE, PH_APPLY = range(6)
_CODEC_IDS = {NoCompression: 0, ScaledFloat16Compression: 1, Float16Compression: 2, Quantile8BitQuantization: 3,
              Uniform8BitQuantization: 4, BlockwiseQuantization: 5}
_NEEDS_STATS, _NEEDS_BORDERS = (1, 4), (3,)
CODEC_NONE = 0  # uncompressed parts take the in-place path (no outbox record, no delta record)


def codec_id(compression: CompressionBase, info: CompressionInfo) -> Optional[int]:
    """Device codec id for a tensor, or None if the codec has no device implementation."""
    while isinstance(compression, AdaptiveCompressionBase):
        compression = compression.choose_compression(info)
    return _CODEC_IDS.get(type(compression))


class _HbPeer(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("outbox", ctypes.c_void_p), ("deltabox", ctypes.c_void_p),
                ("ready", ctypes.c_void_p), ("delta_ready", ctypes.c_void_p), ("avg", ctypes.c_void_p)]


class _HbGroup(ctypes.Structure):
    _fields_ = [("n_peers", ctypes.c_int), ("n_parts", ctypes.c_int), ("me", ctypes.c_int),
                ("max_local_parts", ctypes.c_int), ("epoch", ctypes.c_uint), ("alpha", ctypes.c_float),
                ("sender_timeout_ns", ctypes.c_ulonglong), ("reducer_timeout_ns", ctypes.c_ulonglong),
                ("delta_stride", ctypes.c_ulonglong), ("weight", ctypes.c_float * MAX_PEERS),
                ("sends", ctypes.c_int * MAX_PEERS), ("peer", _HbPeer * MAX_PEERS), ("parts", ctypes.c_void_p),
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


class _RawCuda:
    """Lets torch wrap a raw device pointer without copying (CUDA array interface)."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = dict(shape=(nbytes,), typestr="|u1", data=(ptr, False), version=3)
        self._owner = owner


def _machine_id() -> str:
    try:
        with open("/proc/sys/kernel/random/boot_id") as f:
            return f.read().strip()
    except OSError:
        return socket.gethostname()


@dataclass
class RoundStatus:
    banned_senders: List[int] = field(default_factory=list)
    failed_reducers: List[int] = field(default_factory=list)
    failed_elements: int = 0
    total_elements: int = 1

    @property
    def failed_fraction(self) -> float:
        return self.failed_elements / max(self.total_elements, 1)


def record_bytes(codec: int, length: int) -> int:
    header = {1: 16, 3: 1024, 4: 1024}.get(codec, 0)
    if codec == 5:
        header = ((length + 4095) // 4096 * 4 + 15) // 16 * 16
    elem = 4 if codec == 0 else (2 if codec in (1, 2) else 1)
    return header + (length * elem + 15) // 16 * 16


@dataclass
class _Plan:
    """Everything about one (group shape, my index): part table, work lists, capacities."""

    n_parts: int
    max_local_parts: int
    delta_stride: int
    parts_dev: torch.Tensor
    items: Dict[str, torch.Tensor]
    counts: Dict[str, int]
    scratch: Dict[str, torch.Tensor]
    scratch_blob: torch.Tensor
    group_dev: torch.Tensor
    needed_outbox: int
    needed_delta: int


def _interleave_by_owner(items: List[Tuple[int, int, int, int]], owners: List[int], first_owner: int,
                         n_peers: int) -> List[Tuple[int, int, int, int]]:
    """Order work items round-robin over the GPUs they read from, starting at ``first_owner``.

    CTAs start in list order. With items grouped by owner, every member of a group would pull from owner 0 first,
    then from owner 1, ...: at any moment one GPU's outgoing links serve all readers while the others idle. Rotated
    and interleaved, concurrent reads are spread evenly over all owners.
    """
    queues: Dict[int, List[Tuple[int, int, int, int]]] = {}
    for item, owner in zip(items, owners):
        queues.setdefault(owner, []).append(item)
    order = [(first_owner + t) % n_peers for t in range(n_peers)]
    cursors = {owner: 0 for owner in queues}
    merged = []
    while len(merged) < len(items):
        for owner in order:
            queue = queues.get(owner)
            if queue is not None and cursors[owner] < len(queue):
                merged.append(queue[cursors[owner]])
                cursors[owner] += 1
    return merged


class DeviceEndpoint:
    """The device-side state of one averager: arena, mappings of groupmates' arenas, cached plans."""

    def __init__(self, tensors: Sequence[torch.Tensor], compression: CompressionBase,
                 tensor_infos: Sequence[CompressionInfo], part_size_bytes: int):
        assert len(tensors) > 0 and all(t.is_cuda and t.dtype == torch.float32 for t in tensors)
        self.device = tensors[0].device
        assert all(t.device == self.device for t in tensors), "all averaged tensors must live on one GPU"
        self.lib = _lib.load_library()
        _ensure_code_table(self.device.index)
        self.part_size_bytes = part_size_bytes
        self.numels = [t.numel() for t in tensors]
        self.codecs = [codec_id(compression, info) for info in tensor_infos]
        self.supported = all(c is not None for c in self.codecs)
        self.ratios = [{0: 1.0, 1: 0.5, 2: 0.5}.get(c, 0.25) for c in self.codecs]
        # flat layout: every tensor starts on an ALIGN-element boundary
        self.offsets, cursor = [], 0
        for n in self.numels:
            self.offsets.append(cursor)
            cursor += (n + ALIGN - 1) // ALIGN * ALIGN
        self.total = max(cursor, ALIGN)
        min_part = min([max(ALIGN, int(part_size_bytes / (4 * r)) // ALIGN * ALIGN) for r in self.ratios] or [ALIGN])
        self.max_parts = sum((n + min_part - 1) // min_part for n in self.numels) + MAX_PEERS + len(tensors)
        self.cap_outbox = self.total * 4 + self.max_parts * 1088
        self.cap_delta = int(self.cap_outbox * 2.5) + (1 << 16)  # room for uneven spans; larger groups fall back to RPC
        self.layout, self._guards = {}, {}
        cursor = 0
        for name, nbytes in (("data", self.total * 4), ("avg", self.total * 4), ("outbox", self.cap_outbox),
                             ("deltabox", self.cap_delta), ("ready", self.max_parts * 4),
                             ("delta_ready", MAX_PEERS * self.max_parts * 4)):
            self.layout[name] = cursor
            cursor += (nbytes + 255) // 256 * 256
            self._guards[name] = cursor  # a canary zone follows every region (see check_canaries)
            cursor += GUARD_BYTES
        self.arena_bytes = cursor
        base = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(self.lib.hm_arena_alloc(ctypes.byref(base), ctypes.c_ulonglong(self.arena_bytes)), "hm_arena_alloc", 0)
        self.base = base.value
        handle = (ctypes.c_ubyte * 64)()
        with torch.cuda.device(self.device):
            rc = self.lib.hm_ipc_export(ctypes.c_void_p(self.base), handle)
        self.ipc_handle = bytes(handle) if rc == 0 else None
        self._raw = _RawCuda(self.base, self.arena_bytes, self)
        self._bytes = torch.as_tensor(self._raw, device=self.device)
        for guard in self._guards.values():
            self._bytes[guard:guard + GUARD_BYTES].fill_(GUARD_PATTERN)
        flat = self._bytes[self.layout["data"]:self.layout["data"] + self.total * 4].view(torch.float32)
        self.flat = flat
        self.tensor_views = []
        with torch.no_grad():
            for t, off in zip(tensors, self.offsets):
                view = flat[off:off + t.numel()].view(t.shape)
                view.copy_(t)
                self.tensor_views.append(view.requires_grad_(t.requires_grad))
        stream = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(self.lib.hm_stream_create(ctypes.byref(stream)), "hm_stream_create", 0)
        self.stream = stream
        # torch-side handle of the same stream: every tensor that the round's kernels read is created under it, so
        # that its initialisation is ordered before the kernels (the round's stream does not synchronise with the
        # default stream, where unrelated training work may be queued)
        self._torch_stream = torch.cuda.ExternalStream(stream.value, device=self.device)
        self._mappings: Dict[Tuple[int, bytes], int] = {}
        self._plans: Dict[Tuple, _Plan] = {}
        self._host_status = (ctypes.c_ulonglong * 4)()
        self._closed = False
        self.launch_hook = None
        self.uid = os.urandom(8)

    # ---------------------------------------------------------------------------------------------- handles
    def describe(self) -> Optional[dict]:
        """What groupmates need in order to map this arena (sent in the matchmaking gather blob)."""
        if not self.supported:
            return None
        return dict(machine=_machine_id(), pid=os.getpid(), dev=self.device.index, ptr=self.base,
                    handle=self.ipc_handle, layout=self.layout, total=self.total, max_parts=self.max_parts,
                    cap_outbox=self.cap_outbox, cap_delta=self.cap_delta, uid=self.uid)

    def can_run_with(self, device_infos: Sequence[Optional[dict]], modes: Sequence[AveragingMode]) -> bool:
        if not self.supported or len(device_infos) > MAX_PEERS or len(device_infos) < 2:
            return False
        if any(info is None for info in device_infos) or any(m == AveragingMode.CLIENT for m in modes):
            return False
        mine = self.describe()
        return all(info["machine"] == mine["machine"] and info["total"] == mine["total"]
                   and info["max_parts"] == mine["max_parts"] and (info["pid"] == mine["pid"] or info["handle"])
                   for info in device_infos)

    def _map_peer(self, info: dict) -> int:
        """Base address of a groupmate's arena as seen from this GPU."""
        if info["pid"] == os.getpid():
            if info["dev"] != self.device.index:
                rc = self.lib.hm_enable_peer_access(self.device.index, info["dev"])
                if rc != 0:
                    raise RuntimeError(f"GPU {self.device.index} cannot access GPU {info['dev']} (code {rc})")
            return info["ptr"]
        key = (info["pid"], bytes(info["handle"]))
        if key not in self._mappings:
            out = ctypes.c_void_p()
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(bytes(info["handle"]))
            with torch.cuda.device(self.device):
                _lib.check(self.lib.hm_ipc_open(buf, ctypes.byref(out)), "hm_ipc_open", 0)
            self._mappings[key] = out.value
        return self._mappings[key]

    def check_canaries(self) -> None:
        """Raise if any kernel (of this GPU or of a groupmate) wrote past the end of one of the arena's regions.

        Every region of the arena is followed by ``GUARD_BYTES`` of a fixed pattern that no kernel has a reason to
        touch. Tests call this after their rounds; with ``HIVEMIND_B200_DEBUG=1`` every round ends with it (one
        small device-to-host copy and a synchronisation of the device).
        """
        torch.cuda.synchronize(self.device)
        with torch.cuda.stream(self._torch_stream):
            zones = torch.stack([self._bytes[g:g + GUARD_BYTES] for g in self._guards.values()])
            damaged = (zones != GUARD_PATTERN).any(dim=1).cpu()
        names = [name for name, bad in zip(self._guards, damaged.tolist()) if bad]
        if names:
            raise RuntimeError(f"device butterfly: memory past the end of region(s) {names} was overwritten")

    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        # groupmates pull their deltas out of this arena after this GPU has finished its own part of a round:
        # do not let the process go (and the memory with it) right after a round
        since_round = time.monotonic() - getattr(self, "_last_round_end", -1e9)
        if since_round < EXIT_GRACE_SECONDS:
            time.sleep(EXIT_GRACE_SECONDS - since_round)
        with torch.cuda.device(self.device):
            self.lib.hm_stream_sync(self.stream)
            for ptr in self._mappings.values():
                self.lib.hm_ipc_close(ctypes.c_void_p(ptr))
            self.lib.hm_stream_destroy(self.stream)
        # the arena itself is intentionally kept until process exit: tensor views handed to the user and
        # mappings held by other processes must never dangle

    # ---------------------------------------------------------------------------------------------- planning
    def _make_plan(self, n_peers: int, my_index: int, peer_fractions: Sequence[float], sends: Sequence[bool]) -> _Plan:
        key = (n_peers, my_index, tuple(peer_fractions), tuple(sends))
        plan = self._plans.get(key)
        if plan is not None:
            return plan
        with torch.cuda.stream(self._torch_stream):
            plan = self._build_plan(n_peers, my_index, peer_fractions, sends)
            self._torch_stream.synchronize()  # once per layout: tables and zeroed scratch are in place before any launch
        if len(self._plans) > 8:
            self._plans.pop(next(iter(self._plans)))
        self._plans[key] = plan
        return plan

    def _build_plan(self, n_peers: int, my_index: int, peer_fractions: Sequence[float], sends: Sequence[bool]) -> _Plan:
        lib = self.lib
        chunk = lib.hm_bf_chunk()
        specs = compute_part_layout(self.numels, [4] * len(self.numels), self.ratios, peer_fractions,
                                    self.part_size_bytes, align=ALIGN)
        specs = [s for s in specs if s.length > 0]
        n_parts = len(specs)
        if n_parts > self.max_parts:
            raise RuntimeError("too many parts for the arena's flag pages")
        table = np.zeros(n_parts, dtype=_PART_DTYPE)
        local_count = [0] * n_peers
        span_bytes = [0] * n_peers
        enc_cursor = 0
        for p, s in enumerate(specs):
            codec = self.codecs[s.tensor_index]
            rec = record_bytes(codec, s.length)
            start = self.offsets[s.tensor_index] + s.start
            table[p] = (start, enc_cursor, span_bytes[s.owner], start, s.length, s.owner, local_count[s.owner], codec)
            enc_cursor += rec
            span_bytes[s.owner] += rec
            local_count[s.owner] += 1
        max_local = max(max(local_count), 1)
        delta_stride = (max(span_bytes) + 255) // 256 * 256
        needed_delta = n_peers * delta_stride

        def chunks_of(p):
            return range((int(table[p]["len"]) + chunk - 1) // chunk)

        i_send = sends[my_index]
        mine = [p for p in range(n_parts) if table[p]["owner"] == my_index]
        theirs = [p for p in range(n_parts) if table[p]["owner"] != my_index] if i_send else []
        senders = [s for s in range(n_peers) if s != my_index and sends[s]]
        lists = {
            # uncompressed parts have no records: reducers read the vector in place, senders read the average
            "enc": [(p, c, 0, 0) for p in theirs if table[p]["codec"] != CODEC_NONE for c in chunks_of(p)],
            "enc_stats": [(p, c, 0, 0) for p in theirs if table[p]["codec"] in _NEEDS_STATS for c in chunks_of(p)],
            "enc_borders": [(p, 0, 0, 0) for p in theirs if table[p]["codec"] in _NEEDS_BORDERS],
            "enc_publish": [(p, 0, 0, 0) for p in theirs],
            "reduce": [(p, c, 0, 0) for p in mine for c in chunks_of(p)],
            "delta": [(p, c, s, 0) for s in senders for p in mine if table[p]["codec"] != CODEC_NONE
                      for c in chunks_of(p)],
            "delta_borders": [(p, 0, s, 0) for s in senders for p in mine if table[p]["codec"] in _NEEDS_BORDERS],
            "delta_publish": [(p, 0, s, 0) for s in senders for p in mine],
            "apply": _interleave_by_owner([(p, c, 0, 0) for p in theirs for c in chunks_of(p)],  # own span: applied
                                          [int(table[p]["owner"]) for p in theirs for _ in chunks_of(p)],  # by reduce
                                          first_owner=(my_index + 1) % n_peers, n_peers=n_peers),
        }
        items = {k: torch.tensor(v if v else [(0, 0, 0, 0)], dtype=torch.int32).to(self.device) for k, v in lists.items()}
        counts = {k: len(v) for k, v in lists.items()}
        parts_dev = torch.from_numpy(table.view(np.uint8).copy()).to(self.device)
        slots = MAX_PEERS * max_local
        sizes = [("part_stats", n_parts * 16), ("dstats", slots * 16), ("bins", n_parts * 1024), ("bin_cnt", n_parts * 1024),
                 ("dbins", slots * 1024), ("dbin_cnt", slots * 1024), ("include", max_local * MAX_PEERS * 4),
                 ("apply_decision", n_parts * 4), ("ban", MAX_PEERS * 4), ("t_start", 16), ("status", 32),
                 ("borders", n_parts * 1024), ("dborders", slots * 1024)]
        total = sum((b + 255) // 256 * 256 for _, b in sizes)
        blob = torch.zeros(total, dtype=torch.uint8, device=self.device)
        scratch, cursor = {}, 0
        for name, nbytes in sizes:
            scratch[name] = blob[cursor:cursor + nbytes]
            cursor += (nbytes + 255) // 256 * 256
        group_dev = torch.zeros(ctypes.sizeof(_HbGroup), dtype=torch.uint8, device=self.device)
        return _Plan(n_parts, max_local, delta_stride, parts_dev, items, counts, scratch, blob, group_dev, enc_cursor,
                     needed_delta)

    def _prepare(self, *, group_id: bytes, my_index: int, device_infos, modes, peer_fractions, weights, alpha,
                 sender_timeout, reducer_timeout, stream) -> _Plan:
        n = len(device_infos)
        sends = [m != AveragingMode.AUX for m in modes]
        plan = self._make_plan(n, my_index, peer_fractions, sends)
        for info in device_infos:
            if plan.needed_outbox > info["cap_outbox"] or plan.needed_delta > info["cap_delta"]:
                raise RuntimeError("the staging areas of the arenas are too small for this group layout")
        g = _HbGroup()
        g.n_peers, g.n_parts, g.me, g.max_local_parts = n, plan.n_parts, my_index, plan.max_local_parts
        g.epoch = (zlib.crc32(group_id) & 0x7FFFFFFF) | 1
        g.alpha = alpha
        g.sender_timeout_ns = int(min(sender_timeout if sender_timeout else 10.0, 20.0) * 1e9)
        g.reducer_timeout_ns = int(min(reducer_timeout if reducer_timeout else 20.0, 40.0) * 1e9)
        g.delta_stride = plan.delta_stride
        for r, info in enumerate(device_infos):
            base = self.base if r == my_index else self._map_peer(info)
            lay = info["layout"]
            g.weight[r] = float(weights[r])
            g.sends[r] = int(sends[r])
            g.peer[r].data = base + lay["data"]
            g.peer[r].outbox = base + lay["outbox"]
            g.peer[r].deltabox = base + lay["deltabox"]
            g.peer[r].ready = base + lay["ready"]
            g.peer[r].delta_ready = base + lay["delta_ready"]
            g.peer[r].avg = base + lay["avg"]
        g.parts = plan.parts_dev.data_ptr()
        for name in ("part_stats", "dstats", "bins", "bin_cnt", "dbins", "dbin_cnt", "borders", "dborders", "include",
                     "apply_decision", "ban", "t_start", "status"):
            setattr(g, name, plan.scratch[name].data_ptr())
        g.avg = self.base + self.layout["avg"]
        plan._host_group = g  # keep the host copy alive until the async upload has been consumed
        lib = self.lib
        with torch.cuda.device(self.device):
            _lib.check(lib.hm_memset_async(ctypes.c_void_p(plan.scratch_blob.data_ptr()), 0,
                                           ctypes.c_ulonglong(plan.scratch_blob.numel()), stream), "memset", 0)
            _lib.check(lib.hm_memcpy_h2d_async(ctypes.c_void_p(plan.group_dev.data_ptr()), ctypes.byref(g),
                                               ctypes.c_ulonglong(ctypes.sizeof(g)), stream), "upload group", 0)
        return plan

    def _launch(self, plan: _Plan, phase: int, items: str, mode: int, stream) -> None:
        count = plan.counts[items]
        if count == 0:
            return
        with torch.cuda.device(self.device):
            code = self.lib.hm_bf_launch(phase, ctypes.c_void_p(plan.group_dev.data_ptr()),
                                         ctypes.c_void_p(plan.items[items].data_ptr()), count, mode, stream)
        _lib.check(code, f"hm_bf_launch(phase={phase}, {items})")
        if self.launch_hook is not None:
            self.launch_hook(items)  # benchmarks record an event after every launch of a round

    # the three stages of a round; in normal operation they are launched back to back on one stream
    def _stage_send(self, plan, stream) -> None:
        self._launch(plan, PH_STATS, "enc_stats", 0, stream)
        self._launch(plan, PH_BORDERS, "enc_borders", 0, stream)
        self._launch(plan, PH_ENCODE, "enc", 0, stream)
        self._launch(plan, PH_PUBLISH, "enc_publish", 0, stream)

    def _stage_reduce(self, plan, stream) -> None:
        self._launch(plan, PH_REDUCE, "reduce", 0, stream)
        self._launch(plan, PH_BORDERS, "delta_borders", 1, stream)
        self._launch(plan, PH_ENCODE, "delta", 1, stream)
        self._launch(plan, PH_PUBLISH, "delta_publish", 1, stream)

    def _stage_apply(self, plan, stream) -> None:
        self._launch(plan, PH_APPLY, "apply", 0, stream)

    def _read_status(self, plan: _Plan, stream) -> RoundStatus:
        with torch.cuda.device(self.device):
            _lib.check(self.lib.hm_memcpy_d2h(self._host_status, ctypes.c_void_p(plan.scratch["status"].data_ptr()),
                                              ctypes.c_ulonglong(32), stream), "read status", 0)
        banned, failed, elements = self._host_status[0], self._host_status[1], self._host_status[2]
        return RoundStatus([i for i in range(MAX_PEERS) if banned >> i & 1], [i for i in range(MAX_PEERS) if failed >> i & 1],
                           int(elements), sum(self.numels))

    def run_round(self, *, group_id: bytes, my_index: int, device_infos, modes, peer_fractions, weights, alpha: float,
                  sender_timeout: Optional[float], reducer_timeout: Optional[float]) -> RoundStatus:
        """Run one all-reduce round with the mapped groupmates; blocks the calling thread until this GPU is done."""
        # the caller's writes to the tensors must land before the round reads them: order the round's stream after the
        # caller's stream on the device (no host wait: that stream may hold work that depends on other ranks)
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(self.device))
        self._torch_stream.wait_event(ready)
        plan = self._prepare(group_id=group_id, my_index=my_index, device_infos=device_infos, modes=modes,
                             peer_fractions=peer_fractions, weights=weights, alpha=alpha,
                             sender_timeout=sender_timeout, reducer_timeout=reducer_timeout, stream=self.stream)
        with device_range("butterfly.send", self._torch_stream):
            self._stage_send(plan, self.stream)
        with device_range("butterfly.reduce", self._torch_stream):
            self._stage_reduce(plan, self.stream)
        with device_range("butterfly.apply", self._torch_stream):
            self._stage_apply(plan, self.stream)
        status = self._read_status(plan, self.stream)
        self._last_round_end = time.monotonic()
        if DEBUG_CHECKS:
            self.check_canaries()
        return status


def run_group_emulated(endpoints: Sequence[DeviceEndpoint], *, weights: Sequence[float],
                       peer_fractions: Sequence[float], modes: Optional[Sequence[AveragingMode]] = None,
                       alpha: float = 1.0, group_id: bytes = b"emulated", sender_timeout: float = 1.0,
                       reducer_timeout: float = 2.0, skip_send_of: Sequence[int] = (),
                       publish_only_first_half_of: Sequence[int] = ()) -> List[RoundStatus]:
    """Run a whole group inside one process, stage by stage: first every rank's send stage, then every rank's
    reduce stage, then every rank's apply stage, so that no launch ever waits for a later one. Used when there are
    fewer GPUs than ranks, and by tests that inject host-side faults: ``skip_send_of`` ranks never publish their
    parts (a sender that does not show up), ``publish_only_first_half_of`` ranks stall after half of their parts.
    """
    n = len(endpoints)
    modes = list(modes) if modes is not None else [AveragingMode.NODE] * n
    infos = [e.describe() for e in endpoints]
    streams = [ctypes.c_void_p(torch.cuda.current_stream(e.device).cuda_stream) for e in endpoints]
    plans = [e._prepare(group_id=group_id, my_index=r, device_infos=infos, modes=modes, peer_fractions=peer_fractions,
                        weights=weights, alpha=alpha, sender_timeout=sender_timeout, reducer_timeout=reducer_timeout,
                        stream=streams[r]) for r, e in enumerate(endpoints)]
    for r, e in enumerate(endpoints):
        if r in skip_send_of:
            continue
        if r in publish_only_first_half_of:
            full = plans[r].counts["enc_publish"]
            plans[r].counts["enc_publish"] = full // 2
            e._stage_send(plans[r], streams[r])
            plans[r].counts["enc_publish"] = full
        else:
            e._stage_send(plans[r], streams[r])
    for e in endpoints:
        torch.cuda.synchronize(e.device)
    for r, e in enumerate(endpoints):
        e._stage_reduce(plans[r], streams[r])
    for e in endpoints:
        torch.cuda.synchronize(e.device)
    for r, e in enumerate(endpoints):
        e._stage_apply(plans[r], streams[r])
    return [e._read_status(plans[r], streams[r]) for r, e in enumerate(endpoints)]

"""Host side of the device butterfly: arenas, handle exchange, part tables and the launches of a round.

One ``DeviceEndpoint`` belongs to one averager (one GPU). It owns a single device allocation ("arena") that holds the
averaged tensors as one flat fp32 vector plus the staging areas that other GPUs read: the outbox with encoded chunk
records, the delta box with encoded averages-minus-input, the averages of uncompressed parts and the flag pages. The
staging areas exist twice and alternate between this endpoint's rounds (``parity``), so that a groupmate that is
still reading the results of round r is not disturbed when this endpoint begins round r + 1 with somebody else; before
a staging copy is used again (round r + 2) the gate kernel checks that the readers of round r have acknowledged.

At group assembly every member's ``describe()`` blob travels in the matchmaking ``gather`` field; members map each
other's arenas (CUDA IPC across processes, peer access inside one process) and then each runs ``run_round``: a gate
kernel and ONE persistent round kernel (``ops/csrc/butterfly_round.cu``) on a private stream, with no host
synchronisation until the end. Averaging weights travel inside the senders' flags, so no extra RPC precedes a round.

Division of labour with the reference: ``TensorPartContainer`` / ``TensorPartReducer`` / ``AllReduceRunner``
(hivemind/averaging/partition.py, allreduce.py) become a part table in device memory, bounded flag waits and
per-part inclusion decisions; load balancing, modes, weights and timeouts keep their meaning. A client-mode peer is
an ordinary member with an empty span here: its arena can be read like anybody else's.
"""
from __future__ import annotations

import ctypes
import os
import socket
import threading
import time
import zlib
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from hivemind_b200.averaging.allreduce import AveragingMode
from hivemind_b200.averaging.partition import compute_part_layout
from hivemind_b200.compression import (BlockwiseQuantization, CompressionBase, CompressionInfo, Float16Compression,
                                       NoCompression, Quantile8BitQuantization, ScaledFloat16Compression,
                                       Uniform8BitQuantization)
from hivemind_b200.compression.adaptive import AdaptiveCompressionBase
from hivemind_b200.compression.quantization import dynamic_code_table
from hivemind_b200.ops import _lib
from hivemind_b200.utils.logging import get_logger
from hivemind_b200.utils.profiling import device_range

logger = get_logger(__name__)

GUARD_BYTES, GUARD_PATTERN = 256, 0xA5  # canary zones between the regions of an arena
DEBUG_CHECKS = os.environ.get("HIVEMIND_B200_DEBUG", "0") == "1"
EXIT_GRACE_SECONDS = 2.0  # how long after a round peers may still read this arena (see DeviceEndpoint.close)
MAX_PEERS = 16
ALIGN = 16  # elements: tensor starts and part boundaries are multiples of this, so every access is 16-byte aligned
CHUNK = 8192  # elements per chunk record (HR_CHUNK in butterfly_round.cu)
ACK_RING = 8
CTAS_PER_SM = 2  # the round kernel keeps two 512-thread CTAs on every SM
GRID_CTAS = 296  # CTAs of the round kernel on a B200; a constant, because all members must derive the same part table
MAX_PART_CHUNKS = 16
ITEM_CHUNKS = int(os.environ.get("HIVEMIND_B200_ITEM_CHUNKS", "0"))  # chunks per work item; 0 = one item per part
DELTA_BOX_FACTOR = 1.5  # delta box capacity relative to the outbox: 1.0 suffices for equal spans
_CODEC_IDS = {NoCompression: 0, ScaledFloat16Compression: 1, Float16Compression: 2, Quantile8BitQuantization: 3,
              Uniform8BitQuantization: 4, BlockwiseQuantization: 5}
CODEC_NONE = 0  # uncompressed parts are read in place: no outbox record, no delta record
_HEADER_BYTES = {0: 0, 1: 16, 2: 0, 3: 1024, 4: 1024, 5: 16}
_ELEM_BYTES = {0: 4, 1: 2, 2: 2, 3: 1, 4: 1, 5: 1}

# distinguishes processes reliably (pids repeat across containers that share a boot id)
_PROCESS_TOKEN = os.urandom(16)


def codec_id(compression: CompressionBase, info: CompressionInfo) -> Optional[int]:
    """Device codec id for a tensor, or None if the codec has no device implementation."""
    while isinstance(compression, AdaptiveCompressionBase):
        compression = compression.choose_compression(info)
    return _CODEC_IDS.get(type(compression))


def device_part_chunks(total_elements: int, n_peers: int) -> int:
    """Chunks per part on the device path. A part is the unit of flag publication and (by default) one work item of
    one CTA, so parts are cut such that a reducer's span falls into whole waves of ``GRID_CTAS`` parts of at most
    ``MAX_PART_CHUNKS`` chunks: long enough to spread the fixed cost of an item, short enough that groupmates can start
    on a part soon after its owner has finished it. (The ``part_size_bytes`` of the RPC path plays no part here:
    these parts never leave the box.)"""
    span = -(-(-(-total_elements // CHUNK)) // max(n_peers, 1))
    waves = max(1, -(-span // (GRID_CTAS * MAX_PART_CHUNKS)))
    return max(1, -(-span // (GRID_CTAS * waves)))


def chunk_stride(codec: int) -> int:
    """Bytes of one chunk record: header + a full chunk of payload (also for the last, shorter chunk of a part)."""
    return _HEADER_BYTES[codec] + CHUNK * _ELEM_BYTES[codec]


def record_bytes(codec: int, length: int) -> int:
    """Bytes of all chunk records of one part (0 for uncompressed parts, which have no records)."""
    if codec == CODEC_NONE:
        return 0
    return chunk_stride(codec) * ((length + CHUNK - 1) // CHUNK)


class _HrLayout(ctypes.Structure):
    _fields_ = [("data", ctypes.c_ulonglong), ("avg", ctypes.c_ulonglong * 2), ("outbox", ctypes.c_ulonglong * 2),
                ("deltabox", ctypes.c_ulonglong * 2), ("ready", ctypes.c_ulonglong * 2),
                ("dready", ctypes.c_ulonglong * 2), ("hello", ctypes.c_ulonglong), ("done_ring", ctypes.c_ulonglong)]


class _HrRound(ctypes.Structure):
    _fields_ = [("n_peers", ctypes.c_int), ("n_parts", ctypes.c_int), ("me", ctypes.c_int),
                ("max_local_parts", ctypes.c_int), ("epoch", ctypes.c_uint), ("parity", ctypes.c_int),
                ("alpha", ctypes.c_float), ("my_weight", ctypes.c_float),
                ("sender_timeout_ns", ctypes.c_ulonglong), ("reducer_timeout_ns", ctypes.c_ulonglong),
                ("delta_stride", ctypes.c_ulonglong), ("sends", ctypes.c_int * MAX_PEERS),
                ("base", ctypes.c_void_p * MAX_PEERS), ("lay", _HrLayout), ("parts", ctypes.c_void_p),
                ("items", ctypes.c_void_p), ("pub_list", ctypes.c_void_p), ("n_send", ctypes.c_int),
                ("n_reduce", ctypes.c_int), ("n_apply", ctypes.c_int), ("item_begin", ctypes.c_int),
                ("item_end", ctypes.c_int), ("queue_slot", ctypes.c_int), ("final_stage", ctypes.c_int),
                ("include", ctypes.c_void_p), ("apply_decision", ctypes.c_void_p), ("ban", ctypes.c_void_p),
                ("t_start", ctypes.c_void_p), ("status", ctypes.c_void_p), ("status_out", ctypes.c_void_p),
                ("part_done", ctypes.c_void_p), ("dpart_done", ctypes.c_void_p), ("queue", ctypes.c_void_p),
                ("code", ctypes.c_void_p), ("done_slot", ctypes.c_uint), ("uses_blockwise", ctypes.c_int),
                ("trace", ctypes.c_void_p)]


class _HrGate(ctypes.Structure):
    _fields_ = [("n_peers", ctypes.c_int), ("me", ctypes.c_int), ("parity", ctypes.c_int), ("n_prev", ctypes.c_int),
                ("epoch", ctypes.c_uint), ("prev_epoch", ctypes.c_uint), ("ack_timeout_ns", ctypes.c_ulonglong),
                ("hello_timeout_ns", ctypes.c_ulonglong), ("base", ctypes.c_void_p * MAX_PEERS),
                ("prev_base", ctypes.c_void_p * MAX_PEERS), ("lay", _HrLayout), ("gate_status", ctypes.c_void_p)]


_PART_DTYPE = np.dtype([("start", "<i8"), ("enc_off", "<i8"), ("span_off", "<i8"), ("avg_off", "<i8"), ("len", "<i4"),
                        ("owner", "<i4"), ("local_idx", "<i4"), ("codec", "<i4")])

_code_tables: Dict[int, torch.Tensor] = {}
_code_lock = threading.Lock()


def _code_table_on(device: torch.device) -> torch.Tensor:
    """On the device: the block-wise code (256 fp32, sorted), the midpoints between consecutive entries (256 fp32, the
    last one +inf) and a 16 KB table that starts the search for a value's code: entry k is the number of midpoints
    below the smallest float whose order-preserving key (sign-flipped bits) has k as its top 14 bits."""
    with _code_lock:
        table = _code_tables.get(device.index)
        if table is None:
            lib = _lib.load_library()
            assert lib.hm_br_sizeof_round() == ctypes.sizeof(_HrRound), "HrRound layout mismatch between C and Python"
            assert lib.hm_br_sizeof_gate() == ctypes.sizeof(_HrGate), "HrGate layout mismatch between C and Python"
            assert lib.hm_br_sizeof_part() == _PART_DTYPE.itemsize, "HrPart layout mismatch between C and Python"
            assert lib.hm_br_chunk() == CHUNK
            code = dynamic_code_table().to(torch.float32)
            mid = torch.cat([(code[:-1] + code[1:]) * 0.5, torch.tensor([float("inf")])])
            keys = (torch.arange(1 << 14, dtype=torch.int64) << 18).numpy().astype(np.uint32)
            bits = np.where(keys >> 31 != 0, keys ^ np.uint32(0x80000000), ~keys)  # undo the order-preserving map
            lowest = torch.from_numpy(bits.view(np.float32).copy())
            lowest = torch.nan_to_num(lowest, nan=float("inf"), posinf=float("inf"), neginf=-float("inf"))
            start = torch.bucketize(lowest, mid[:255].contiguous()).to(torch.uint8)  # midpoints strictly below the value
            table = torch.cat([code, mid, torch.from_numpy(start.numpy().view(np.float32).copy())]).to(device)
            _code_tables[device.index] = table
        return table


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


@dataclass
class _Plan:
    """Everything about one (group shape, my index): part table, the ordered work list, scratch."""

    n_parts: int
    max_local_parts: int
    delta_stride: int
    parts_dev: torch.Tensor
    items_dev: torch.Tensor
    pub_dev: torch.Tensor
    n_send: int
    n_reduce: int
    n_apply: int
    send_cut: int  # number of send items that cover the first half of the parts this rank sends (fault injection)
    scratch: Dict[str, torch.Tensor]
    scratch_blob: torch.Tensor
    needed_outbox: int
    needed_delta: int
    needed_avg: int
    rounds: Dict[Tuple, "_HrRound"] = field(default_factory=dict)  # parameter blocks by (groupmates, timeouts)


def _interleave_by_owner(items: List[Tuple[int, int, int, int]], owners: List[int], first_owner: int,
                         n_peers: int) -> List[Tuple[int, int, int, int]]:
    """Order work items round-robin over the GPUs they read from, starting at ``first_owner``.

    CTAs take items in list order. With items grouped by owner, every member of a group would pull from owner 0
    first, then from owner 1, ...: at any moment one GPU's outgoing links serve all readers while the others idle.
    Rotated and interleaved, concurrent reads are spread evenly over all owners.
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


def peers_can_share_memory(mine: dict, infos: Sequence[Optional[dict]]) -> bool:
    """Whether a group described by ``infos`` can run on the device path from the point of view of ``mine``.

    The rule is symmetric, so that every member reaches the same verdict: same machine, identical arena layouts, and
    for every pair of members that live in different processes BOTH sides exported an IPC handle. Processes are told
    apart by a random per-process token (pids and device indices repeat across containers of one host).
    """
    if len(infos) < 2 or len(infos) > MAX_PEERS or any(info is None for info in infos):
        return False
    if any(not info.get("supported", True) for info in infos):
        return False
    for info in infos:
        if info["machine"] != mine["machine"] or info["layout"] != mine["layout"] or info["total"] != mine["total"]:
            return False
    procs = {bytes(info["proc"]) for info in infos}
    if len(procs) > 1 and any(not info.get("handle") for info in infos):
        return False
    return True


class DeviceEndpoint:
    """The device-side state of one averager: arena, mappings of groupmates' arenas, cached plans."""

    def __init__(self, tensors: Sequence[torch.Tensor], compression: CompressionBase,
                 tensor_infos: Sequence[CompressionInfo], part_size_bytes: int):
        assert len(tensors) > 0 and all(t.is_cuda and t.dtype == torch.float32 for t in tensors)
        self.device = tensors[0].device
        assert all(t.device == self.device for t in tensors), "all averaged tensors must live on one GPU"
        self.lib = _lib.load_library()
        self._code = _code_table_on(self.device)
        self.part_size_bytes = part_size_bytes  # the RPC path's part size; device parts are sized by device_part_chunks
        self.numels = [t.numel() for t in tensors]
        self.codecs = [codec_id(compression, info) for info in tensor_infos]
        self.supported = all(c is not None for c in self.codecs)
        codecs = [c if c is not None else 0 for c in self.codecs]
        # flat layout: every tensor starts on an ALIGN-element boundary; uncompressed tensors also get a place in
        # the (compact) average buffer
        self.offsets, self.avg_offsets, cursor, avg_cursor = [], [], 0, 0
        for n, c in zip(self.numels, codecs):
            padded = (n + ALIGN - 1) // ALIGN * ALIGN
            self.offsets.append(cursor)
            self.avg_offsets.append(avg_cursor)
            cursor += padded
            if c == CODEC_NONE:
                avg_cursor += padded
        self.total = max(cursor, ALIGN)
        # flag pages hold the largest part table that any group size can produce
        self.max_parts = max(sum(-(-n // (device_part_chunks(sum(self.numels), peers) * CHUNK)) for n in self.numels)
                             for peers in range(1, MAX_PEERS + 1)) + MAX_PEERS + len(tensors)
        # staging capacities by codec: records exist only for compressed tensors, averages only for uncompressed ones.
        # Parts are whole chunks except where a tensor ends or a peer's share ends: at most MAX_PEERS + 1 extra records
        self.cap_avg = max(avg_cursor * 4, 256)
        self.cap_outbox = max(256, sum(((n + CHUNK - 1) // CHUNK + MAX_PEERS + 1) * chunk_stride(c)
                                       for n, c in zip(self.numels, codecs) if c != CODEC_NONE))
        self.cap_delta = int(self.cap_outbox * DELTA_BOX_FACTOR) + (1 << 12) if self.cap_outbox > 256 else 256
        self.layout: Dict[str, int] = {}
        self._guards: Dict[str, int] = {}
        cursor = 0
        regions = [("data", self.total * 4)]
        for par in (0, 1):
            regions += [(f"avg{par}", self.cap_avg), (f"outbox{par}", self.cap_outbox), (f"deltabox{par}", self.cap_delta),
                        (f"ready{par}", self.max_parts * 8), (f"dready{par}", MAX_PEERS * self.max_parts * 4)]
        regions += [("hello", 16), ("done_ring", ACK_RING * 4)]
        for name, nbytes in regions:
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
        for name in ("ready0", "ready1", "dready0", "dready1", "hello", "done_ring"):  # flags start out as "no round"
            lo = self.layout[name]
            self._bytes[lo:self._guards[name]].zero_()
        flat = self._bytes[self.layout["data"]:self.layout["data"] + self.total * 4].view(torch.float32)
        flat.zero_()  # the padding between tensors is averaged along with them: it must hold numbers
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
        with torch.cuda.stream(self._torch_stream):
            self._status_out = torch.zeros(4, dtype=torch.int64, device=self.device)
            self._gate_status = torch.zeros(2, dtype=torch.int64, device=self.device)
            self._torch_stream.synchronize()
        self._mappings: Dict[Tuple[bytes, bytes], int] = {}
        self._plans: Dict[Tuple, _Plan] = {}
        self._host_status = (ctypes.c_ulonglong * 4)()
        self._closed = False
        self.launch_hook = None
        self.uid = os.urandom(8)
        self._round_seq = 0
        self._history: Dict[int, Tuple[int, List[int]]] = {}  # parity -> (epoch, bases of that round's groupmates)
        self._sms = _lib.sm_count(self.device)
        self.fault_publish_half = False  # host-side fault injection: publish only the first half of the parts sent
        self.trace: Optional[torch.Tensor] = None  # see enable_trace()
        self._gate = _HrGate()  # the gate kernel's parameter block (launches copy it, so one instance serves all rounds)
        self._gate.lay = self._layout_struct()
        self._gate.gate_status = self._gate_status.data_ptr()

    # ---------------------------------------------------------------------------------------------- handles
    def describe(self) -> Optional[dict]:
        """What groupmates need in order to map this arena (sent in the matchmaking gather blob)."""
        if not self.supported:
            return None
        return dict(machine=_machine_id(), proc=_PROCESS_TOKEN, dev=self.device.index, ptr=self.base,
                    handle=self.ipc_handle, layout=self.layout, total=self.total, max_parts=self.max_parts,
                    cap_outbox=self.cap_outbox, cap_delta=self.cap_delta, cap_avg=self.cap_avg, uid=self.uid,
                    supported=True)

    def can_run_with(self, device_infos: Sequence[Optional[dict]], modes: Sequence[AveragingMode]) -> bool:
        """True if this round can use the device path; every member of the group reaches the same verdict."""
        if not self.supported or self._closed:
            return False
        return peers_can_share_memory(self.describe(), device_infos)

    def _map_peer(self, info: dict) -> int:
        """Base address of a groupmate's arena as seen from this GPU."""
        if bytes(info["proc"]) == _PROCESS_TOKEN:
            if info["dev"] != self.device.index:
                rc = self.lib.hm_enable_peer_access(self.device.index, info["dev"])
                if rc != 0:
                    raise RuntimeError(f"GPU {self.device.index} cannot access GPU {info['dev']} (code {rc})")
            return info["ptr"]
        key = (bytes(info["proc"]), bytes(info["handle"]))
        if key not in self._mappings:
            out = ctypes.c_void_p()
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(bytes(info["handle"]))
            with torch.cuda.device(self.device):
                _lib.check(self.lib.hm_ipc_open(buf, ctypes.byref(out)), "hm_ipc_open", 0)
            self._mappings[key] = out.value
        return self._mappings[key]

    def map_group(self, device_infos: Sequence[dict], my_index: int) -> List[int]:
        """Map every groupmate's arena. If that fails, this endpoint stops offering the device path (its later
        ``describe()`` blobs say so, and whole groups then use the RPC butterfly) and the error is re-raised."""
        try:
            return [self.base if r == my_index else self._map_peer(info) for r, info in enumerate(device_infos)]
        except Exception:
            self.supported = False
            logger.warning("could not map a groupmate's device arena; this peer uses the RPC butterfly from now on")
            raise

    def enable_trace(self) -> torch.Tensor:
        """Let the round kernel stamp, per CTA, when it started, entered and left its first reduce and apply items,
        learned about their flags and finished (12 ``globaltimer`` values per CTA, zero where a CTA had no such item).
        The tensor is overwritten by every round; zero it between rounds that are to be compared."""
        if self.trace is None:
            with torch.cuda.stream(self._torch_stream):
                self.trace = torch.zeros(CTAS_PER_SM * self._sms, 12, dtype=torch.int64, device=self.device)
                self._torch_stream.synchronize()
        return self.trace

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
        part_bytes = device_part_chunks(sum(self.numels), n_peers) * CHUNK * 4
        specs = compute_part_layout(self.numels, [4] * len(self.numels), [1.0] * len(self.numels), peer_fractions,
                                    part_bytes, align=ALIGN)
        specs = [s for s in specs if s.length > 0]
        n_parts = len(specs)
        if n_parts > self.max_parts:
            raise RuntimeError("too many parts for the arena's flag pages")
        table = np.zeros(n_parts, dtype=_PART_DTYPE)
        local_count, span_bytes, enc_cursor = [0] * n_peers, [0] * n_peers, 0
        for p, s in enumerate(specs):
            codec = self.codecs[s.tensor_index]
            rec = record_bytes(codec, s.length)
            start = self.offsets[s.tensor_index] + s.start
            avg_off = self.avg_offsets[s.tensor_index] + s.start if codec == CODEC_NONE else 0
            # kernels move four elements at a time; a tensor's last part borrows from the zero padding behind it
            length = (s.length + 3) // 4 * 4
            table[p] = (start, enc_cursor, span_bytes[s.owner], avg_off, length, s.owner, local_count[s.owner], codec)
            enc_cursor += rec
            span_bytes[s.owner] += rec
            local_count[s.owner] += 1
        max_local = max(max(local_count), 1)
        delta_stride = (max(span_bytes) + 255) // 256 * 256
        needed_delta = n_peers * delta_stride

        def n_chunks(p):
            return (int(table[p]["len"]) + CHUNK - 1) // CHUNK

        # an item is a run of consecutive chunks of one part; by default the whole part (see device_part_chunks)
        run = ITEM_CHUNKS if ITEM_CHUNKS > 0 else MAX_PART_CHUNKS

        def runs_of(p):
            total = n_chunks(p)
            return [(p, c, min(run, total - c), 0) for c in range(0, total, run)]

        i_send = sends[my_index]
        mine = [p for p in range(n_parts) if table[p]["owner"] == my_index]
        theirs = [p for p in range(n_parts) if table[p]["owner"] != my_index] if i_send else []
        # send items in part order; runs of uncompressed parts become "publish the flags of pub_list[a : a + n]" items
        send_items: List[Tuple[int, int, int, int]] = []
        pub_list: List[int] = []
        half_index, send_cut = len(theirs) // 2, 0
        for rank, p in enumerate(theirs):
            if rank == half_index:
                send_cut = len(send_items)
            if table[p]["codec"] == CODEC_NONE:
                last = send_items[-1] if send_items else None
                if last is not None and last[0] == -1 and last[1] + last[2] == len(pub_list) and last[2] < 512 \
                        and rank != half_index:
                    send_items[-1] = (-1, last[1], last[2] + 1, 0)
                else:
                    send_items.append((-1, len(pub_list), 1, 0))
                pub_list.append(p)
            else:
                send_items += runs_of(p)
        reduce_items = [item for p in mine for item in runs_of(p)]
        apply_items = _interleave_by_owner([item for p in theirs for item in runs_of(p)],
                                           [int(table[p]["owner"]) for p in theirs for _ in runs_of(p)],
                                           first_owner=(my_index + 1) % n_peers, n_peers=n_peers)
        items = send_items + reduce_items + apply_items
        items_dev = torch.tensor(items if items else [(0, 0, 0, 0)], dtype=torch.int32).to(self.device)
        pub_dev = torch.tensor(pub_list if pub_list else [0], dtype=torch.int32).to(self.device)
        parts_dev = torch.from_numpy(table.view(np.uint8).copy()).to(self.device)
        slots = MAX_PEERS * max_local
        sizes = [("include", slots * 8), ("dpart_done", slots * 4), ("apply_decision", n_parts * 8),
                 ("part_done", n_parts * 4), ("ban", MAX_PEERS * 4), ("t_start", 16), ("status", 32), ("queue", 16)]
        total = sum((b + 255) // 256 * 256 for _, b in sizes)
        blob = torch.zeros(total, dtype=torch.uint8, device=self.device)
        scratch, cursor = {}, 0
        for name, nbytes in sizes:
            scratch[name] = blob[cursor:cursor + nbytes]
            cursor += (nbytes + 255) // 256 * 256
        needed_avg = max([(int(table[p]["avg_off"]) + int(table[p]["len"])) * 4 for p in range(n_parts)
                          if table[p]["codec"] == CODEC_NONE] or [0])
        return _Plan(n_parts, max_local, delta_stride, parts_dev, items_dev, pub_dev, len(send_items), len(reduce_items),
                     len(apply_items), send_cut, scratch, blob, enc_cursor, needed_delta, needed_avg)

    def _layout_struct(self) -> _HrLayout:
        lay = _HrLayout()
        lay.data = self.layout["data"]
        for par in (0, 1):
            lay.avg[par] = self.layout[f"avg{par}"]
            lay.outbox[par] = self.layout[f"outbox{par}"]
            lay.deltabox[par] = self.layout[f"deltabox{par}"]
            lay.ready[par] = self.layout[f"ready{par}"]
            lay.dready[par] = self.layout[f"dready{par}"]
        lay.hello, lay.done_ring = self.layout["hello"], self.layout["done_ring"]
        return lay

    def _prepare(self, *, group_id: bytes, my_index: int, device_infos, modes, peer_fractions, weight: float, alpha,
                 sender_timeout, reducer_timeout) -> Tuple[_Plan, _HrRound, List[int]]:
        """Part table, work list and the kernel parameter block of one round; also advances the round counter.

        The parameter block of a (layout, groupmates, timeouts) combination is built once and kept: a later round of
        the same combination only changes the epoch, the parity and the weights."""
        n = len(device_infos)
        sends = [m != AveragingMode.AUX for m in modes]
        plan = self._make_plan(n, my_index, peer_fractions, sends)
        bases = self.map_group(device_infos, my_index)
        key = (tuple(bases), sender_timeout, reducer_timeout)
        template = plan.rounds.get(key)
        if template is None:
            if plan.needed_outbox > self.cap_outbox or plan.needed_delta > self.cap_delta or plan.needed_avg > self.cap_avg:
                raise RuntimeError("the staging areas of the arenas are too small for this group layout")
            sender_timeout = min(sender_timeout if sender_timeout else 10.0, 20.0)
            reducer_timeout = max(min(reducer_timeout if reducer_timeout else 2 * sender_timeout, 40.0), 2 * sender_timeout)
            g = _HrRound()
            g.n_peers, g.n_parts, g.me, g.max_local_parts = n, plan.n_parts, my_index, plan.max_local_parts
            g.sender_timeout_ns, g.reducer_timeout_ns = int(sender_timeout * 1e9), int(reducer_timeout * 1e9)
            g.delta_stride = plan.delta_stride
            for r in range(n):
                g.sends[r] = int(sends[r])
                g.base[r] = bases[r]
            g.lay = self._layout_struct()
            g.parts, g.items, g.pub_list = plan.parts_dev.data_ptr(), plan.items_dev.data_ptr(), plan.pub_dev.data_ptr()
            g.n_send, g.n_reduce, g.n_apply = plan.n_send, plan.n_reduce, plan.n_apply
            for name in ("include", "apply_decision", "ban", "t_start", "status", "part_done", "dpart_done", "queue"):
                setattr(g, name, plan.scratch[name].data_ptr())
            g.status_out = self._status_out.data_ptr()
            g.code = self._code.data_ptr()
            g.uses_blockwise = int(any(c == 5 for c in self.codecs))
            if len(plan.rounds) > 8:
                plan.rounds.pop(next(iter(plan.rounds)))
            plan.rounds[key] = template = g
        g = _HrRound.from_buffer_copy(template)  # rounds may overlap (one being finished while the next is prepared)
        g.item_begin, g.item_end, g.queue_slot, g.final_stage = 0, plan.n_send + plan.n_reduce + plan.n_apply, 0, 1
        g.trace = self.trace.data_ptr() if self.trace is not None else None
        g.epoch = (zlib.crc32(group_id) & 0x7FFFFFFF) | 1
        g.parity = self._round_seq & 1
        g.done_slot = self._round_seq
        g.alpha, g.my_weight = alpha, float(weight)
        self._round_seq += 1
        return plan, g, bases

    def _gate_params(self, g: _HrRound, bases: List[int], sender_timeout_ns: int) -> _HrGate:
        gate = self._gate
        gate.n_peers, gate.me, gate.parity, gate.epoch = g.n_peers, g.me, g.parity, g.epoch
        prev_epoch, prev_bases = self._history.get(g.parity, (0, []))
        gate.prev_epoch, gate.n_prev = prev_epoch, len(prev_bases)
        for t, b in enumerate(prev_bases):
            gate.prev_base[t] = b
        for r in range(g.n_peers):
            gate.base[r] = bases[r]
        gate.ack_timeout_ns = min(int(g.reducer_timeout_ns), int(2e9))
        gate.hello_timeout_ns = sender_timeout_ns
        self._history[g.parity] = (g.epoch, [b for r, b in enumerate(bases) if r != g.me][:MAX_PEERS])
        return gate

    def _launch_round(self, g: _HrRound, begin: int, end: int, slot: int, final: bool, stream, name: str) -> None:
        g.item_begin, g.item_end, g.queue_slot, g.final_stage = begin, end, slot, int(final)
        if end <= begin and not final:
            return
        with torch.cuda.device(self.device):
            code = self.lib.hm_br_round(ctypes.byref(g), CTAS_PER_SM * self._sms, stream)
        _lib.check(code, f"hm_br_round({name})")
        if self.launch_hook is not None:
            self.launch_hook(name)  # benchmarks record an event after every launch of a round

    def _read_status(self, stream) -> RoundStatus:
        with torch.cuda.device(self.device):
            _lib.check(self.lib.hm_memcpy_d2h(self._host_status, ctypes.c_void_p(self._status_out.data_ptr()),
                                              ctypes.c_ulonglong(32), stream), "read status", 0)
        banned, failed, elements = self._host_status[0], self._host_status[1], self._host_status[2]
        return RoundStatus([i for i in range(MAX_PEERS) if banned >> i & 1], [i for i in range(MAX_PEERS) if failed >> i & 1],
                           int(elements), sum(self.numels))

    def run_round(self, *, group_id: bytes, my_index: int, device_infos, modes, peer_fractions, weight: float,
                  alpha: float, sender_timeout: Optional[float], reducer_timeout: Optional[float],
                  wait: bool = True) -> Optional[RoundStatus]:
        """Run one all-reduce round with the mapped groupmates. Blocks the calling thread until this GPU is done,
        unless ``wait`` is False: then the round is only enqueued on the endpoint's stream (several rounds may be
        queued back to back) and ``wait_round()`` returns the status of the last one."""
        # the caller's writes to the tensors must land before the round reads them: order the round's stream after the
        # caller's stream on the device (no host wait: that stream may hold work that depends on other ranks)
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(self.device))
        self._torch_stream.wait_event(ready)
        plan, g, bases = self._prepare(group_id=group_id, my_index=my_index, device_infos=device_infos, modes=modes,
                                       peer_fractions=peer_fractions, weight=weight, alpha=alpha,
                                       sender_timeout=sender_timeout, reducer_timeout=reducer_timeout)
        gate = self._gate_params(g, bases, int(g.sender_timeout_ns))
        total = plan.n_send + plan.n_reduce + plan.n_apply
        with device_range("butterfly.round", self._torch_stream):
            with torch.cuda.device(self.device):
                _lib.check(self.lib.hm_br_gate(ctypes.byref(gate), self.stream), "hm_br_gate")
            if self.launch_hook is not None:
                self.launch_hook("gate")
            if self.fault_publish_half:
                # injected on the host: this rank stalls after it has sent half of its parts
                self._launch_round(g, 0, plan.send_cut, 0, False, self.stream, "send(half)")
                self._launch_round(g, plan.n_send, total, 1, True, self.stream, "reduce+apply")
            else:
                self._launch_round(g, 0, total, 0, True, self.stream, "round")
        return self.wait_round() if wait else None

    def wait_round(self) -> RoundStatus:
        """Wait for the rounds enqueued so far and return the status words of the last one."""
        status = self._read_status(self.stream)
        self._last_round_end = time.monotonic()
        if DEBUG_CHECKS:
            self.check_canaries()
        return status


def run_group_emulated(endpoints: Sequence[DeviceEndpoint], *, weights: Sequence[float],
                       peer_fractions: Sequence[float], modes: Optional[Sequence[AveragingMode]] = None,
                       alpha: float = 1.0, group_id: bytes = b"emulated", sender_timeout: float = 1.0,
                       reducer_timeout: float = 2.0, skip_send_of: Sequence[int] = (),
                       publish_only_first_half_of: Sequence[int] = (), members: Optional[Sequence[int]] = None,
                       stop_after_stage: int = 3) -> List[RoundStatus]:
    """Run a whole group inside one process, stage by stage: first every rank's send items, then every rank's
    reduce items, then every rank's apply items, so that no launch ever waits for a later one. Used when there are
    fewer GPUs than ranks, and by tests that inject host-side faults: ``skip_send_of`` ranks never publish their
    parts (a sender that does not show up), ``publish_only_first_half_of`` ranks stall after half of their parts.
    ``stop_after_stage`` (1 or 2) leaves the round unfinished, e.g. to let a rank begin its next round with another
    group while a slow member of this one has not applied its results yet; ``finish_group_emulated`` completes it.
    """
    n = len(endpoints)
    modes = list(modes) if modes is not None else [AveragingMode.NODE] * n
    infos = [e.describe() for e in endpoints]
    streams = [ctypes.c_void_p(torch.cuda.current_stream(e.device).cuda_stream) for e in endpoints]
    prepared = [e._prepare(group_id=group_id, my_index=r, device_infos=infos, modes=modes, peer_fractions=peer_fractions,
                           weight=weights[r], alpha=alpha, sender_timeout=sender_timeout,
                           reducer_timeout=reducer_timeout) for r, e in enumerate(endpoints)]
    for r, e in enumerate(endpoints):
        plan, g, bases = prepared[r]
        e._history[g.parity] = (g.epoch, [b for q, b in enumerate(bases) if q != r])
        if r in skip_send_of:
            continue
        end = plan.send_cut if r in publish_only_first_half_of else plan.n_send
        e._launch_round(g, 0, end, 0, False, streams[r], "send")
    for e in endpoints:
        torch.cuda.synchronize(e.device)
    if stop_after_stage < 2:
        return prepared  # type: ignore[return-value]
    for r, e in enumerate(endpoints):
        plan, g, _ = prepared[r]
        e._launch_round(g, plan.n_send, plan.n_send + plan.n_reduce, 1, False, streams[r], "reduce")
    for e in endpoints:
        torch.cuda.synchronize(e.device)
    if stop_after_stage < 3:
        return prepared  # type: ignore[return-value]
    return finish_group_emulated(endpoints, prepared, only=members)


def finish_group_emulated(endpoints: Sequence[DeviceEndpoint], prepared, only: Optional[Sequence[int]] = None
                          ) -> List[RoundStatus]:
    """Run the apply stage of a round started by ``run_group_emulated(..., stop_after_stage=2)`` for the ranks in
    ``only`` (default: all) and return their status words."""
    ranks = list(range(len(endpoints))) if only is None else list(only)
    streams = {r: ctypes.c_void_p(torch.cuda.current_stream(endpoints[r].device).cuda_stream) for r in ranks}
    for r in ranks:
        plan, g, _ = prepared[r]
        begin = plan.n_send + plan.n_reduce
        endpoints[r]._launch_round(g, begin, begin + plan.n_apply, 2, True, streams[r], "apply")
    return [endpoints[r]._read_status(streams[r]) for r in ranks]

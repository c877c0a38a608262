"""``PowerSGDGradientAverager``: rank-r gradient compression with error feedback (https://arxiv.org/abs/1905.13727).

Algorithm as in the reference (hivemind/optim/power_sgd_averager.py:28-222): for every gradient that compresses
well when viewed as a matrix M (others are averaged as they are),
    m += g;  P = M Q;  all-reduce P;  orthogonalise P;  Q = M^T P;  all-reduce Q (and the uncompressed gradients);
    g^ = P Q^T;  m -= g^;  the averaged gradient is g^.
Two all-reduce phases share one matched group (group id + b"PHASE_P" / b"PHASE_Q").

B200 version: M, P, Q stay on the GPU; the three products run on the tcgen05 kernel in tf32 with fp32 accumulation
(``ops/powersgd.py``); all P (resp. all Q plus the uncompressed gradients) live in one peer-mappable arena each and
are averaged by the device butterfly; orthogonalisation is a batched CholeskyQR2 kernel. On CPU the same class runs
the reference math with PyTorch and averages through RPC.
"""
from __future__ import annotations

import asyncio
import contextlib
from enum import Enum
from typing import Any, Iterable, Optional, Sequence

import torch

from hivemind_b200.averaging.allreduce import AveragingMode
from hivemind_b200.averaging.group_info import GroupInfo
from hivemind_b200.averaging.load_balancing import load_balance_peers
from hivemind_b200.averaging.matchmaking import MatchmakingException
from hivemind_b200.compression import CompressionInfo, TensorRole
from hivemind_b200.dht import DHT
from hivemind_b200.ops import multi_tensor as mt
from hivemind_b200.ops import powersgd as ps_ops
from hivemind_b200.optim.grad_averager import GradientAverager
from hivemind_b200.utils import get_logger
from hivemind_b200.utils.asyncio import enter_asynchronously
from hivemind_b200.utils.profiling import traced
from hivemind_b200.utils.math import get_flatten_greedy_dims, orthogonalize_

GatheredData = Any
logger = get_logger(__name__)


class AllReducePhases(Enum):
    PHASE_P = 1
    PHASE_Q = 2


class PowerSGDGradientAverager(GradientAverager):
    """
    :param parameters: parameters whose gradients are averaged
    :param averager_rank: rank r of the approximation
    :param min_compression_ratio: compress a tensor only if ``1 - r (m + n) / (m n)`` is at least this much
    :param q_init: ``"uniform"`` (reference default, U[0, 1)) or ``"normal"`` initial Q
    other parameters: see ``GradientAverager``
    """

    def __init__(self, parameters: Iterable[torch.nn.Parameter], averager_rank: int, *, dht: DHT, prefix: str,
                 reuse_grad_buffers: bool = False, accumulate_grads_on: Optional[torch.device] = None,
                 client_mode: bool = None, warn: bool = True, min_compression_ratio: float = 0.5,
                 averaged_grads: Optional[Sequence[torch.Tensor]] = None, q_init: str = "uniform", **kwargs):
        self.rank = averager_rank
        self.parameters = tuple(parameters)
        grads = list(self._grads_from_parameters())
        self._uncompressed_gradients_indexes = set(
            i for i, grad in enumerate(grads)
            if grad.ndim <= 1 or (1 - self.rank * sum(get_flatten_greedy_dims(grad)) / grad.numel()) < min_compression_ratio)
        compressed = [g for i, g in enumerate(grads) if i not in self._uncompressed_gradients_indexes]
        dims = [get_flatten_greedy_dims(g) for g in compressed]
        # Matrices of one shape are kept in stacks ([count, rows, cols] error feedback and averaged gradients,
        # [count, rows, r] P, [count, cols, r] Q) so that each of the three products is ONE grouped launch per shape
        # instead of one launch per matrix. The internal order of the compressed tensors is therefore "by shape";
        # self._order[k] says which compressed gradient (in parameter order) is the k-th internally.
        by_shape = {}
        for i, (d, g) in enumerate(zip(dims, compressed)):
            by_shape.setdefault((d[0], d[1], g.device), []).append(i)
        self._order = [i for members in by_shape.values() for i in members]
        self._dims = [dims[i] for i in self._order]
        make_q = torch.rand if q_init == "uniform" else torch.randn
        self._stacks, self._ms, self._qs, self._ps, stacked_grads = [], [], [], [], {}
        for (rows, cols, device), members in by_shape.items():
            count, first = len(members), len(self._ms)
            m = torch.zeros(count, rows, cols, dtype=torch.float32, device=device)
            g = torch.zeros(count, rows, cols, dtype=torch.float32, device=device)
            q = make_q((count, cols, self.rank), device=device, dtype=torch.float32)
            p = torch.zeros(count, rows, self.rank, dtype=torch.float32, device=device)
            self._stacks.append(dict(first=first, count=count, rows=rows, cols=cols, m=m, g=g, p=p, q=q,
                                     fused=device.type == "cuda" and ps_ops.can_stack(rows, cols, self.rank)))
            for k, i in enumerate(members):
                self._ms.append(m[k].view(compressed[i].shape))
                self._qs.append(q[k])
                self._ps.append(p[k])
                stacked_grads[i] = g[k].view(compressed[i].shape)
        if averaged_grads is None or len(averaged_grads) == 0:
            it = iter(range(len(compressed)))
            averaged_grads = [torch.zeros_like(g, dtype=torch.float32) if i in self._uncompressed_gradients_indexes
                              else stacked_grads[next(it)] for i, g in enumerate(grads)]
        else:
            for stack in self._stacks:  # the caller's buffers are used as they are: no stacked launches for them
                stack["fused"] = False
        self._p_endpoint = self._q_endpoint = None
        kwargs["use_device_path"] = False  # this class drives its own arenas (one per phase)
        super().__init__(self.parameters, dht=dht, prefix=prefix, reuse_grad_buffers=reuse_grad_buffers,
                         accumulate_grads_on=accumulate_grads_on, client_mode=client_mode, warn=warn,
                         averaged_grads=averaged_grads, **kwargs)
        on_gpu = len(grads) > 0 and all(g.is_cuda for g in grads)
        if on_gpu and self._ps:
            self._setup_device_arenas()

    def _setup_device_arenas(self) -> None:
        from hivemind_b200.parallel.device_butterfly import DeviceEndpoint

        compression = self.allreduce_kwargs["compression"]
        part_size = self.allreduce_kwargs["part_size_bytes"]
        p_infos = [CompressionInfo.from_tensor(p, key=f"p_{i}", role=TensorRole.GRADIENT) for i, p in enumerate(self._ps)]
        self._p_endpoint = DeviceEndpoint(self._ps, compression, p_infos, part_size)
        self._ps = list(self._p_endpoint.tensor_views)
        with self.get_tensors() as averaged_grads:
            plain = [g for i, g in enumerate(averaged_grads) if i in self._uncompressed_gradients_indexes]
            q_tensors = list(self._qs) + plain
            q_infos = [CompressionInfo.from_tensor(t, key=f"q_{i}", role=TensorRole.GRADIENT) for i, t in enumerate(q_tensors)]
            self._q_endpoint = DeviceEndpoint(q_tensors, compression, q_infos, part_size)
            views = list(self._q_endpoint.tensor_views)
            self._qs = views[:len(self._qs)]
            # uncompressed averaged gradients now live inside the Q arena
            new_averaged, it = [], iter(views[len(self._qs):])
            for i, g in enumerate(averaged_grads):
                new_averaged.append(next(it) if i in self._uncompressed_gradients_indexes else g)
        self._averaged_tensors = tuple(new_averaged)
        # the stacks of P and Q are now runs of consecutive arena views
        for stack in self._stacks:
            first, count, rows, cols = stack["first"], stack["count"], stack["rows"], stack["cols"]
            for name, endpoint, width in (("p", self._p_endpoint, rows), ("q", self._q_endpoint, cols)):
                start, numel = endpoint.offsets[first], width * self.rank
                contiguous = all(endpoint.offsets[first + k] == start + k * numel for k in range(count))
                if contiguous:
                    stack[name] = endpoint.flat[start:start + count * numel].view(count, width, self.rank)
                else:
                    stack["fused"] = False
        if not (self._p_endpoint.supported and self._q_endpoint.supported):
            self._p_endpoint = self._q_endpoint = None

    def _describe_device(self) -> Optional[dict]:
        if self._p_endpoint is None:
            return None
        return dict(p=self._p_endpoint.describe(), q=self._q_endpoint.describe())

    @contextlib.contextmanager
    def _register_allreduce_group(self, group_info: GroupInfo):
        """One matched group serves two all-reduce rounds, addressed as group id + phase name."""
        try:
            for phase in list(AllReducePhases):
                self._running_groups[group_info.group_id + phase.name.encode()] = asyncio.Future()
            self._pending_groups_registered.set()
            yield
        finally:
            for phase in list(AllReducePhases):
                maybe_future = self._running_groups.pop(group_info.group_id + phase.name.encode(), None)
                if maybe_future and not maybe_future.done():
                    logger.warning(f"All-reduce group {group_info.group_id + phase.name.encode()} did not finish.")
            self._pending_groups_registered.set()

    async def _aggregate_with_group(self, group_info: GroupInfo, min_vector_size: int, **kwargs) -> GatheredData:
        try:
            unpacked = [self.serializer.loads(blob) for blob in group_info.gathered]
            bandwidths = [item[0] for item in unpacked]
            modes = tuple(AveragingMode(item[1]) for item in unpacked)
            user_gathered = dict(zip(group_info.peer_ids, (self.serializer.loads(item[2]) for item in unpacked)))
            device_infos = [item[3] if len(item) > 3 else None for item in unpacked]
            download_bandwidths = [thr if mode != AveragingMode.CLIENT else 0.0 for thr, mode in zip(bandwidths, modes)]
            p_size = sum(p.numel() for p in self._ps) or 1
            q_size = sum(q.numel() for q in self._qs) + sum(
                g.numel() for i, g in enumerate(self._averaged_tensors) if i in self._uncompressed_gradients_indexes) or 1
            loop = asyncio.get_event_loop()
            p_fractions = await loop.run_in_executor(None, load_balance_peers, p_size, download_bandwidths, min_vector_size)
            q_fractions = await loop.run_in_executor(None, load_balance_peers, q_size, download_bandwidths, min_vector_size)

            use_device = (self._p_endpoint is not None and all(isinstance(d, dict) and "p" in d for d in device_infos)
                          and self._p_endpoint.can_run_with([d["p"] for d in device_infos], modes)
                          and self._q_endpoint.can_run_with([d["q"] for d in device_infos], modes))
            p_group_id = group_info.group_id + AllReducePhases.PHASE_P.name.encode()
            q_group_id = group_info.group_id + AllReducePhases.PHASE_Q.name.encode()
            weight = kwargs.get("weight")

            async with enter_asynchronously(self.get_tensors()) as averaged_grads:
                compressed = [g for i, g in enumerate(averaged_grads) if i not in self._uncompressed_gradients_indexes]
                plain = [g for i, g in enumerate(averaged_grads) if i in self._uncompressed_gradients_indexes]
                await loop.run_in_executor(None, self._begin_round, compressed)
                if use_device:
                    await self._run_device_allreduce_(group_info, p_fractions, modes, [d["p"] for d in device_infos],
                                                      weight=weight, endpoint=self._p_endpoint, group_id=p_group_id,
                                                      lock=False,
                                                      sender_timeout=kwargs.get("sender_timeout"),
                                                      reducer_timeout=kwargs.get("reducer_timeout"))
                else:
                    await self._run_allreduce_inplace_(self._ps, group_info, p_group_id, peer_fractions=p_fractions,
                                                       modes=modes, **kwargs)
                await loop.run_in_executor(None, self._middle_round)
                if use_device:
                    await self._run_device_allreduce_(group_info, q_fractions, modes, [d["q"] for d in device_infos],
                                                      weight=weight, endpoint=self._q_endpoint, group_id=q_group_id,
                                                      lock=False,
                                                      sender_timeout=kwargs.get("sender_timeout"),
                                                      reducer_timeout=kwargs.get("reducer_timeout"))
                else:
                    await self._run_allreduce_inplace_(list(self._qs) + plain, group_info, q_group_id,
                                                       peer_fractions=q_fractions, modes=modes, **kwargs)
                await loop.run_in_executor(None, self._finish_round, compressed)
                return user_gathered
        except BaseException as e:
            if isinstance(e, Exception):
                logger.exception(e)
                raise MatchmakingException(f"Unable to run All-Reduce: {e!r}")
            raise

    # ---------------------------------------------------------------------------------------------- the three stages
    # All three run on the caller's stream without waiting on the host: the all-reduce rounds in between are ordered
    # after them by an event (DeviceEndpoint.run_round) and block their own thread until the round's stream is done.
    def _in_internal_order(self, compressed: Sequence[torch.Tensor]) -> list:
        return [compressed[i] for i in self._order]

    def _per_matrix(self, stack) -> range:
        return range(stack["first"], stack["first"] + stack["count"])

    @traced("powersgd.compress_p")
    @torch.no_grad()
    def _begin_round(self, compressed: Sequence[torch.Tensor]) -> None:
        """m += g;  P = M Q."""
        if not self._ms:
            return
        grads = self._in_internal_order(compressed)
        if all(m.device == g.device for m, g in zip(self._ms, grads)):
            mt.axpy_(self._ms, grads, 1.0)
        else:
            for m, g in zip(self._ms, grads):
                m.add_(g.to(m.device))
        for stack in self._stacks:
            if stack["fused"]:
                ps_ops.compute_p_stacked_(stack["p"], stack["m"], stack["q"])
            else:
                for k in self._per_matrix(stack):
                    ps_ops.compute_p_(self._ps[k], self._ms[k].view(*self._dims[k]), self._qs[k])

    @traced("powersgd.orthogonalize_q")
    @torch.no_grad()
    def _middle_round(self) -> None:
        """orthogonalise P;  Q = M^T P."""
        if not self._ps:
            return
        if self._ps[0].is_cuda and self.rank <= 64:
            ps_ops.orthogonalize_batch_(self._ps)
        else:
            for p in self._ps:
                orthogonalize_(p)
        for stack in self._stacks:
            if stack["fused"]:
                ps_ops.compute_q_stacked_(stack["q"], stack["m"], stack["p"])
            else:
                for k in self._per_matrix(stack):
                    ps_ops.compute_q_(self._qs[k], self._ms[k].view(*self._dims[k]), self._ps[k])

    @traced("powersgd.reconstruct")
    @torch.no_grad()
    def _finish_round(self, compressed: Sequence[torch.Tensor]) -> None:
        """g^ = P Q^T;  m -= g^;  averaged gradient = g^."""
        if not self._ps:
            return
        grads = self._in_internal_order(compressed)
        for stack in self._stacks:
            if stack["fused"]:
                ps_ops.reconstruct_stacked_(stack["g"], stack["p"], stack["q"])
            else:
                for k in self._per_matrix(stack):
                    ps_ops.reconstruct_(grads[k].view(*self._dims[k]), self._ps[k], self._qs[k])
        if all(m.device == g.device for m, g in zip(self._ms, grads)):
            mt.axpy_(self._ms, grads, -1.0)
        else:
            for m, g in zip(self._ms, grads):
                m.sub_(g.to(m.device))

    # ---------------------------------------------------------------------------------------------- state sharing
    def get_current_state(self):
        """Peers that join later need the Q factors (the error-feedback buffers stay local)."""
        with torch.no_grad(), self.lock_averaged_tensors:
            buffers = [q.detach().cpu().clone() for q in self._qs]
            infos = [CompressionInfo.from_tensor(buffer, key=f"buffer_q_{i}", role=TensorRole.GRADIENT)
                     for i, buffer in enumerate(buffers)]
        return dict(group_bits=self.get_group_bits()), buffers, infos

    def load_state_from_peers(self, **kwargs):
        loaded_state = super().load_state_from_peers(**kwargs)
        if loaded_state is None:
            return
        metadata, flat_tensors = loaded_state
        logger.info("Starting loading gradient averager buffers from peers")
        if len(flat_tensors) != len(self._qs):
            logger.error("Failed to load state from peer, received invalid parameters, extras or metadata")
            return
        with torch.no_grad(), self.lock_averaged_tensors:
            for local_q, loaded_q in zip(self._qs, flat_tensors):
                local_q.copy_(loaded_q.to(local_q.device), non_blocking=True)

    def shutdown(self) -> None:
        super().shutdown()
        for endpoint in (self._p_endpoint, self._q_endpoint):
            if endpoint is not None:
                endpoint.close()

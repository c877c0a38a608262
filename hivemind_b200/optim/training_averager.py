"""``TrainingAverager`` (legacy interface): average an existing optimizer's parameters, gradients and/or statistics.

Kept for users of the older API (hivemind/optim/training_averager.py:18-252); new code should use
``hivemind_b200.Optimizer``. One ``step()`` copies the local tensors into the averager, averages them with a group and
writes the result back; if the model kept training in the meantime (``data_lock`` given), only the change produced by
averaging is added to the local tensors. Copies are fused multi-tensor kernels when everything is on one GPU.
"""
from __future__ import annotations

from concurrent.futures import ThreadPoolExecutor
from contextlib import nullcontext
from threading import Event, Lock
from typing import Iterator, List, Optional, Sequence, Tuple

import torch

from hivemind_b200.averaging import DecentralizedAverager
from hivemind_b200.compression import CompressionInfo, TensorRole
from hivemind_b200.ops import multi_tensor as mt
from hivemind_b200.optim.state_averager import (_bulk_copy, dump_optimizer_state, initialize_optimizer_state_,
                                                load_optimizer_state)
from hivemind_b200.utils import get_logger

logger = get_logger(__name__)


class TrainingAverager(DecentralizedAverager):
    """
    :param opt: the optimizer whose tensors are averaged
    :param average_parameters / average_gradients: what to average in ``step``
    :param average_opt_statistics: names of optimizer statistics to average as well
    :param extra_tensors: further tensors to average and to ship in state downloads
    :param initialize_optimizer: run one zero-gradient step so that statistics exist
    """

    def __init__(self, opt: torch.optim.Optimizer, *, average_parameters: bool, average_gradients: bool,
                 average_opt_statistics: Sequence[str] = (), extra_tensors: Sequence[torch.Tensor] = (),
                 parameter_names: Optional[Sequence[str]] = None, initialize_optimizer: bool = True, **kwargs):
        if initialize_optimizer:
            initialize_optimizer_state_(opt)
        self.opt = opt
        self.average_parameters, self.average_gradients = average_parameters, average_gradients
        self.opt_statistics = tuple(average_opt_statistics)
        self.extra_tensors = tuple(extra_tensors)
        self.parameter_names = tuple(parameter_names) if parameter_names is not None else tuple(range(len(self._params())))
        assert len(self.parameter_names) == len(self._params()), "one name per optimized parameter"
        self.local_step = 0
        self.step_executor = ThreadPoolExecutor(max_workers=1)
        self.lock_averager_step = Lock()
        self.pending_updates_done = Event()  # clear while local tensors are being read or written by a step
        self.pending_updates_done.set()
        sections = list(self._sections())
        with torch.no_grad():
            shadows = [tensor.detach().float().clone() for _, _, tensor in sections]
        infos = [CompressionInfo.from_tensor(tensor, key=key, role=role) for role, key, tensor in sections]
        super().__init__(averaged_tensors=shadows, tensor_infos=infos, **kwargs)

    # ------------------------------------------------------------------------------------------ what is averaged
    def _params(self) -> List[torch.Tensor]:
        return [p for group in self.opt.param_groups for p in group["params"]]

    def _sections(self, replace_none: bool = True) -> Iterator[Tuple[TensorRole, object, torch.Tensor]]:
        """(role, key, tensor) of everything that takes part in a round, in averaging order: parameters, gradients,
        the chosen optimizer statistics, extras. A parameter without a gradient contributes zeros."""
        named = list(zip(self.parameter_names, self._params()))
        if self.average_parameters:
            for name, p in named:
                yield TensorRole.PARAMETER, name, p
        if self.average_gradients:
            for name, p in named:
                if p.grad is not None:
                    yield TensorRole.GRADIENT, name, p.grad
                elif replace_none:
                    yield TensorRole.GRADIENT, name, torch.zeros_like(p)
        for statistic in self.opt_statistics:
            for name, p in named:
                yield TensorRole.OPTIMIZER, (name, statistic), self.opt.state[p][statistic]
        for index, extra in enumerate(self.extra_tensors):
            yield TensorRole.UNSPECIFIED, index, extra

    def local_tensors(self, replace_none: bool = True) -> Iterator[torch.Tensor]:
        """Local tensors in averaging order: parameters, gradients, optimizer statistics, extras."""
        return (tensor for _, _, tensor in self._sections(replace_none))

    def tensor_infos(self) -> Iterator[CompressionInfo]:
        return (CompressionInfo.from_tensor(tensor, key=key, role=role) for role, key, tensor in self._sections())

    # ------------------------------------------------------------------------------------------ one round
    def step(self, data_lock: Optional[Lock] = None, wait: bool = True, **kwargs):
        """Average with peers; ``data_lock`` is held only while local tensors are read or written."""
        if not wait:
            return self.step_executor.submit(self.step, data_lock, wait=True, **kwargs)
        concurrent_training = data_lock is not None  # the model may change between the two copies
        guard = data_lock if concurrent_training else nullcontext()
        local = list(self.local_tensors())
        with self.lock_averager_step, torch.no_grad():
            snapshot = self._copy_in(local, guard, keep_snapshot=concurrent_training)
            gathered = super().step(**kwargs)
            if gathered is not None:
                self._copy_out(local, guard, snapshot)
            self.local_step += 1
            return gathered

    def _copy_in(self, local: List[torch.Tensor], guard, keep_snapshot: bool) -> Optional[List[torch.Tensor]]:
        self.pending_updates_done.clear()
        try:
            with guard, self.get_tensors() as shadows:
                if len(shadows) != len(local):
                    raise RuntimeError("the set of optimized tensors changed since the averager was created")
                snapshot = [t.detach().float().clone() for t in local] if keep_snapshot else None
                _bulk_copy(list(shadows), local)
            return snapshot
        finally:
            self.pending_updates_done.set()

    def _copy_out(self, local: List[torch.Tensor], guard, snapshot: Optional[List[torch.Tensor]]) -> None:
        self.pending_updates_done.clear()
        try:
            with guard, self.get_tensors() as shadows:
                shadows = list(shadows)
                if len(shadows) != len(local):
                    raise RuntimeError("the set of optimized tensors changed since the averager was created")
                if snapshot is None:
                    _bulk_copy(local, shadows)
                elif all(l.device == a.device and l.dtype == torch.float32 for l, a in zip(local, shadows)):
                    mt.delta_update_(local, shadows, snapshot)  # local += averaged - what went into the round
                else:
                    for mine, averaged, before in zip(local, shadows, snapshot):
                        mine.add_((averaged - before).to(mine.device, mine.dtype))
        finally:
            self.pending_updates_done.set()

    # ------------------------------------------------------------------------------------------ state transfer
    def get_current_state(self):
        """(metadata, tensors, infos): parameters, extras, then optimizer tensors (same layout as the state averager)."""
        with torch.no_grad():
            tensors, infos = [], []
            for name, p in zip(self.parameter_names, self._params()):
                tensors.append(p.detach().cpu())
                infos.append(CompressionInfo.from_tensor(tensors[-1], key=name, role=TensorRole.PARAMETER))
            for index, extra in enumerate(self.extra_tensors):
                tensors.append(extra.detach().cpu())
                infos.append(CompressionInfo.from_tensor(tensors[-1], key=index, role=TensorRole.UNSPECIFIED))
            optimizer_metadata, optimizer_tensors = dump_optimizer_state(self.opt)
            for index, t in enumerate(optimizer_tensors):
                tensors.append(t)
                infos.append(CompressionInfo.from_tensor(t, key=index, role=TensorRole.OPTIMIZER))
        metadata = dict(step=self.local_step, group_bits=self.get_group_bits(), optimizer_metadata=optimizer_metadata)
        return metadata, tensors, infos

    def load_state_from_peers(self, **kwargs):
        targets = self._params() + list(self.extra_tensors)
        loaded = super().load_state_from_peers(**kwargs)
        if loaded is None:
            return
        metadata, flat = loaded
        with torch.no_grad():
            for mine, theirs in zip(targets, flat[:len(targets)]):
                mine.copy_(theirs.to(mine.device, mine.dtype))
            load_optimizer_state(self.opt, metadata["optimizer_metadata"], flat[len(targets):])
        self.local_step = max(self.local_step, metadata["step"])


def initialize_optimizer_state(opt: torch.optim.Optimizer) -> None:
    """Make ``opt`` allocate its statistics by taking one step with zero gradients
    (reference: hivemind/optim/training_averager.py:220-225)."""
    initialize_optimizer_state_(opt)

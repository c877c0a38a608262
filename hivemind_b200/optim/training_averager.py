"""``TrainingAverager`` (legacy interface): average an existing optimizer's parameters, gradients and/or statistics.

Kept for users of the older API (hivemind/optim/training_averager.py:18-252); new code should use
``hivemind_b200.Optimizer``. One ``step()`` copies the local tensors into the averager, averages them with a group and
writes the result back; if the model kept training in the meantime (``data_lock`` given), only the change produced by
averaging is added to the local tensors. Copies are fused multi-tensor kernels when everything is on one GPU.
"""
from __future__ import annotations

from concurrent.futures import ThreadPoolExecutor
from contextlib import nullcontext
from itertools import chain
from threading import Event, Lock
from typing import Iterator, Optional, Sequence

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
        if parameter_names is None:
            parameter_names = tuple(i for group in opt.param_groups for i in range(len(group["params"])))
        self.opt, self.extra_tensors, self.local_step = opt, tuple(extra_tensors), 0
        self.opt_statistics = tuple(average_opt_statistics)
        self.average_parameters, self.average_gradients = average_parameters, average_gradients
        self.parameter_names = parameter_names
        self.step_executor = ThreadPoolExecutor(max_workers=1)
        self.lock_averager_step = Lock()
        self.pending_updates_done = Event()
        self.pending_updates_done.set()
        with torch.no_grad():
            averaged_tensors = [tensor.detach().float().clone() for tensor in self.local_tensors()]
        super().__init__(averaged_tensors=averaged_tensors, tensor_infos=list(self.tensor_infos()), **kwargs)

    def step(self, data_lock: Optional[Lock] = None, wait: bool = True, **kwargs):
        """Average with peers; ``data_lock`` is held only while local tensors are read or written."""
        if not wait:
            return self.step_executor.submit(self.step, data_lock, wait=True, **kwargs)
        use_old_local_tensors = data_lock is not None
        data_lock = data_lock if data_lock is not None else nullcontext()
        local_tensors = list(self.local_tensors())
        with self.lock_averager_step, torch.no_grad():
            self.pending_updates_done.clear()
            with data_lock, self.get_tensors() as averaged_tensors:
                assert len(local_tensors) == len(averaged_tensors), "The number of optimized parameters should not change."
                if use_old_local_tensors:
                    old_local_tensors = tuple(x.detach().float().clone() for x in local_tensors)
                _bulk_copy(list(averaged_tensors), local_tensors)
            self.pending_updates_done.set()
            gathered = super().step(**kwargs)
            if gathered is not None:
                self.pending_updates_done.clear()
                with data_lock, self.get_tensors() as averaged_tensors:
                    if len(averaged_tensors) != len(local_tensors):
                        raise RuntimeError("The number of optimized parameters should not change.")
                    if use_old_local_tensors:
                        # the model moved on while we averaged: add only what averaging changed
                        same = all(l.device == a.device and l.dtype == torch.float32 for l, a in zip(local_tensors, averaged_tensors))
                        if same:
                            mt.delta_update_(local_tensors, list(averaged_tensors), list(old_local_tensors))
                        else:
                            for local, new, old in zip(local_tensors, averaged_tensors, old_local_tensors):
                                local.add_((new - old).to(local.device, local.dtype))
                    else:
                        _bulk_copy(local_tensors, list(averaged_tensors))
                self.pending_updates_done.set()
            self.local_step += 1
            return gathered

    def local_tensors(self, replace_none: bool = True) -> Iterator[torch.Tensor]:
        """Local tensors in averaging order: parameters, gradients, optimizer statistics, extras."""
        if self.average_parameters:
            for group in self.opt.param_groups:
                yield from group["params"]
        if self.average_gradients:
            for group in self.opt.param_groups:
                for param in group["params"]:
                    if param.grad is not None:
                        yield param.grad
                    elif replace_none:
                        yield torch.zeros_like(param)
        for stats in self.opt_statistics:
            for group in self.opt.param_groups:
                for param in group["params"]:
                    yield self.opt.state[param][stats]
        yield from iter(self.extra_tensors)

    def tensor_infos(self):
        params = tuple(param for group in self.opt.param_groups for param in group["params"])
        assert len(params) == len(self.parameter_names)
        if self.average_parameters:
            for param, key in zip(params, self.parameter_names):
                yield CompressionInfo.from_tensor(param, key=key, role=TensorRole.PARAMETER)
        if self.average_gradients:
            for param, key in zip(params, self.parameter_names):
                if param.grad is not None:
                    grad = param.grad if param.grad is not None else torch.zeros_like(param)
                    yield CompressionInfo.from_tensor(grad, key=key, role=TensorRole.GRADIENT)
        for stats in self.opt_statistics:
            for param, key in zip(params, self.parameter_names):
                yield CompressionInfo.from_tensor(self.opt.state[param][stats], key=(key, stats), role=TensorRole.OPTIMIZER)
        for i, extra_tensor in enumerate(self.extra_tensors):
            yield CompressionInfo.from_tensor(extra_tensor, key=i, role=TensorRole.UNSPECIFIED)

    def get_current_state(self):
        """(metadata, tensors, infos): parameters, extras, then optimizer tensors (same layout as the state averager)."""
        with torch.no_grad():
            optimized_parameters = tuple(param.detach().cpu() for group in self.opt.param_groups for param in group["params"])
            parameter_infos = [CompressionInfo.from_tensor(param, key=key, role=TensorRole.PARAMETER)
                               for param, key in zip(optimized_parameters, self.parameter_names)]
            extra_tensors = tuple(tensor.detach().cpu() for tensor in self.extra_tensors)
            extra_infos = [CompressionInfo.from_tensor(t, key=i, role=TensorRole.UNSPECIFIED) for i, t in enumerate(extra_tensors)]
            optimizer_metadata, optimizer_tensors = dump_optimizer_state(self.opt)
            optimizer_infos = [CompressionInfo.from_tensor(t, key=i, role=TensorRole.OPTIMIZER) for i, t in enumerate(optimizer_tensors)]
        metadata = dict(step=self.local_step, group_bits=self.get_group_bits(), optimizer_metadata=optimizer_metadata)
        return metadata, list(chain(optimized_parameters, extra_tensors, optimizer_tensors)), \
            list(chain(parameter_infos, extra_infos, optimizer_infos))

    def load_state_from_peers(self, **kwargs):
        parameters_and_extras = [param for group in self.opt.param_groups for param in group["params"]]
        parameters_and_extras.extend(self.extra_tensors)
        num_local = len(parameters_and_extras)
        loaded_state = super().load_state_from_peers(**kwargs)
        if loaded_state is None:
            return
        metadata, flat_tensors = loaded_state
        loaded_parameters_and_extras, loaded_opt_tensors = flat_tensors[:num_local], flat_tensors[num_local:]
        with torch.no_grad():
            for local_param, loaded_param in zip(parameters_and_extras, loaded_parameters_and_extras):
                local_param[...] = loaded_param.to(local_param.device, local_param.dtype)
            load_optimizer_state(self.opt, metadata["optimizer_metadata"], loaded_opt_tensors)
        self.local_step = max(self.local_step, metadata["step"])


def initialize_optimizer_state(opt: torch.optim.Optimizer) -> None:
    """Make ``opt`` allocate its statistics by taking one step with zero gradients
    (reference: hivemind/optim/training_averager.py:220-225)."""
    initialize_optimizer_state_(opt)

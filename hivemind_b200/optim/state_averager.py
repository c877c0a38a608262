"""``TrainingStateAverager``: owns the optimizer, the LR schedule and the averaged copy of the training state.

State = parameters (+ selected optimizer statistics + extra tensors). The same state machine as the reference
(hivemind/optim/state_averager.py:37-740): one ``step(...)`` call can run, in order and each optionally in the
background, an optimizer step, ``zero_grad``, a scheduler step and an averaging round; results of background work
are applied by a later call with ``apply_delayed_updates=True``.

B200 design notes: averaged copies stay on the parameters' device (for CUDA in the averager's peer-mappable arena),
so "offloading" means "the optimizer updates the fp32 arena copy while the model keeps training on its own
tensors" instead of a round trip through host memory; copies between the model and the arena and the delta rule
are single multi-tensor kernels.
"""
from __future__ import annotations

import logging
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from contextlib import nullcontext
from itertools import chain
from typing import Any, Callable, Dict, Iterable, Iterator, Optional, Sequence, Tuple, Union

import torch

from hivemind_b200.averaging import DecentralizedAverager, StepControl
from hivemind_b200.compression import CompressionInfo, TensorRole
from hivemind_b200.dht import DHT
from hivemind_b200.ops import multi_tensor as mt
from hivemind_b200.utils import DHTExpiration, PerformanceEMA, get_dht_time, get_logger, nested_flatten, nested_pack

logger = get_logger(__name__)

Parameters = Iterable[torch.Tensor]
ParamGroups = Iterable[Dict[str, Any]]
TorchOptimizer = torch.optim.Optimizer
try:
    LRSchedulerBase = torch.optim.lr_scheduler.LRScheduler
except AttributeError:  # pragma: no cover
    LRSchedulerBase = torch.optim.lr_scheduler._LRScheduler
OptimizerFactory = Callable[[Union[Parameters, ParamGroups]], TorchOptimizer]
SchedulerFactory = Callable[[TorchOptimizer], LRSchedulerBase]


def _copy_all_(dst: Sequence[torch.Tensor], src: Sequence[torch.Tensor]) -> None:
    """dst[i] <- src[i]; one kernel when all pairs share a device, plain copies otherwise."""
    pairs = [(d, s) for d, s in zip(dst, src) if d.data_ptr() != s.data_ptr() or d.device != s.device]
    if not pairs:
        return
    if all(d.device == s.device and d.is_contiguous() and s.is_contiguous() and d.is_floating_point()
           and s.is_floating_point() for d, s in pairs):
        mt.scale_copy_([d for d, _ in pairs], [s for _, s in pairs], 1.0)
    else:
        for d, s in pairs:
            d.copy_(s, non_blocking=True)


class TrainingStateAverager(DecentralizedAverager):
    """
    :param optimizer: a ``torch.optim.Optimizer`` or a factory ``params -> optimizer`` (required for offloading)
    :param params: parameters or param groups (default: the optimizer's groups)
    :param scheduler: an LR scheduler or a factory ``optimizer -> scheduler``
    :param initialize_optimizer: run one zero-gradient step so that optimizer statistics exist (default: if needed)
    :param offload_optimizer: the optimizer updates the averaged copies instead of the model's own tensors
    :param custom_gradients: with offloading, the caller writes gradients into the optimizer's tensors itself
    :param reuse_tensors: average the optimizer's tensors in place instead of keeping separate averaged copies
    :param delta_rule_averaging: apply ``local += averaged_new - averaged_old`` so that local progress made while
      averaging ran in the background is kept
    :param sync_epoch_when_averaging: adopt the highest epoch seen among groupmates
    :param parameter_names: names for codecs that choose per tensor
    :param average_opt_statistics: names of optimizer statistics to average (e.g. ``("exp_avg_sq",)``)
    :param extra_tensors: further tensors to average (e.g. batch-norm statistics)
    :param kwargs: forwarded to ``DecentralizedAverager``
    """

    def __init__(self, *, dht: DHT, optimizer: Union[TorchOptimizer, OptimizerFactory],
                 params: Optional[Union[Parameters, ParamGroups]] = None,
                 scheduler: Optional[Union[LRSchedulerBase, SchedulerFactory]] = None,
                 initialize_optimizer: Optional[bool] = None, offload_optimizer: bool = False,
                 custom_gradients: bool = False, reuse_tensors: Optional[bool] = None,
                 delta_rule_averaging: bool = False, performance_ema_alpha: float = 0.1,
                 sync_epoch_when_averaging: bool = False, parameter_names: Optional[Sequence[str]] = None,
                 average_opt_statistics: Sequence[str] = (), extra_tensors: Sequence[torch.Tensor] = (),
                 status_loglevel: int = logging.DEBUG, **kwargs):
        average_opt_statistics = tuple(average_opt_statistics)
        assert all(isinstance(key, str) for key in average_opt_statistics)
        if reuse_tensors is None:
            reuse_tensors = offload_optimizer and not delta_rule_averaging
        if custom_gradients and not offload_optimizer:
            logger.warning("Setting custom_gradients=True has no effect because the optimizer is not offloaded")
        if reuse_tensors and delta_rule_averaging:
            raise ValueError("reuse_tensors and delta_rule_averaging are mutually exclusive")
        param_groups, main_parameters, parameter_names = self._check_params(optimizer, params, parameter_names)
        self.status_loglevel = status_loglevel
        self.offload_optimizer, self.custom_gradients = offload_optimizer, custom_gradients
        self.reuse_tensors, self.delta_rule_averaging = reuse_tensors, delta_rule_averaging
        self._old_tensors: Optional[Sequence[torch.Tensor]] = None
        self.main_parameters, self.parameter_names = main_parameters, parameter_names
        self._averaged_parameters = self._make_averaged_parameters(main_parameters)
        self.optimizer, self.scheduler = self._init_components(param_groups, optimizer, scheduler, initialize_optimizer)
        self.opt_keys_for_averaging, self.extra_tensors = average_opt_statistics, extra_tensors
        self.sync_epoch_when_averaging = sync_epoch_when_averaging
        self.local_epoch = 0
        self.delay_before_averaging = PerformanceEMA(alpha=performance_ema_alpha)
        self.step_executor = ThreadPoolExecutor(max_workers=2 if self.delta_rule_averaging else 1)
        self.finished_optimizer_step = threading.Event()
        self.finished_averaging_round = threading.Event()
        self.lock_optimizer = threading.Lock()
        self.lock_averaging = threading.Lock()
        self.pending_updates = set()
        # the device data path re-homes averaged tensors into an arena, which would break tensor sharing
        if reuse_tensors:
            kwargs.setdefault("use_device_path", False)
        super().__init__(dht=dht, averaged_tensors=self._init_averaged_tensors(), tensor_infos=self._init_tensor_infos(),
                         **kwargs)

    @staticmethod
    def _check_params(optimizer, param_groups, parameter_names):
        if param_groups is None:
            assert hasattr(optimizer, "param_groups"), "Must provide param_groups or an optimizer with .param_groups"
            param_groups = optimizer.param_groups
        param_groups = tuple(param_groups)
        if all(isinstance(p, torch.Tensor) for p in param_groups):
            param_groups = (dict(params=param_groups),)
        for group in param_groups:
            assert isinstance(group, dict) and group.get("params") is not None
            assert all(isinstance(p, torch.Tensor) for p in group["params"])
        parameters = tuple(chain(*(group["params"] for group in param_groups)))
        if parameter_names is None:
            parameter_names = tuple(i for i in range(len(parameters)))
        parameter_names = tuple(nested_flatten(parameter_names))
        assert len(parameters) == len(parameter_names), f"Expected {len(parameters)} names, got {len(parameter_names)}"
        assert len(set(parameters)) == len(parameters), "Found duplicate parameters in param_groups"
        with_grad = sum(p.numel() for p in parameters if p.requires_grad)
        without_grad = sum(p.numel() for p in parameters if not p.requires_grad)
        if without_grad >= with_grad:
            logger.warning("Most parameters have requires_grad=False but are still synchronized with peers; "
                           "leave frozen parameters out of the optimizer to save communication")
        return param_groups, parameters, parameter_names

    def _make_averaged_parameters(self, main_parameters: Sequence[torch.Tensor]):
        return tuple(self._make_averaged_tensor(param, force_copy=self.offload_optimizer) for param in main_parameters)

    def _make_averaged_tensor(self, source_tensor: torch.Tensor, force_copy: bool = False) -> torch.Tensor:
        """A new fp32 tensor on the same device for averaging, or the source itself when tensors are reused."""
        if self.reuse_tensors and not force_copy:
            return source_tensor
        averaged = source_tensor.detach().to(dtype=torch.float32, copy=True)
        return averaged.requires_grad_(source_tensor.requires_grad)

    def _init_components(self, param_groups, optimizer_or_factory, scheduler_or_factory, initialize_optimizer):
        assert hasattr(self, "_averaged_parameters"), "Internal error: must initialize averaged parameters first"
        optimizer_is_factory = callable(optimizer_or_factory) and not isinstance(optimizer_or_factory, TorchOptimizer)
        scheduler_is_factory = callable(scheduler_or_factory) and not isinstance(scheduler_or_factory, LRSchedulerBase)
        if optimizer_is_factory and not scheduler_is_factory and scheduler_or_factory is not None:
            raise ValueError("If optimizer is created internally, scheduler must also be initialized internally")
        if self.offload_optimizer and not optimizer_is_factory:
            raise ValueError("Using offload_optimizer requires creating optimizer inside hivemind")
        if optimizer_is_factory:
            if self.offload_optimizer:
                if self.reuse_tensors:
                    parameters_for_optimizer = self._averaged_parameters
                else:
                    parameters_for_optimizer = tuple(t.detach().clone().requires_grad_(t.requires_grad)
                                                     for t in self._averaged_parameters)
                next_index, groups_for_optimizer = 0, []
                for group in param_groups:
                    count = len(group["params"])
                    groups_for_optimizer.append(dict(group, params=parameters_for_optimizer[next_index:next_index + count]))
                    next_index += count
                assert next_index == len(parameters_for_optimizer)
                for param in parameters_for_optimizer:
                    if param.grad is None:
                        param.grad = torch.zeros_like(param)
            else:
                groups_for_optimizer = param_groups
            optimizer = optimizer_or_factory(groups_for_optimizer)
        else:
            optimizer = optimizer_or_factory
        if initialize_optimizer is None:
            initialize_optimizer = not any(isinstance(x, torch.Tensor) for x in nested_flatten(optimizer.state_dict()))
            logger.log(self.status_loglevel, "Initializing optimizer manually since it has no tensors in state dict. "
                                             "To override this, provide initialize_optimizer=False")
        if initialize_optimizer:
            initialize_optimizer_state_(optimizer)  # note: runs one optimizer step with zero gradients
        scheduler = scheduler_or_factory(optimizer) if scheduler_is_factory else scheduler_or_factory
        assert isinstance(optimizer, TorchOptimizer) and len(optimizer.param_groups) == len(list(param_groups))
        assert isinstance(scheduler, (LRSchedulerBase, type(None)))
        if scheduler is not None:
            assert scheduler.optimizer == optimizer
        return optimizer, scheduler

    def _local_tensors(self) -> Iterator[torch.Tensor]:
        """The trainer's own tensors that correspond, one to one, to the averaged tensors."""
        for group in self.optimizer.param_groups:
            yield from group["params"]
        for stats in self.opt_keys_for_averaging:
            for group in self.optimizer.param_groups:
                for param in group["params"]:
                    yield self.optimizer.state[param][stats]
        yield from self.extra_tensors

    @torch.no_grad()
    def _init_averaged_tensors(self) -> Sequence[torch.Tensor]:
        assert hasattr(self, "optimizer") and hasattr(self, "_averaged_parameters")
        local_tensors = tuple(self._local_tensors())
        local_non_parameters = local_tensors[len(self._averaged_parameters):]
        averaged = tuple(map(torch.Tensor.detach, self._averaged_parameters))
        averaged += tuple(map(self._make_averaged_tensor, local_non_parameters))
        assert len(averaged) == len(local_tensors)
        for local_tensor, averaged_tensor in zip(local_tensors, averaged):
            assert local_tensor.shape == averaged_tensor.shape
        return averaged

    def _init_tensor_infos(self) -> Sequence[CompressionInfo]:
        infos = [CompressionInfo.from_tensor(param, key=name, role=TensorRole.PARAMETER)
                 for param, name in zip(self.main_parameters, self.parameter_names)]
        for stats_name in self.opt_keys_for_averaging:
            opt_parameters = [param for group in self.optimizer.param_groups for param in group["params"]]
            assert len(opt_parameters) == len(self.parameter_names)
            for param, name in zip(opt_parameters, self.parameter_names):
                infos.append(CompressionInfo.from_tensor(self.optimizer.state[param][stats_name], key=(name, stats_name),
                                                         role=TensorRole.OPTIMIZER))
        for i, extra_tensor in enumerate(self.extra_tensors):
            infos.append(CompressionInfo.from_tensor(extra_tensor, key=i, role=TensorRole.UNSPECIFIED))
        return tuple(infos)

    def schedule_step(self, scheduled_time: Optional[DHTExpiration] = None, **kwargs) -> StepControl:
        """Begin matchmaking for a state-averaging round ahead of time (see ``step(averaging_control=...)``)."""
        assert kwargs.get("weight") is None, "setting weight in schedule_step is not supported"
        return super().step(scheduled_time=scheduled_time, wait=False, require_trigger=True, **kwargs)

    def step(self, wait_for_delayed_updates: bool = None, apply_delayed_updates: bool = True,
             increment_epoch: bool = False, optimizer_step: bool = False, zero_grad: bool = False,
             delay_optimizer_step: bool = False, averaging_round: bool = False, delay_averaging: Optional[bool] = None,
             averaging_control: Optional[StepControl] = None, wait_for_trigger: Optional[Callable[[], Any]] = None,
             grad_scaler=None, averaging_opts: Optional[Dict[str, Any]] = None, set_to_none: bool = False):
        """Run any combination of: apply finished background results, optimizer step, zero_grad, averaging round.

        :param wait_for_delayed_updates: wait for background work started by earlier calls
        :param apply_delayed_updates: copy finished background results into the model
        :param increment_epoch: ``local_epoch += 1`` (also steps the scheduler)
        :param optimizer_step / zero_grad: run these on the (possibly offloaded) optimizer
        :param delay_optimizer_step: run them in the background (needs ``offload_optimizer``)
        :param averaging_round: average state with peers; ``delay_averaging`` runs it in the background
        :param averaging_control: a pre-scheduled round from ``schedule_step``
        :param wait_for_trigger: callable awaited in the background before anything is modified
        :param grad_scaler: ``hivemind_b200.optim.GradScaler`` when training with loss scaling
        :param averaging_opts: extra arguments for the averaging step (``timeout``, ...)
        """
        if delay_averaging is None:
            delay_averaging = delay_optimizer_step
        should_wait = averaging_round or optimizer_step or zero_grad if self.delta_rule_averaging else averaging_round
        if wait_for_delayed_updates is None:
            wait_for_delayed_updates = should_wait
        if should_wait and not (wait_for_delayed_updates and apply_delayed_updates):
            raise ValueError("Should wait for background operation to finish before scheduling new one")
        assert not delay_optimizer_step or delay_averaging, "Delayed optimizer step requires delayed averaging"
        if delay_optimizer_step:
            assert self.offload_optimizer, "Delayed optimizer step is only available with offload_optimizer"
            assert not averaging_round or delay_averaging, "Averaging after delayed optimizer should also be delayed"
        if averaging_opts and not averaging_round:
            logger.warning(f"Averaging parameters not used because averaging_round=False: {averaging_opts}")
        if averaging_control is not None:
            assert averaging_round, "averaging_control is unused if averaging_round is not performed"
        if wait_for_trigger is not None:
            assert optimizer_step or zero_grad or averaging_round, "trigger is only used for updating parameters"
            if not (self.reuse_tensors or self.custom_gradients):
                # the trigger fires in the background, i.e. possibly after the caller has overwritten its gradients:
                # only safe when the optimizer has its own gradient buffers that the caller fills explicitly
                raise ValueError("wait_for_trigger requires reuse_tensors or custom_gradients (manual gradient handling)")
        output = None

        if wait_for_delayed_updates:
            for pending_update in list(self.pending_updates):
                try:
                    timeout = (averaging_opts or {}).get("averaging_timeout", self._allreduce_timeout)
                    logger.log(self.status_loglevel, "Waiting for delayed updates to finish...")
                    output = pending_update.result(timeout)
                except BaseException:
                    if not pending_update.done():
                        pending_update.cancel()
        finished = {update for update in self.pending_updates if update.done()}
        self.pending_updates = {update for update in self.pending_updates if not update.done()}
        for update in finished:
            if update.cancelled() or update.exception():
                logger.log(self.status_loglevel, f"Background update failed: {update}")

        if apply_delayed_updates:
            if self.finished_averaging_round.is_set():
                if not self.reuse_tensors:
                    self._apply_averaging_results_()
                if self.offload_optimizer and not self.finished_optimizer_step.is_set():
                    self._apply_optimizer_parameters_()
                logger.log(self.status_loglevel, "Received parameters from background averaging round")
                self.finished_averaging_round.clear()
            if self.finished_optimizer_step.is_set():
                if self.offload_optimizer:
                    self._apply_optimizer_parameters_()
                logger.debug("Received parameters from background optimizer step")
                self.finished_optimizer_step.clear()

        if increment_epoch:
            self.local_epoch += 1

        if optimizer_step or zero_grad or averaging_round:
            if self.offload_optimizer and not self.custom_gradients:
                self._load_local_grads_into_optimizer_()
            pending_update = self.step_executor.submit(self._do, wait_for_trigger, optimizer_step, zero_grad,
                                                       averaging_round, averaging_control, grad_scaler, set_to_none,
                                                       **averaging_opts or {})
            self.pending_updates.add(pending_update)
            should_await_optimizer = (optimizer_step or zero_grad) and not delay_optimizer_step
            should_await_averaging = averaging_round and not delay_averaging
            if should_await_optimizer:
                self.finished_optimizer_step.wait()
                self.finished_optimizer_step.clear()
                if self.offload_optimizer and not should_await_averaging:
                    self._apply_optimizer_parameters_()
                logger.debug("Finished optimizer step")
            if should_await_averaging:
                self.finished_averaging_round.wait()
                self.finished_averaging_round.clear()
                if not self.reuse_tensors:
                    self._apply_averaging_results_()
                if self.offload_optimizer:
                    self._apply_optimizer_parameters_()
                logger.log(self.status_loglevel, "Finished averaging round")
            async_averaging = averaging_round and delay_averaging
            async_optimizer = (optimizer_step or zero_grad) and delay_optimizer_step
            if not (async_averaging or async_optimizer):
                try:
                    output = pending_update.result()
                finally:
                    self.pending_updates.discard(pending_update)
        return output

    def _do(self, wait_for_trigger, optimizer_step: bool, zero_grad: bool, averaging_round: bool,
            averaging_control: Optional[StepControl], grad_scaler, set_to_none: bool, timeout: Optional[float] = None,
            **kwargs):
        """Background worker: (trigger) -> optimizer step -> zero_grad -> scheduler -> averaging round."""
        if averaging_control is not None and (averaging_control.triggered or averaging_control.done()):
            logger.log(self.status_loglevel, f"Discarding failed matchmaking results: {averaging_control}")
            averaging_control = None
        start_time = time.perf_counter()
        began_running = False
        try:
            if averaging_round and averaging_control is None:
                averaging_control = super().step(gather=self.local_epoch, require_trigger=True, timeout=timeout,
                                                 wait=False, **kwargs)
            if wait_for_trigger is not None:
                wait_for_trigger()
            began_running = True
            with self.lock_optimizer:
                if optimizer_step:
                    with self.lock_averaged_tensors if self.reuse_tensors else nullcontext():
                        logger.debug("Running optimizer step")
                        if grad_scaler is None:
                            self.optimizer.step()
                        else:
                            with grad_scaler.running_global_step():
                                assert grad_scaler.step(self.optimizer)
                if zero_grad:
                    logger.debug("Running zero grad")
                    self.optimizer.zero_grad()
                    if self.offload_optimizer:
                        for parameter in self.main_parameters:
                            if set_to_none:
                                parameter.grad = None
                            elif parameter.grad is not None:
                                parameter.grad.zero_()
                self._update_scheduler()
                self.finished_optimizer_step.set()
            if averaging_round:
                with self.lock_averaging:
                    if not self.reuse_tensors:
                        self._load_local_tensors_into_averager_()
                    if self.delta_rule_averaging:
                        with torch.no_grad(), self.get_tensors() as averaged_tensors:
                            self._old_tensors = tuple(x.clone() for x in averaged_tensors)
                    self.delay_before_averaging.update(task_size=1, interval=time.perf_counter() - start_time)
                    try:
                        averaging_control.allow_allreduce()
                        gathered = averaging_control.result(timeout=timeout)
                        logger.log(self.status_loglevel, f"Averaged parameters with {len(gathered)} peers")
                    except BaseException as e:
                        logger.log(self.status_loglevel, f"Averaging failed with {type(e)}")
                        gathered = {}
                    self.finished_averaging_round.set()
                if self.sync_epoch_when_averaging:
                    old_epoch = self.local_epoch
                    for peer_epoch in gathered.values():
                        self.local_epoch = max(self.local_epoch, peer_epoch)
                    if self.local_epoch != old_epoch:
                        logger.log(self.status_loglevel, f"Found peer with newer epoch ({self.local_epoch})")
                        self._update_scheduler()
        except Exception as e:
            if not began_running:
                logger.error(f"Aborted {self.__class__.__name__}.step because wait_for_trigger raised exception")
            logger.exception(e)
            if averaging_control is not None and not averaging_control.done():
                logger.error("Cancelled scheduled state averaging round")
                averaging_control.cancel()
            self.finished_optimizer_step.set()
            self.finished_averaging_round.set()

    # ---------------------------------------------------------------------------------------------- copies
    def _optimizer_parameters(self):
        return [param for group in self.optimizer.param_groups for param in group["params"]]

    @torch.no_grad()
    def _load_local_grads_into_optimizer_(self) -> None:
        """Copy the model's gradients into the gradient buffers of the offloaded optimizer."""
        assert self.offload_optimizer
        dst, src = [], []
        for main_param, opt_param in zip(self.main_parameters, self._optimizer_parameters()):
            if main_param.grad is not None:
                if opt_param.grad is None:
                    opt_param.grad = main_param.grad.detach().to(opt_param.dtype, copy=True)
                else:
                    dst.append(opt_param.grad)
                    src.append(main_param.grad)
        _copy_all_(dst, src)

    @torch.no_grad()
    def _apply_optimizer_parameters_(self) -> None:
        """Copy parameters from the offloaded optimizer into the model."""
        assert self.offload_optimizer
        offloaded = self._optimizer_parameters()
        assert len(offloaded) == len(self.main_parameters), "Optimizer parameters changed during training"
        _copy_all_(list(self.main_parameters), offloaded)
        for p in self.main_parameters:
            torch.autograd.graph.increment_version(p)

    @torch.no_grad()
    def _load_local_tensors_into_averager_(self) -> None:
        assert not self.reuse_tensors
        with self.get_tensors() as averaged_tensors:
            _copy_all_(list(averaged_tensors), list(self._local_tensors()))

    @torch.no_grad()
    def _apply_averaging_results_(self) -> None:
        """Copy averaged tensors into the local ones (or add the change since the round began: the delta rule)."""
        assert not self.reuse_tensors
        if self.delta_rule_averaging and self._old_tensors is None:
            logger.warning("Using delta_rule_averaging, but old tensors were not found. Averaging may have failed")
        with self.get_tensors() as averaged_tensors:
            local_tensors = list(self._local_tensors())
            assert len(local_tensors) == len(averaged_tensors), "Tensor structure changed during training"
            if not self.delta_rule_averaging or self._old_tensors is None:
                _copy_all_(local_tensors, list(averaged_tensors))
            else:
                assert len(self._old_tensors) == len(local_tensors)
                if all(l.device == n.device and l.dtype == torch.float32 for l, n in zip(local_tensors, averaged_tensors)):
                    mt.delta_update_(local_tensors, list(averaged_tensors), list(self._old_tensors))
                else:
                    for local_tensor, new_tensor, old_tensor in zip(local_tensors, averaged_tensors, self._old_tensors):
                        local_tensor.add_((new_tensor - old_tensor).to(local_tensor.device, local_tensor.dtype))
            for t in local_tensors:
                torch.autograd.graph.increment_version(t)

    @property
    def averaging_in_progress(self) -> bool:
        return self.lock_averaging.locked()

    # ---------------------------------------------------------------------------------------------- state exchange
    def get_current_state(self):
        """(metadata, tensors, infos) for peers that download our state.

        Layout contract (hivemind/optim/state_averager.py:627-656): metadata = {epoch, group_bits,
        optimizer_metadata}; tensors = parameters, extra tensors, then optimizer tensors in ``nested_flatten``
        order of the optimizer's ``state_dict()``.
        """
        with torch.no_grad(), self.lock_averaged_tensors:
            optimized_parameters = tuple(param.detach().cpu() for param in self._optimizer_parameters())
            parameter_infos = [CompressionInfo.from_tensor(param, key=key, role=TensorRole.PARAMETER)
                               for param, key in zip(optimized_parameters, self.parameter_names)]
            extra_tensors = tuple(tensor.detach().cpu() for tensor in self.extra_tensors)
            extra_infos = [CompressionInfo.from_tensor(extra_tensor, key=i, role=TensorRole.UNSPECIFIED)
                           for i, extra_tensor in enumerate(extra_tensors)]
            optimizer_metadata, optimizer_tensors = dump_optimizer_state(self.optimizer)
            optimizer_infos = [CompressionInfo.from_tensor(opt_tensor, key=i, role=TensorRole.OPTIMIZER)
                               for i, opt_tensor in enumerate(optimizer_tensors)]
        metadata = dict(epoch=self.local_epoch, group_bits=self.get_group_bits(), optimizer_metadata=optimizer_metadata)
        all_tensors = list(chain(optimized_parameters, extra_tensors, optimizer_tensors))
        all_tensor_infos = list(chain(parameter_infos, extra_infos, optimizer_infos))
        return metadata, all_tensors, all_tensor_infos

    def load_state_from_peers(self, **kwargs) -> None:
        """Download the latest training state from a peer and load it into the model, optimizer and scheduler."""
        opt_parameters = tuple(self._optimizer_parameters())
        main_parameters_and_extras = tuple(chain(opt_parameters, self.extra_tensors))
        num_parameters_and_extras = len(main_parameters_and_extras)
        loaded_state = super().load_state_from_peers(**kwargs)
        if loaded_state is None:
            return
        metadata, flat_tensors = loaded_state
        if (not isinstance(metadata.get("epoch"), int)) or metadata["epoch"] < self.local_epoch:
            logger.warning("Cowardly refusing to load state from peer: peer's epoch is behind our local epoch")
            return
        loaded_parameters_and_extras = flat_tensors[:num_parameters_and_extras]
        loaded_opt_tensors = flat_tensors[num_parameters_and_extras:]
        if num_parameters_and_extras != len(loaded_parameters_and_extras):
            logger.error("Failed to load state from peer, received parameters, extras or metadata")
            return
        with torch.no_grad(), self.lock_averaged_tensors:
            try:
                load_optimizer_state(self.optimizer, metadata["optimizer_metadata"], loaded_opt_tensors)
            except StopIteration:
                logger.warning("Failed to load state from peer, received inconsistent number of optimizer statistics")
                return
            for local_param, loaded_param in zip(main_parameters_and_extras, loaded_parameters_and_extras):
                local_param.copy_(loaded_param.to(local_param.device, local_param.dtype), non_blocking=True)
        if self.offload_optimizer:
            self._apply_optimizer_parameters_()
        if not self.reuse_tensors:
            self._load_local_tensors_into_averager_()
        self.local_epoch = metadata["epoch"]
        self._update_scheduler()

    def _update_scheduler(self) -> None:
        """Bring the LR schedule to ``local_epoch`` (one scheduler step per epoch)."""
        if self.scheduler:
            while self.scheduler._step_count <= self.local_epoch:
                self.scheduler.step()

    def shutdown(self) -> None:
        self.step_executor.shutdown(wait=False)
        super().shutdown()


def initialize_optimizer_state_(opt: torch.optim.Optimizer) -> None:
    """Create optimizer statistics by running one step with zero gradients (parameters are restored afterwards)."""
    flat_params = tuple(param for group in opt.param_groups for param in group["params"])
    old_grads, old_values = [], []
    for param in flat_params:
        old_grads.append(param.grad)
        old_values.append(param.detach().clone())
        param.grad = torch.zeros_like(param)
    opt.step()
    with torch.no_grad():
        for param, old_grad, old_value in zip(flat_params, old_grads, old_values):
            param.grad = old_grad
            param.copy_(old_value)


def dump_optimizer_state(opt: torch.optim.Optimizer):
    """Split an optimizer ``state_dict`` into msgpack-friendly metadata and a list of CPU tensors."""
    with torch.no_grad():
        flat_metadata, flat_tensors = [], []
        for elem in nested_flatten(opt.state_dict()):
            if isinstance(elem, torch.Tensor):
                flat_metadata.append(dict(type="tensor", index=len(flat_tensors)))
                flat_tensors.append(elem.cpu())
            else:
                flat_metadata.append(dict(type="value", value=elem))
        return flat_metadata, flat_tensors


def load_optimizer_state(optimizer: torch.optim.Optimizer, flat_metadata, flat_tensors: Sequence[torch.Tensor]):
    """Inverse of ``dump_optimizer_state``: rebuild the state dict in the optimizer's own structure and load it."""
    flat_optimizer_state = []
    for elem in flat_metadata:
        if elem.get("type") == "tensor" and isinstance(elem.get("index"), int):
            flat_optimizer_state.append(flat_tensors[elem["index"]])
        elif elem.get("type") == "value" and "value" in elem:
            flat_optimizer_state.append(elem["value"])
    return optimizer.load_state_dict(nested_pack(flat_optimizer_state, structure=optimizer.state_dict()))

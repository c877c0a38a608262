"""``TrainingStateAverager``: owns the optimizer, the LR schedule and the copy of the training state that peers average.

Contract (hivemind/optim/state_averager.py:37-740): the *state* is the parameters, optionally some optimizer
statistics and extra tensors. One ``step(...)`` call may, in this order and each optionally in the background, run an
optimizer step, ``zero_grad``, a scheduler step and an averaging round with peers; what finished in the background is
copied into the model by a later call. Peers that fell behind download the whole state (``load_state_from_peers``),
whose layout is fixed by ``get_current_state``.

How the tensors are kept here. There are up to three sets, all on the parameters' own device:

* ``main_parameters`` — the tensors the model trains with;
* the optimizer's parameters — the same tensors, or with ``offload_optimizer`` separate fp32 "shadow" copies, so that
  a delayed optimizer step never races with the next forward pass;
* the averaged tensors — with ``reuse_tensors`` the optimizer's tensors themselves, otherwise one more copy.

On CUDA the averaged tensors live in the averager's peer-mappable arena, and with ``offload_optimizer`` +
``reuse_tensors`` (the default pairing) the shadow copies ARE arena views: the fused optimizer updates the arena in
place and the butterfly kernels average it in place, with no staging copy in between. Copies between the sets and the
delta rule are single multi-tensor launches.
"""
from __future__ import annotations

import logging
import os
import threading
import time
from concurrent.futures import Future, ThreadPoolExecutor
from dataclasses import dataclass
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple, Union

import torch

from hivemind_b200.averaging import DecentralizedAverager, StepControl
from hivemind_b200.compression import CompressionInfo, NoCompression, TensorRole
from hivemind_b200.dht import DHT
from hivemind_b200.ops import multi_tensor as mt
from hivemind_b200.utils import DHTExpiration, PerformanceEMA, get_logger, nested_flatten, nested_pack

logger = get_logger(__name__)

Parameters = Iterable[torch.Tensor]
ParamGroups = Iterable[Dict[str, Any]]
TorchOptimizer = torch.optim.Optimizer
LRSchedulerBase = getattr(torch.optim.lr_scheduler, "LRScheduler", None) or torch.optim.lr_scheduler._LRScheduler
OptimizerFactory = Callable[[Union[Parameters, ParamGroups]], TorchOptimizer]
SchedulerFactory = Callable[[TorchOptimizer], LRSchedulerBase]


def _bulk_copy(dst: Sequence[torch.Tensor], src: Sequence[torch.Tensor]) -> None:
    """``dst[i] <- src[i]`` for all pairs that are not already the same memory; one launch when the kernels apply."""
    todo = [(d, s) for d, s in zip(dst, src) if d.data_ptr() != s.data_ptr() or d.device != s.device]
    if not todo:
        return
    fusable = all(d.device == s.device and d.is_contiguous() and s.is_contiguous() and d.is_floating_point()
                  and s.is_floating_point() for d, s in todo)
    if fusable:
        mt.scale_copy_([d for d, _ in todo], [s for _, s in todo], 1.0)
    else:
        for d, s in todo:
            d.copy_(s, non_blocking=True)


def _bump_versions(tensors: Iterable[torch.Tensor]) -> None:
    """Tell autograd-side caches (e.g. bf16 weight copies keyed by ``_version``) that the tensors changed."""
    for t in tensors:
        torch.autograd.graph.increment_version(t)


@dataclass
class _Request:
    """What one ``step`` call asked the background worker to do."""

    trigger: Optional[Callable[[], Any]]
    optimizer_step: bool
    zero_grad: bool
    averaging_round: bool
    control: Optional[StepControl]
    grad_scaler: Any
    set_to_none: bool
    averaging_opts: Dict[str, Any]


class TrainingStateAverager(DecentralizedAverager):
    """
    :param optimizer: a ``torch.optim.Optimizer`` or a factory ``params -> optimizer`` (required for offloading)
    :param params: parameters or param groups (default: the optimizer's groups)
    :param scheduler: an LR scheduler or a factory ``optimizer -> scheduler``
    :param initialize_optimizer: run one zero-gradient step so that optimizer statistics exist (default: if needed)
    :param offload_optimizer: the optimizer updates shadow copies instead of the model's own tensors
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
        self.opt_keys_for_averaging = tuple(average_opt_statistics)
        if not all(isinstance(key, str) for key in self.opt_keys_for_averaging):
            raise TypeError("average_opt_statistics must be names of optimizer statistics")
        self.extra_tensors = tuple(extra_tensors)
        if reuse_tensors is None:
            reuse_tensors = offload_optimizer and not delta_rule_averaging
        if reuse_tensors and delta_rule_averaging:
            raise ValueError("reuse_tensors and delta_rule_averaging are mutually exclusive")
        if custom_gradients and not offload_optimizer:
            logger.warning("custom_gradients=True has no effect unless the optimizer is offloaded")
        self.status_loglevel = status_loglevel
        self.offload_optimizer, self.custom_gradients = offload_optimizer, custom_gradients
        self.reuse_tensors, self.delta_rule_averaging = reuse_tensors, delta_rule_averaging
        self.sync_epoch_when_averaging = sync_epoch_when_averaging
        self.local_epoch = 0

        groups, self.main_parameters, self.parameter_names = self._normalise_params(optimizer, params, parameter_names)
        optimizer_is_factory = callable(optimizer) and not isinstance(optimizer, TorchOptimizer)
        scheduler_is_factory = callable(scheduler) and not isinstance(scheduler, LRSchedulerBase)
        if offload_optimizer and not optimizer_is_factory:
            raise ValueError("offload_optimizer needs an optimizer factory: the optimizer must be built on the copies")
        if optimizer_is_factory and scheduler is not None and not scheduler_is_factory:
            raise ValueError("with an optimizer factory the scheduler must be a factory too")

        # the optimizer's tensors: the model's own, or shadow copies (in the device arena when they are also averaged)
        endpoint = None
        if offload_optimizer:
            shadow = [p.detach().to(torch.float32, copy=True) for p in self.main_parameters]
            endpoint = self._maybe_arena_for(shadow, kwargs)
            if endpoint is not None:
                shadow = [v.detach() for v in endpoint.tensor_views]
            shadow = [s.requires_grad_(p.requires_grad) for s, p in zip(shadow, self.main_parameters)]
            for s in shadow:
                s.grad = torch.zeros_like(s)
            groups_for_optimizer, cursor = [], 0
            for group in groups:
                count = len(group["params"])
                groups_for_optimizer.append(dict(group, params=shadow[cursor:cursor + count]))
                cursor += count
        else:
            groups_for_optimizer = list(groups)
        self.optimizer = optimizer(groups_for_optimizer) if optimizer_is_factory else optimizer
        if not isinstance(self.optimizer, TorchOptimizer) or len(self.optimizer.param_groups) != len(groups):
            raise TypeError("the optimizer (factory) must yield a torch optimizer with the given parameter groups")
        if initialize_optimizer is None:
            initialize_optimizer = not any(torch.is_tensor(x) for x in nested_flatten(self.optimizer.state_dict()))
        if initialize_optimizer:
            logger.log(status_loglevel, "Creating optimizer statistics with one zero-gradient step")
            initialize_optimizer_state_(self.optimizer)
        self.scheduler = scheduler(self.optimizer) if scheduler_is_factory else scheduler
        if self.scheduler is not None and self.scheduler.optimizer is not self.optimizer:
            raise ValueError("the scheduler must belong to this optimizer")

        tracked = self._tracked_tensors()
        if reuse_tensors:
            averaged = [t.detach() if endpoint is None else t for t in tracked]
        else:
            averaged = [t.detach().to(torch.float32, copy=True) for t in tracked]
        if reuse_tensors and endpoint is None:
            # tensors that other code holds on to cannot move into an arena
            kwargs.setdefault("use_device_path", False)
        self._rounds_lock = threading.Lock()            # held while a round may modify the averaged tensors
        self._optimizer_lock = threading.Lock()
        self._snapshot: Optional[List[torch.Tensor]] = None   # averaged tensors as they were when the round began
        self.delay_before_averaging = PerformanceEMA(alpha=performance_ema_alpha)
        self._worker = ThreadPoolExecutor(max_workers=2 if delta_rule_averaging else 1,
                                          thread_name_prefix="state-averager")
        self.finished_optimizer_step = threading.Event()
        self.finished_averaging_round = threading.Event()
        self.pending_updates: set = set()
        super().__init__(dht=dht, averaged_tensors=averaged, tensor_infos=self._describe_tensors(),
                         device_endpoint=endpoint, **kwargs)

    # ---------------------------------------------------------------------------------------------- set-up helpers
    @staticmethod
    def _normalise_params(optimizer, params, names) -> Tuple[Tuple[dict, ...], Tuple[torch.Tensor, ...], Tuple]:
        if params is None:
            if not hasattr(optimizer, "param_groups"):
                raise ValueError("pass params, or an optimizer instance whose param_groups can be used")
            params = optimizer.param_groups
        params = tuple(params)
        groups = (dict(params=list(params)),) if all(torch.is_tensor(p) for p in params) else params
        flat: List[torch.Tensor] = []
        for group in groups:
            if not isinstance(group, dict) or not all(torch.is_tensor(p) for p in group.get("params", [None])):
                raise TypeError("params must be tensors or dicts with a 'params' list of tensors")
            flat.extend(group["params"])
        if len({id(p) for p in flat}) != len(flat):
            raise ValueError("a parameter appears in more than one group")
        names = tuple(range(len(flat))) if names is None else tuple(nested_flatten(names))
        if len(names) != len(flat):
            raise ValueError(f"{len(flat)} parameters but {len(names)} names")
        frozen = sum(p.numel() for p in flat if not p.requires_grad)
        if frozen and frozen >= sum(p.numel() for p in flat) - frozen:
            logger.warning("most synchronised parameters are frozen; leave them out of the optimizer to save traffic")
        return tuple(groups), tuple(flat), names

    def _maybe_arena_for(self, shadow: Sequence[torch.Tensor], averager_kwargs: Dict[str, Any]):
        """An arena that holds the shadow parameters, if they are also the averaged tensors and the device data
        path applies (CUDA, nothing but parameters to average); None otherwise."""
        wanted = averager_kwargs.get("use_device_path")
        if wanted is None:
            wanted = os.environ.get("HIVEMIND_DEVICE_BUTTERFLY", "1") != "0"
        if not (wanted and self.reuse_tensors and shadow and all(s.is_cuda for s in shadow)):
            return None
        if self.opt_keys_for_averaging or self.extra_tensors:
            return None
        from hivemind_b200.parallel.device_butterfly import DeviceEndpoint

        infos = [CompressionInfo.from_tensor(s, key=name, role=TensorRole.PARAMETER)
                 for s, name in zip(shadow, self.parameter_names)]
        return DeviceEndpoint(shadow, averager_kwargs.get("compression", NoCompression()), infos,
                              averager_kwargs.get("part_size_bytes", 2 ** 19))

    def _optimizer_parameters(self) -> List[torch.Tensor]:
        return [p for group in self.optimizer.param_groups for p in group["params"]]

    def _tracked_tensors(self) -> List[torch.Tensor]:
        """The trainer-side tensors that correspond one to one to the averaged tensors: optimizer parameters, the
        chosen optimizer statistics (statistic by statistic), extra tensors."""
        tensors = self._optimizer_parameters()
        for key in self.opt_keys_for_averaging:
            tensors += [self.optimizer.state[p][key] for p in self._optimizer_parameters()]
        return tensors + list(self.extra_tensors)

    def _describe_tensors(self) -> Tuple[CompressionInfo, ...]:
        infos = [CompressionInfo.from_tensor(p, key=name, role=TensorRole.PARAMETER)
                 for p, name in zip(self.main_parameters, self.parameter_names)]
        for key in self.opt_keys_for_averaging:
            infos += [CompressionInfo.from_tensor(self.optimizer.state[p][key], key=(name, key), role=TensorRole.OPTIMIZER)
                      for p, name in zip(self._optimizer_parameters(), self.parameter_names)]
        infos += [CompressionInfo.from_tensor(t, key=i, role=TensorRole.UNSPECIFIED) for i, t in enumerate(self.extra_tensors)]
        return tuple(infos)

    # ---------------------------------------------------------------------------------------------- public API
    @property
    def averaging_in_progress(self) -> bool:
        return self._rounds_lock.locked()

    def schedule_step(self, scheduled_time: Optional[DHTExpiration] = None, **kwargs) -> StepControl:
        """Begin matchmaking for a state-averaging round ahead of time (see ``step(averaging_control=...)``)."""
        if kwargs.get("weight") is not None:
            raise ValueError("a pre-scheduled state averaging round cannot carry a weight")
        return super().step(scheduled_time=scheduled_time, wait=False, require_trigger=True, **kwargs)

    def step(self, wait_for_delayed_updates: bool = None, apply_delayed_updates: bool = True,
             increment_epoch: bool = False, optimizer_step: bool = False, zero_grad: bool = False,
             delay_optimizer_step: bool = False, averaging_round: bool = False, delay_averaging: Optional[bool] = None,
             averaging_control: Optional[StepControl] = None, wait_for_trigger: Optional[Callable[[], Any]] = None,
             grad_scaler=None, averaging_opts: Optional[Dict[str, Any]] = None, set_to_none: bool = False):
        """Run any combination of: apply finished background results, optimizer step, zero_grad, averaging round.

        :param wait_for_delayed_updates: wait for background work started by earlier calls
        :param apply_delayed_updates: copy finished background results into the model
        :param increment_epoch: ``local_epoch += 1`` (the scheduler follows the epoch)
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
        touches_state = averaging_round or (self.delta_rule_averaging and (optimizer_step or zero_grad))
        if wait_for_delayed_updates is None:
            wait_for_delayed_updates = touches_state
        if touches_state and not (wait_for_delayed_updates and apply_delayed_updates):
            raise ValueError("earlier background work must be awaited and applied before new work is scheduled")
        if delay_optimizer_step and not self.offload_optimizer:
            raise ValueError("a delayed optimizer step needs offload_optimizer")
        if delay_optimizer_step and not delay_averaging:
            raise ValueError("averaging that follows a delayed optimizer step must be delayed too")
        if averaging_control is not None and not averaging_round:
            raise ValueError("averaging_control was given but no averaging round was requested")
        if averaging_opts and not averaging_round:
            logger.warning(f"averaging_opts ignored without an averaging round: {averaging_opts}")
        if wait_for_trigger is not None:
            if not (optimizer_step or zero_grad or averaging_round):
                raise ValueError("wait_for_trigger only makes sense with work that modifies the state")
            if not (self.reuse_tensors or self.custom_gradients):
                # the trigger fires in the background, possibly after the caller has overwritten its gradients: only
                # safe when the optimizer has its own gradient buffers that the caller fills explicitly
                raise ValueError("wait_for_trigger requires reuse_tensors or custom_gradients")

        result = None
        if wait_for_delayed_updates:
            limit = (averaging_opts or {}).get("averaging_timeout", self._allreduce_timeout)
            for job in list(self.pending_updates):
                try:
                    logger.log(self.status_loglevel, "Waiting for background updates to finish")
                    result = job.result(limit)
                except BaseException:
                    job.cancel()
        for job in [j for j in self.pending_updates if j.done()]:
            self.pending_updates.discard(job)
            if job.cancelled() or job.exception() is not None:
                logger.log(self.status_loglevel, f"A background update failed: {job}")

        if apply_delayed_updates:
            self._collect_background_results()
        if increment_epoch:
            self.local_epoch += 1
        if not (optimizer_step or zero_grad or averaging_round):
            return result

        if self.offload_optimizer and not self.custom_gradients:
            self._hand_gradients_to_optimizer()
        request = _Request(wait_for_trigger, optimizer_step, zero_grad, averaging_round, averaging_control, grad_scaler,
                           set_to_none, dict(averaging_opts or {}))
        job: Future = self._worker.submit(self._background, request)
        self.pending_updates.add(job)
        optimizer_in_foreground = (optimizer_step or zero_grad) and not delay_optimizer_step
        averaging_in_foreground = averaging_round and not delay_averaging
        if optimizer_in_foreground:
            self.finished_optimizer_step.wait()
            self.finished_optimizer_step.clear()
            if self.offload_optimizer and not averaging_in_foreground:
                self._publish_optimizer_parameters()
        if averaging_in_foreground:
            self.finished_averaging_round.wait()
            self.finished_averaging_round.clear()
            self._take_over_averaged_state()
            logger.log(self.status_loglevel, "Finished the averaging round")
        everything_awaited = (optimizer_in_foreground or not (optimizer_step or zero_grad)) and \
                             (averaging_in_foreground or not averaging_round)
        if everything_awaited:
            try:
                result = job.result()
            finally:
                self.pending_updates.discard(job)
        return result

    def _collect_background_results(self) -> None:
        """Bring what the worker has finished since the last call into the model."""
        if self.finished_averaging_round.is_set():
            self._take_over_averaged_state(optimizer_too=not self.finished_optimizer_step.is_set())
            self.finished_averaging_round.clear()
            logger.log(self.status_loglevel, "Took over parameters from a background averaging round")
        if self.finished_optimizer_step.is_set():
            if self.offload_optimizer:
                self._publish_optimizer_parameters()
            self.finished_optimizer_step.clear()

    def _take_over_averaged_state(self, optimizer_too: bool = True) -> None:
        if not self.reuse_tensors:
            self._adopt_averaged_tensors()
        if self.offload_optimizer and optimizer_too:
            self._publish_optimizer_parameters()

    # ---------------------------------------------------------------------------------------------- background
    def _background(self, req: _Request):
        """Worker body: (trigger) -> optimizer step -> zero_grad -> scheduler -> averaging round."""
        control = req.control
        if control is not None and (control.triggered or control.done()):
            logger.log(self.status_loglevel, f"The pre-scheduled round is of no use any more: {control}")
            control = None
        began, started_at = False, time.perf_counter()
        timeout = req.averaging_opts.pop("timeout", None)
        try:
            if req.averaging_round and control is None:
                control = super().step(gather=self.local_epoch, require_trigger=True, timeout=timeout, wait=False,
                                       **req.averaging_opts)
            if req.trigger is not None:
                req.trigger()
            began = True
            with self._optimizer_lock:
                if req.optimizer_step:
                    guard = self.lock_averaged_tensors if self.reuse_tensors else threading.Lock()
                    with guard:
                        if req.grad_scaler is None:
                            self.optimizer.step()
                        else:
                            with req.grad_scaler.running_global_step():
                                if not req.grad_scaler.step(self.optimizer):
                                    raise RuntimeError("the gradient scaler refused a global optimizer step")
                if req.zero_grad:
                    self.optimizer.zero_grad()
                    if self.offload_optimizer:
                        for p in self.main_parameters:
                            if req.set_to_none:
                                p.grad = None
                            elif p.grad is not None:
                                p.grad.zero_()
                self._update_scheduler()
                self.finished_optimizer_step.set()
            if req.averaging_round:
                gathered = self._averaging_round(control, timeout, started_at)
                if self.sync_epoch_when_averaging:
                    newest = max([self.local_epoch, *[e for e in gathered.values() if isinstance(e, int)]])
                    if newest != self.local_epoch:
                        logger.log(self.status_loglevel, f"A groupmate is at epoch {newest}; catching up")
                        self.local_epoch = newest
                        self._update_scheduler()
        except Exception as e:
            if not began:
                logger.error(f"{type(self).__name__}: the trigger failed, nothing was modified")
            logger.exception(e)
            if control is not None and not control.done():
                control.cancel()
            self.finished_optimizer_step.set()
            self.finished_averaging_round.set()

    def _averaging_round(self, control: StepControl, timeout: Optional[float], started_at: float) -> Dict:
        with self._rounds_lock:
            if not self.reuse_tensors:
                self._refresh_averaged_tensors()
            if self.delta_rule_averaging:
                with torch.no_grad(), self.get_tensors() as averaged:
                    self._snapshot = [t.clone() for t in averaged]
            self.delay_before_averaging.update(task_size=1, interval=time.perf_counter() - started_at)
            try:
                control.allow_allreduce()
                gathered = control.result(timeout=timeout)
                logger.log(self.status_loglevel, f"Averaged state with {len(gathered)} peers")
            except BaseException as e:
                logger.log(self.status_loglevel, f"State averaging failed: {e!r}")
                gathered = {}
            self.finished_averaging_round.set()
        return gathered

    # ---------------------------------------------------------------------------------------------- copies
    @torch.no_grad()
    def _hand_gradients_to_optimizer(self) -> None:
        """Model gradients -> gradient buffers of the offloaded optimizer."""
        dst, src = [], []
        for model_p, opt_p in zip(self.main_parameters, self._optimizer_parameters()):
            if model_p.grad is None:
                continue
            if opt_p.grad is None:
                opt_p.grad = model_p.grad.detach().to(opt_p.dtype, copy=True)
            else:
                dst.append(opt_p.grad)
                src.append(model_p.grad)
        _bulk_copy(dst, src)

    @torch.no_grad()
    def _publish_optimizer_parameters(self) -> None:
        """Offloaded optimizer parameters -> model."""
        shadow = self._optimizer_parameters()
        if len(shadow) != len(self.main_parameters):
            raise RuntimeError("the optimizer's parameters changed during training")
        _bulk_copy(list(self.main_parameters), shadow)
        _bump_versions(self.main_parameters)

    @torch.no_grad()
    def _refresh_averaged_tensors(self) -> None:
        """Trainer-side tensors -> averaged copies (only when they are separate)."""
        with self.get_tensors() as averaged:
            _bulk_copy(list(averaged), self._tracked_tensors())

    @torch.no_grad()
    def _adopt_averaged_tensors(self) -> None:
        """Averaged copies -> trainer-side tensors; with the delta rule, only what the round changed is added."""
        if self.delta_rule_averaging and self._snapshot is None:
            logger.warning("delta_rule_averaging is on but there is no snapshot; did the averaging round fail?")
        with self.get_tensors() as averaged:
            local = self._tracked_tensors()
            if len(local) != len(averaged):
                raise RuntimeError("the set of averaged tensors changed during training")
            if not self.delta_rule_averaging or self._snapshot is None:
                _bulk_copy(local, list(averaged))
            elif all(l.device == a.device and l.dtype == torch.float32 for l, a in zip(local, averaged)):
                mt.delta_update_(local, list(averaged), list(self._snapshot))
            else:
                for l, new, old in zip(local, averaged, self._snapshot):
                    l.add_((new - old).to(l.device, l.dtype))
            _bump_versions(local)

    # ---------------------------------------------------------------------------------------------- state exchange
    def get_current_state(self):
        """(metadata, tensors, infos) for peers that download our state.

        Layout (hivemind/optim/state_averager.py:627-656): metadata = {epoch, group_bits, optimizer_metadata};
        tensors = parameters, extra tensors, then the optimizer's tensors in ``nested_flatten`` order of its
        ``state_dict()``. CUDA tensors are handed over as they are: the state codecs have device encoders, so only
        compressed bytes travel to the host.
        """
        with torch.no_grad(), self.lock_averaged_tensors:
            params = [p.detach().clone() for p in self._optimizer_parameters()]
            extras = [t.detach().clone() for t in self.extra_tensors]
            opt_meta, opt_tensors = dump_optimizer_state(self.optimizer, to_cpu=False)
        infos = [CompressionInfo.from_tensor(p, key=name, role=TensorRole.PARAMETER)
                 for p, name in zip(params, self.parameter_names)]
        infos += [CompressionInfo.from_tensor(t, key=i, role=TensorRole.UNSPECIFIED) for i, t in enumerate(extras)]
        infos += [CompressionInfo.from_tensor(t, key=i, role=TensorRole.OPTIMIZER) for i, t in enumerate(opt_tensors)]
        metadata = dict(epoch=self.local_epoch, group_bits=self.get_group_bits(), optimizer_metadata=opt_meta)
        return metadata, params + extras + list(opt_tensors), infos

    def load_state_from_peers(self, **kwargs) -> None:
        """Download the newest training state on offer and load it into model, optimizer and scheduler."""
        targets = self._optimizer_parameters() + list(self.extra_tensors)
        downloaded = super().load_state_from_peers(**kwargs)
        if downloaded is None:
            return
        metadata, tensors = downloaded
        epoch = metadata.get("epoch")
        if not isinstance(epoch, int) or epoch < self.local_epoch:
            logger.warning("Not loading a peer's state: it is older than ours")
            return
        if len(tensors) < len(targets):
            logger.error("Not loading a peer's state: it has fewer tensors than we have parameters")
            return
        with torch.no_grad(), self.lock_averaged_tensors:
            try:
                load_optimizer_state(self.optimizer, metadata["optimizer_metadata"], tensors[len(targets):])
            except (StopIteration, KeyError, ValueError):
                logger.warning("Not loading a peer's state: its optimizer statistics do not match ours")
                return
            for mine, theirs in zip(targets, tensors):
                mine.copy_(theirs.to(mine.device, mine.dtype), non_blocking=True)
        if self.offload_optimizer:
            self._publish_optimizer_parameters()
        if not self.reuse_tensors:
            self._refresh_averaged_tensors()
        self.local_epoch = epoch
        self._update_scheduler()

    def _update_scheduler(self) -> None:
        """One scheduler step per epoch: catch the schedule up with ``local_epoch``."""
        if self.scheduler is not None:
            while self.scheduler._step_count <= self.local_epoch:
                self.scheduler.step()

    def shutdown(self) -> None:
        self._worker.shutdown(wait=False)
        super().shutdown()


def initialize_optimizer_state_(opt: torch.optim.Optimizer) -> None:
    """Make the optimizer allocate its statistics: one step on zero gradients, after which parameters and
    gradients are put back as they were."""
    saved = [(p, p.grad, p.detach().clone()) for group in opt.param_groups for p in group["params"]]
    for p, _, _ in saved:
        p.grad = torch.zeros_like(p)
    opt.step()
    with torch.no_grad():
        for p, grad, value in saved:
            p.grad = grad
            p.copy_(value)


def dump_optimizer_state(opt: torch.optim.Optimizer, to_cpu: bool = True):
    """Flatten ``opt.state_dict()`` into msgpack-friendly metadata plus the list of tensors it refers to."""
    metadata, tensors = [], []
    with torch.no_grad():
        for leaf in nested_flatten(opt.state_dict()):
            if torch.is_tensor(leaf):
                metadata.append(dict(type="tensor", index=len(tensors)))
                tensors.append(leaf.cpu() if to_cpu else leaf.detach().clone())
            else:
                metadata.append(dict(type="value", value=leaf))
    return metadata, tensors


def load_optimizer_state(optimizer: torch.optim.Optimizer, flat_metadata, flat_tensors: Sequence[torch.Tensor]):
    """Inverse of ``dump_optimizer_state``: rebuild the state dict in the optimizer's own structure and load it."""
    leaves = []
    for entry in flat_metadata:
        kind = entry.get("type")
        if kind == "tensor" and isinstance(entry.get("index"), int):
            leaves.append(flat_tensors[entry["index"]])
        elif kind == "value" and "value" in entry:
            leaves.append(entry["value"])
    return optimizer.load_state_dict(nested_pack(leaves, structure=optimizer.state_dict()))

"""``hivemind_b200.Optimizer``: wraps a PyTorch optimizer for collaborative large-batch training.

Peers accumulate gradients locally; once the swarm as a whole has processed ``target_batch_size`` samples (an
*epoch*), peers average gradients in a matched group, run the same optimizer step, and optionally average
parameters. Modes (all as in the reference, hivemind/optim/optimizer.py:32-790): synchronous; delayed parameter
updates (``delay_optimizer_step`` / ``delay_grad_averaging`` / ``delay_state_averaging``: communication and the
optimizer step overlap with the next epoch's computation); local updates with periodic state averaging
(``use_local_updates``); client-mode and auxiliary peers. Any averaging failure degrades to a local step; a peer
that falls behind downloads the state from others. ``state_dict()`` is the inner optimizer's state dict plus
``state["local_epoch"]``.

On a B200 box every peer is one GPU: gradient accumulators, averaged gradients, master weights and optimizer
statistics stay in HBM, are averaged by the device butterfly over NVLink, and the per-parameter loops are fused
multi-tensor kernels; the control flow around them is unchanged.
"""
from __future__ import annotations

import logging
import os
import time
from functools import partial
from typing import Callable, Optional, Sequence, Union

import torch

from hivemind_b200.averaging.control import AveragingStage, StepControl
from hivemind_b200.compression import CompressionBase, NoCompression
from hivemind_b200.dht import DHT
from hivemind_b200.optim.grad_averager import GradientAverager
from hivemind_b200.optim.grad_scaler import GradScaler
from hivemind_b200.optim.progress_tracker import LocalTrainingProgress, ProgressTracker
from hivemind_b200.optim.state_averager import (LRSchedulerBase, OptimizerFactory, Parameters, ParamGroups,
                                                SchedulerFactory, TorchOptimizer, TrainingStateAverager)
from hivemind_b200.utils import PerformanceEMA, get_dht_time, get_logger

logger = get_logger(__name__)
GradientAveragerFactory = Callable[..., GradientAverager]


class Optimizer(torch.optim.Optimizer):
    """
    :param dht: a running DHT
    :param run_id: unique name of the training run; peers with the same run_id train together
    :param target_batch_size: global number of samples per optimizer step (epoch)
    :param batch_size_per_step: samples processed between two ``step()`` calls (or pass ``batch_size`` to step)
    :param optimizer: a PyTorch optimizer, or a factory ``params -> optimizer`` (needed for offloading / delays)
    :param params: parameters or param groups (required with an optimizer factory)
    :param scheduler: LR scheduler, or a factory ``optimizer -> scheduler``; it is stepped once per epoch
    :param matchmaking_time: start looking for a group this many seconds before the epoch is expected to end
    :param averaging_timeout: give up on an averaging round after this long
    :param allreduce_timeout / next_chunk_timeout: timeouts of the all-reduce proper (defaults derive from above)
    :param load_state_timeout: per-chunk timeout when downloading state from a peer
    :param reuse_grad_buffers: accumulate in ``param.grad`` (do not call ``zero_grad`` yourself)
    :param offload_optimizer: keep the optimizer on separate fp32 copies (default: when ``params`` is given)
    :param delay_optimizer_step / delay_grad_averaging / delay_state_averaging: run these in the background
    :param average_state_every: average parameters every this many epochs
    :param use_local_updates: step the optimizer after every batch and only average states periodically
    :param client_mode: this peer cannot accept incoming connections
    :param auxiliary: this peer only assists averaging and has no data
    :param grad_compression / state_averaging_compression / load_state_compression: codecs
    :param grad_averager_factory: e.g. ``PowerSGDGradientAverager`` with its options bound
    :param average_opt_statistics: optimizer statistics averaged along with parameters
    :param extra_tensors: other tensors to average with the state
    :param averager_opts / tracker_opts: extra kwargs for both averagers / for the progress tracker
    :param verbose: log status messages at INFO level
    """

    def __init__(self, *, dht: DHT, run_id: str, target_batch_size: int, batch_size_per_step: Optional[int] = None,
                 optimizer: Union[TorchOptimizer, OptimizerFactory],
                 params: Optional[Union[Parameters, ParamGroups]] = None,
                 scheduler: Optional[Union[LRSchedulerBase, SchedulerFactory]] = None,
                 matchmaking_time: Optional[float] = 15.0, averaging_timeout: Optional[float] = 60.0,
                 allreduce_timeout: Optional[float] = None, next_chunk_timeout: Optional[float] = None,
                 load_state_timeout: float = 600.0, reuse_grad_buffers: bool = False,
                 offload_optimizer: Optional[bool] = None, delay_optimizer_step: Optional[bool] = None,
                 delay_grad_averaging: bool = False, delay_state_averaging: bool = True, average_state_every: int = 1,
                 use_local_updates: bool = False, client_mode: bool = None, auxiliary: bool = False,
                 grad_compression: CompressionBase = NoCompression(),
                 grad_averager_factory: Optional[GradientAveragerFactory] = None,
                 state_averaging_compression: CompressionBase = NoCompression(),
                 load_state_compression: CompressionBase = NoCompression(), average_opt_statistics: Sequence[str] = (),
                 extra_tensors: Sequence[torch.Tensor] = (), averager_opts: Optional[dict] = None,
                 tracker_opts: Optional[dict] = None, performance_ema_alpha: float = 0.1, shutdown_timeout: float = 5,
                 verbose: bool = False):
        self._parent_pid = os.getpid()
        client_mode = client_mode if client_mode is not None else dht.client_mode
        delay_optimizer_step = delay_optimizer_step if delay_optimizer_step is not None else delay_grad_averaging
        if offload_optimizer is None:
            offload_optimizer = params is not None and not use_local_updates
        allreduce_timeout = allreduce_timeout if allreduce_timeout is not None else averaging_timeout
        next_chunk_timeout = next_chunk_timeout if next_chunk_timeout is not None else matchmaking_time
        assert not delay_grad_averaging or delay_optimizer_step, "delay_grad_averaging requires delay_optimizer_step"
        assert not (client_mode and auxiliary), "Client-mode peers cannot serve as auxiliaries"
        assert not auxiliary or batch_size_per_step is None, "Auxiliary peers should not accumulate batches"
        if callable(optimizer) and params is not None:
            if scheduler is not None and (not callable(scheduler) or isinstance(scheduler, LRSchedulerBase)):
                raise ValueError("For this mode, please provide scheduler factory: callable(optimizer) -> scheduler")
        elif all(hasattr(optimizer, attr) for attr in ("param_groups", "step", "zero_grad")):
            if offload_optimizer or delay_optimizer_step or delay_grad_averaging:
                raise ValueError("To enable offload_optimizer or delayed updates, please initialize Optimizer as "
                                 "Optimizer(..., params=params, optimizer=lambda params: create_opt(params))")
        else:
            raise ValueError("Please initialize the optimizer in one of the following two ways:\n"
                             "(A) Optimizer(..., params=params, optimizer=lambda params: create_opt(params))\n"
                             "(B) Optimizer(..., optimizer=pre_initialized_optimizer)")
        if use_local_updates:
            assert not reuse_grad_buffers, "if local_updates is True, gradients will not be accumulated"
            assert not delay_grad_averaging, "if local_updates is True, gradients will not be averaged"
            assert grad_averager_factory is None, "if local_updates is True, grad_averager_factory will not be used"

        self.dht, self.run_id, self.client_mode, self.auxiliary = dht, run_id, client_mode, auxiliary
        self.batch_size_per_step, self.target_batch_size = batch_size_per_step, target_batch_size
        self.delay_state_averaging, self.average_state_every = delay_state_averaging, average_state_every
        self.matchmaking_time, self.offload_optimizer = matchmaking_time, offload_optimizer
        self.delay_grad_averaging, self.delay_optimizer_step = delay_grad_averaging, delay_optimizer_step
        self.averaging_timeout, self.allreduce_timeout = averaging_timeout, allreduce_timeout
        self.load_state_timeout, self.shutdown_timeout = load_state_timeout, shutdown_timeout
        self.next_chunk_timeout = next_chunk_timeout
        self.status_loglevel = logging.INFO if verbose else logging.DEBUG
        self.scheduled_grads: Optional[StepControl] = None
        self.scheduled_state: Optional[StepControl] = None

        self.tracker = self._make_progress_tracker(target_batch_size, performance_ema_alpha=performance_ema_alpha,
                                                   **tracker_opts or {})
        self.state_averager = self._make_state_averager(
            optimizer=optimizer, params=params, scheduler=scheduler,
            delta_rule_averaging=use_local_updates and self.delay_state_averaging,
            compression=state_averaging_compression, state_compression=load_state_compression,
            average_opt_statistics=average_opt_statistics, performance_ema_alpha=performance_ema_alpha,
            extra_tensors=extra_tensors, **averager_opts or {})
        if not use_local_updates:
            self.grad_averager = self._make_gradient_averager(grad_averager_factory, reuse_grad_buffers=reuse_grad_buffers,
                                                              compression=grad_compression, **averager_opts or {})
        else:
            self.grad_averager = None
        self._should_check_synchronization_on_update = True
        self._schema_hash = self._compute_schema_hash()
        self.delay_before_state_averaging = PerformanceEMA(alpha=performance_ema_alpha)
        self._step_supports_amp_scaling = reuse_grad_buffers  # torch AMP consults this flag
        # intentionally no super().__init__: this object delegates to the inner optimizer

    # ---------------------------------------------------------------------------------------------- factories
    def _make_state_averager(self, **kwargs) -> TrainingStateAverager:
        return TrainingStateAverager(
            dht=self.dht, prefix=f"{self.run_id}_state_averager", min_matchmaking_time=self.matchmaking_time,
            allreduce_timeout=self.allreduce_timeout, shutdown_timeout=self.shutdown_timeout,
            offload_optimizer=self.offload_optimizer, custom_gradients=self.offload_optimizer,
            status_loglevel=self.status_loglevel, next_chunk_timeout=self.next_chunk_timeout,
            client_mode=self.client_mode, auxiliary=self.auxiliary, start=True, **kwargs)

    def _make_gradient_averager(self, factory: Optional[GradientAveragerFactory], **kwargs) -> GradientAverager:
        assert hasattr(self, "state_averager"), "must initialize state averager first"
        factory = factory if factory is not None else GradientAverager
        grad_averager = factory(
            dht=self.dht, prefix=f"{self.run_id}_grad_averager", parameters=self.state_averager.main_parameters,
            min_matchmaking_time=self.matchmaking_time, allreduce_timeout=self.allreduce_timeout,
            shutdown_timeout=self.shutdown_timeout, next_chunk_timeout=self.next_chunk_timeout,
            client_mode=self.client_mode, auxiliary=self.auxiliary, start=True, **kwargs)
        if self.offload_optimizer:
            # the offloaded optimizer reads its gradients straight from the averaged-gradient buffers
            optimized_parameters = [param for group in self.state_averager.optimizer.param_groups for param in group["params"]]
            with grad_averager.get_tensors() as averaged_gradients:
                assert len(averaged_gradients) == len(optimized_parameters)
                for opt_param, averaged_grad in zip(optimized_parameters, averaged_gradients):
                    opt_param.grad = averaged_grad if averaged_grad.dtype == opt_param.dtype else None
                    if opt_param.grad is None:
                        opt_param.grad = averaged_grad.to(opt_param.dtype)
        return grad_averager

    def _make_progress_tracker(self, target_batch_size: int, **kwargs) -> ProgressTracker:
        return ProgressTracker(dht=self.dht, prefix=self.run_id, target_batch_size=target_batch_size,
                               client_mode=self.client_mode, status_loglevel=self.status_loglevel, start=True, **kwargs)

    def _compute_schema_hash(self) -> int:
        optimized_parameters = [param for group in self.state_averager.optimizer.param_groups for param in group["params"]]
        param_shapes = tuple(tuple(param.shape) for param in optimized_parameters)
        grad_ids = tuple(id(param.grad) for param in optimized_parameters) if self.offload_optimizer else None
        return hash((grad_ids, param_shapes))

    # ---------------------------------------------------------------------------------------------- status
    def is_alive(self) -> bool:
        return self.state_averager.is_alive()

    @property
    def local_epoch(self) -> int:
        """This peer's epoch; one epoch = ``target_batch_size`` samples across the swarm."""
        return self.state_averager.local_epoch

    @property
    def local_progress(self) -> LocalTrainingProgress:
        return self.tracker.local_progress

    @property
    def use_local_updates(self) -> bool:
        return self.grad_averager is None

    @property
    def use_gradient_averaging(self) -> bool:
        return self.grad_averager is not None

    # ---------------------------------------------------------------------------------------------- step
    def step(self, closure: Optional[Callable[[], torch.Tensor]] = None, batch_size: Optional[int] = None,
             grad_scaler: Optional[GradScaler] = None):
        """Register one more local batch; run or schedule whatever the swarm's progress calls for.

        Unlike a plain optimizer, most calls only accumulate gradients; the inner optimizer steps once per epoch.
        """
        if grad_scaler is not None and not isinstance(grad_scaler, GradScaler):
            raise ValueError("Optimizer requires a collaboration-aware gradient scaler (hivemind_b200.GradScaler)")
        if self.batch_size_per_step is None and batch_size is None and not self.auxiliary:
            raise ValueError("Please either set batch_size_per_step parameter at init or when calling .step")
        if self.auxiliary and (closure is not None or batch_size is not None or grad_scaler is not None):
            raise ValueError("Auxiliary peers should not have batch size, run closures, or use grad_scaler")
        batch_size = batch_size if batch_size is not None else self.batch_size_per_step

        self.state_averager.step(apply_delayed_updates=True)  # pick up finished background work
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()

        if not self.auxiliary and self._should_load_state_from_peers():
            logger.log(self.status_loglevel, "Peer is out of sync")
            self.load_state_from_peers()
            return loss  # gradients were computed with stale parameters: start the epoch over

        if self.use_gradient_averaging:
            if not self.auxiliary:
                if not self._check_and_accumulate_gradients(batch_size, grad_scaler):
                    return loss  # overflow: local gradients were dropped
            self._maybe_schedule_gradient_averaging()
            self._maybe_schedule_state_averaging()
        elif not self.auxiliary:
            if grad_scaler is not None:
                with grad_scaler.running_global_step():
                    assert grad_scaler.unscale_(self)
            new_samples_accumulated = self.tracker.local_progress.samples_accumulated + batch_size
            self.tracker.report_local_progress(self.local_epoch, new_samples_accumulated)
            self._maybe_schedule_state_averaging()
            self.state_averager.step(increment_epoch=False, optimizer_step=True,
                                     delay_optimizer_step=self.delay_optimizer_step, grad_scaler=grad_scaler)

        if self.tracker.ready_to_update_epoch:
            self._update_global_epoch(grad_scaler)
        return loss

    def _update_global_epoch(self, grad_scaler: Optional[GradScaler]) -> None:
        """The swarm reached the target batch: average gradients, step, maybe average state, start a new epoch."""
        assert self._schema_hash == self._compute_schema_hash(), "parameters or gradients changed during iteration"
        _epoch_start_time = time.perf_counter()
        with self.tracker.pause_updates():
            wait_for_trigger = None
            if self.use_gradient_averaging:
                logger.log(self.status_loglevel, f"Beginning optimizer step #{self.local_epoch}")
                if self.delay_optimizer_step:
                    self.state_averager.step(wait_for_delayed_updates=True)  # previous delayed update must be done
                began_averaging_gradients = self._begin_averaging_gradients(grad_scaler)
                if not began_averaging_gradients:
                    self.grad_averager.load_accumulators_into_averager_()  # step with local gradients
                elif self.delay_grad_averaging:
                    wait_for_trigger = partial(self._average_gradients_and_load_into_optimizer, self.scheduled_grads)
                else:
                    self._average_gradients_and_load_into_optimizer(self.scheduled_grads)

            next_epoch = max(self.local_epoch + 1, self.tracker.global_epoch)
            swarm_not_empty = self.tracker.global_progress.num_peers > 1
            should_perform_optimizer_step = not self.auxiliary and not self.use_local_updates
            should_average_state = (swarm_not_empty and next_epoch % self.average_state_every == 0
                                    and not self.state_averager.averaging_in_progress)
            if should_average_state and self.scheduled_state is not None:
                if self.scheduled_state.triggered or self.scheduled_state.done():
                    logger.log(self.status_loglevel, f"Not using pre-scheduled group for state averaging because it "
                                                     f"was already used elsewhere: {self.scheduled_state}")
                    self.scheduled_state = None
                self.delay_before_state_averaging.update(task_size=1, interval=time.perf_counter() - _epoch_start_time)

            self.state_averager.step(
                increment_epoch=True, wait_for_trigger=wait_for_trigger, optimizer_step=should_perform_optimizer_step,
                delay_optimizer_step=self.delay_optimizer_step and should_perform_optimizer_step,
                grad_scaler=grad_scaler, averaging_round=should_average_state,
                delay_averaging=self.delay_state_averaging and not self.auxiliary,
                averaging_control=self.scheduled_state if should_average_state else None,
                averaging_opts=dict(timeout=self.averaging_timeout) if should_average_state else None)

            if not should_average_state and self.scheduled_state is not None and not self.scheduled_state.done():
                self.scheduled_state.cancel()
            self.scheduled_state = None

            self.tracker.update_epoch(new_epoch=self.state_averager.local_epoch)
            self._should_check_synchronization_on_update = True
            if not self.client_mode:
                self.state_averager.state_sharing_priority = self.local_epoch
            if self.use_gradient_averaging and not self.auxiliary:
                self.grad_averager.reset_accumulated_grads_()
                if not self.client_mode:
                    self.grad_averager.state_sharing_priority = self.local_epoch
            logger.log(self.status_loglevel, f"Transitioning to epoch {self.local_epoch}")

    def _begin_averaging_gradients(self, grad_scaler: Optional[GradScaler]) -> bool:
        """Hand accumulated gradients to the averager and let the all-reduce begin (without waiting for it)."""
        if grad_scaler is not None:
            with grad_scaler.running_global_step():
                assert grad_scaler.unscale_(self)
        began_averaging_gradients = False
        if self.scheduled_grads is not None and (self.scheduled_grads.triggered or self.scheduled_grads.done()):
            logger.log(self.status_loglevel, f"Not using pre-scheduled group for gradient averaging because it "
                                             f"was already used elsewhere: {self.scheduled_grads}")
            self.scheduled_grads = None
        elif self.tracker.global_progress.num_peers > 1:
            try:
                self.scheduled_grads = self.grad_averager.step(control=self.scheduled_grads, reset_accumulators=True,
                                                               wait=False)
                began_averaging_gradients = True
            except BaseException as e:
                logger.exception(e)
        if not began_averaging_gradients and self.scheduled_grads is not None and not self.scheduled_grads.done():
            if self.tracker.global_progress.num_peers > 1:
                logger.log(self.status_loglevel, "Tagging along for a pre-scheduled gradient averaging round")
                self._tag_along_with_zero_weight(self.scheduled_grads)
            else:
                logger.log(self.status_loglevel, "Skipping pre-scheduled averaging round: there are no other peers")
                self._load_local_gradients_into_optimizer()
                self.scheduled_grads.cancel()
            self.scheduled_grads = None
        return began_averaging_gradients

    def _check_and_accumulate_gradients(self, batch_size: int, grad_scaler: Optional[GradScaler]) -> bool:
        assert not self.use_local_updates and not self.auxiliary
        if grad_scaler is not None and not grad_scaler.are_grads_finite(self):
            logger.log(self.status_loglevel, "Encountered incorrect value in fp16 grads, resetting local gradients")
            self.tracker.report_local_progress(self.local_epoch, samples_accumulated=0)
            self.grad_averager.reset_accumulated_grads_()
            return False
        self.grad_averager.accumulate_grads_(batch_size)
        self.tracker.report_local_progress(self.local_epoch, self.grad_averager.local_samples_accumulated)
        return True

    def _maybe_schedule_gradient_averaging(self) -> None:
        """Start matchmaking for gradients ``matchmaking_time`` before the epoch is expected to end."""
        assert self.use_gradient_averaging
        if self.tracker.estimated_next_update_time - get_dht_time() <= self.matchmaking_time:
            if self.scheduled_grads is None or self.scheduled_grads.triggered or self.scheduled_grads.done():
                eta_seconds = self.tracker.estimated_next_update_time - get_dht_time()
                eta_seconds = max(eta_seconds, self.grad_averager.matchmaking_kwargs["min_matchmaking_time"])
                logger.log(self.status_loglevel, f"Pre-scheduling gradient averaging round in {eta_seconds:.2f} sec")
                self.scheduled_grads = self.grad_averager.schedule_step(timeout=self.averaging_timeout)

    def _maybe_schedule_state_averaging(self) -> None:
        """Same for the parameter-averaging round, which begins a little after the epoch switch."""
        next_epoch = max(self.local_epoch + 1, self.tracker.global_epoch)
        if next_epoch % self.average_state_every != 0:
            return
        if self.state_averager.averaging_in_progress:
            return
        if self.delay_before_state_averaging.num_updates == 0:
            return  # no estimate yet of how long after the switch averaging starts
        estimated_time = self.tracker.estimated_next_update_time
        estimated_time += self.delay_before_state_averaging.ema_seconds_per_sample
        estimated_time += self.state_averager.delay_before_averaging.ema_seconds_per_sample
        eta_seconds_to_averaging = estimated_time - get_dht_time()
        if eta_seconds_to_averaging <= self.matchmaking_time:
            if self.scheduled_state is None or self.scheduled_state.triggered or self.scheduled_state.done():
                min_matchmaking_time = self.state_averager.matchmaking_kwargs["min_matchmaking_time"]
                actual_seconds = max(eta_seconds_to_averaging, min_matchmaking_time)
                logger.log(self.status_loglevel, f"Pre-scheduling state averaging round in {actual_seconds:.2f} sec")
                self.scheduled_state = self.state_averager.schedule_step(gather=next_epoch, timeout=self.averaging_timeout)

    def _average_gradients_and_load_into_optimizer(self, maybe_step_control: Optional[StepControl]) -> None:
        """Wait for the gradient round (this may run in the state averager's background thread)."""
        assert self.use_gradient_averaging and maybe_step_control is None or maybe_step_control.triggered
        averaged_gradients = False
        try:
            if maybe_step_control is not None:
                group_info = maybe_step_control.result(self.averaging_timeout)
                logger.log(self.status_loglevel, f"Averaged gradients with {len(group_info)} peers")
                self._load_averaged_gradients_into_optimizer_()
                averaged_gradients = True
            else:
                logger.log(self.status_loglevel, "Skipped averaging: there are no other peers")
        except BaseException as e:
            logger.log(self.status_loglevel, f"Averaging gradients failed with {e!r}")
        if not averaged_gradients:
            self._load_local_gradients_into_optimizer()

    def _load_averaged_gradients_into_optimizer_(self) -> None:
        assert self.use_gradient_averaging
        if not self.offload_optimizer:  # with offloading the optimizer already reads the averaged buffers
            optimized_parameters = [param for group in self.state_averager.optimizer.param_groups for param in group["params"]]
            with torch.no_grad(), self.grad_averager.get_tensors() as averaged_gradients:
                assert len(averaged_gradients) == len(optimized_parameters)
                for opt_param, averaged_grad in zip(optimized_parameters, averaged_gradients):
                    if opt_param.grad is None:
                        opt_param.grad = averaged_grad.to(opt_param.device, opt_param.dtype, copy=True)
                    else:
                        opt_param.grad.copy_(averaged_grad, non_blocking=True)
        self.grad_averager.notify_used_averaged_gradients()

    def _load_local_gradients_into_optimizer(self) -> None:
        """Fallback: use this peer's own accumulated gradients for the step."""
        logger.log(self.status_loglevel, "Proceeding with local gradients")
        self.grad_averager.load_accumulators_into_averager_()
        self._load_averaged_gradients_into_optimizer_()

    def zero_grad(self, set_to_none: bool = True):
        """Reset model gradients; forbidden with ``reuse_grad_buffers=True`` (accumulation lives in param.grad)."""
        if self.use_gradient_averaging and self.grad_averager.reuse_grad_buffers:
            raise ValueError(f"When running {self.__class__.__name__} with reuse_grad_buffers=True, user should never "
                             f"call zero_grad manually. Gradients will be refreshed internally")
        for param_group in self.param_groups:
            for param in param_group["params"]:
                if set_to_none:
                    param.grad = None
                elif param.grad is not None:
                    param.grad.zero_()

    # ---------------------------------------------------------------------------------------------- synchronisation
    def _should_load_state_from_peers(self) -> bool:
        """Out of sync if the epoch differs right after an epoch switch, or lags by more than one at other times
        (a lag of one means that the others have just switched and this peer is about to follow)."""
        if self._should_check_synchronization_on_update and self.tracker.fetched_global_progress_this_epoch.is_set():
            self._should_check_synchronization_on_update = False
            return self.local_epoch != self.tracker.global_epoch
        return self.local_epoch < self.tracker.global_epoch - 1

    def is_synchronized_with_peers(self) -> bool:
        return self.local_epoch >= self.tracker.global_epoch - 1

    def load_state_from_peers(self, **kwargs) -> None:
        """Download parameters, optimizer statistics, epoch and LR schedule position from the freshest peer."""
        if self.scheduled_grads is not None and not self.scheduled_grads.done():
            self._tag_along_with_zero_weight(self.scheduled_grads)  # do not leave the group one member short
            self.scheduled_grads = None
        self.state_averager.step(wait_for_delayed_updates=True)
        with self.tracker.pause_updates():
            while True:
                try:
                    self.state_averager.load_state_from_peers(timeout=self.load_state_timeout, **kwargs)
                    if self.grad_averager is not None:
                        self.grad_averager.load_state_from_peers(timeout=self.load_state_timeout, **kwargs)
                    break
                except KeyboardInterrupt:
                    raise
                except BaseException as e:
                    logger.exception(f"Failed to load state from peers: {e}, retrying ...")
                    continue
            if self.tracker.global_epoch - 1 <= self.local_epoch < self.tracker.global_epoch:
                logger.log(self.status_loglevel, f"Catching up with collaboration step {self.tracker.global_epoch}")
                self.state_averager.local_epoch = self.tracker.global_epoch
            self.tracker.report_local_progress(local_epoch=self.local_epoch, samples_accumulated=0)
            if not self.client_mode:
                self.state_averager.state_sharing_priority = self.local_epoch
            if self.use_gradient_averaging:
                self.grad_averager.reset_accumulated_grads_()
                if not self.client_mode:
                    self.grad_averager.state_sharing_priority = self.local_epoch

    # ---------------------------------------------------------------------------------------------- torch.optim API
    def state_dict(self) -> dict:
        state_dict = self.state_averager.optimizer.state_dict()
        state_dict["state"]["local_epoch"] = self.local_epoch
        return state_dict

    def load_state_dict(self, state_dict: dict):
        if "local_epoch" in state_dict["state"]:
            self.state_averager.local_epoch = state_dict["state"].pop("local_epoch")
        return self.state_averager.optimizer.load_state_dict(state_dict)

    @property
    def state(self):
        return dict(self.state_averager.optimizer.state, local_epoch=self.local_epoch)

    @property
    def opt(self) -> TorchOptimizer:
        return self.state_averager.optimizer

    @property
    def param_groups(self) -> ParamGroups:
        """The inner optimizer's groups, but listing the model's own parameters (not the offloaded copies)."""
        next_index = 0
        param_groups = tuple(dict(param_group) for param_group in self.state_averager.optimizer.param_groups)
        for param_group in param_groups:
            num_params = len(param_group["params"])
            param_group["params"] = self.state_averager.main_parameters[next_index:next_index + num_params]
            next_index += num_params
        assert next_index == len(self.state_averager.main_parameters)
        return param_groups

    def add_param_group(self, param_group: dict) -> None:
        raise ValueError(f"{self.__class__.__name__} does not support calling add_param_group after creation. "
                         f"Please provide all parameter groups at init")

    def __repr__(self):
        return f"{self.__class__.__name__}(prefix={self.run_id}, epoch={self.local_epoch})"

    def _tag_along_with_zero_weight(self, control: StepControl) -> None:
        """Take part in a round we no longer need, with zero weight, so that groupmates are not kept waiting."""
        if not control.triggered:
            control.weight = 0
            control.allow_allreduce()
        if not control.done():
            try:
                control.result(self.averaging_timeout)
            except BaseException as e:
                logger.exception(e)
                if not control.done():
                    control.cancel()

    def shutdown(self):
        logger.log(self.status_loglevel, "Sending goodbye to peers...")
        self.tracker.shutdown(self.shutdown_timeout)
        self.state_averager.step(wait_for_delayed_updates=True)
        for scheduled_round in self.scheduled_grads, self.scheduled_state:
            if scheduled_round is not None:
                if scheduled_round.stage == AveragingStage.LOOKING_FOR_GROUP:
                    scheduled_round.cancel()
                else:
                    self._tag_along_with_zero_weight(scheduled_round)
        logger.log(self.status_loglevel, "Shutting down averagers...")
        self.state_averager.shutdown()
        if self.use_gradient_averaging:
            self.grad_averager.shutdown()
        logger.log(self.status_loglevel, f"{self.__class__.__name__} is shut down")

    def __del__(self):
        try:
            if self._parent_pid == os.getpid() and self.is_alive():
                self.shutdown()
        except Exception:
            pass

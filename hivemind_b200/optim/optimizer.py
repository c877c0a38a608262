"""``hivemind_b200.Optimizer``: wraps a PyTorch optimizer for collaborative large-batch training.

Peers accumulate gradients locally; once the swarm as a whole has processed ``target_batch_size`` samples (an
*epoch*), peers average gradients in a matched group, run the same optimizer step, and optionally average
parameters. Modes (behaviour contract: hivemind/optim/optimizer.py:32-790): synchronous; delayed parameter updates
(``delay_optimizer_step`` / ``delay_grad_averaging`` / ``delay_state_averaging``: communication and the optimizer
step overlap with the next epoch's computation); local updates with periodic state averaging
(``use_local_updates``); client-mode and auxiliary peers. Any averaging failure degrades to a local step; a peer
that falls behind downloads the state from others. ``state_dict()`` is the inner optimizer's state dict plus
``state["local_epoch"]``.

On a B200 box every peer is one GPU: gradient accumulators, averaged gradients, master weights and optimizer
statistics stay in HBM, are averaged by the device butterfly over NVLink, and the per-parameter loops are fused
multi-tensor kernels.

Structure of this file: ``_Prescheduled`` looks after one matchmaking round that was started ahead of time (for
gradients, for state); ``Optimizer.step`` books the batch, keeps those rounds scheduled, and calls
``_close_epoch`` when the swarm has reached the target batch.
"""
from __future__ import annotations

import logging
import os
import time
from typing import Callable, List, Optional, Sequence, Union

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


class _Prescheduled:
    """A slot for one averaging round whose matchmaking starts before the data is ready.

    The slot is *usable* while its round has neither been triggered nor finished; a round that turns out not to be
    needed is either cancelled (still looking for a group) or seen through with weight zero, so that the groupmates
    that already count on this peer are not left one member short.
    """

    def __init__(self, what: str, timeout: Optional[float], loglevel: int):
        self.what, self.timeout, self.loglevel = what, timeout, loglevel
        self.control: Optional[StepControl] = None

    @property
    def usable(self) -> bool:
        return self.control is not None and not (self.control.triggered or self.control.done())

    def take(self) -> Optional[StepControl]:
        """Hand the round over (the slot becomes empty); a round that is no longer usable is dropped instead."""
        control, self.control = self.control, None
        if control is not None and (control.triggered or control.done()):
            logger.log(self.loglevel, f"The pre-scheduled {self.what} round was already used elsewhere: {control}")
            return None
        return control

    def retire(self) -> None:
        """Get rid of the round without harming its group."""
        control, self.control = self.control, None
        if control is None or control.done():
            return
        if control.stage == AveragingStage.LOOKING_FOR_GROUP and not control.triggered:
            control.cancel()
        else:
            ride_along_with_zero_weight(control, self.timeout)


def ride_along_with_zero_weight(control: StepControl, timeout: Optional[float]) -> None:
    """Take part in a round this peer has nothing to contribute to: weight zero, wait for it to end."""
    if not control.triggered:
        control.weight = 0
        control.allow_allreduce()
    if control.done():
        return
    try:
        control.result(timeout)
    except BaseException as e:
        logger.debug(f"a zero-weight round ended with {e!r}")
        if not control.done():
            control.cancel()


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
        # intentionally no super().__init__: this object delegates to the inner optimizer
        self._owner_pid = os.getpid()
        if client_mode is None:
            client_mode = dht.client_mode
        if delay_optimizer_step is None:
            delay_optimizer_step = delay_grad_averaging
        if offload_optimizer is None:
            offload_optimizer = params is not None and not use_local_updates
        self._check_arguments(optimizer, params, scheduler, offload_optimizer, delay_optimizer_step, delay_grad_averaging,
                              use_local_updates, reuse_grad_buffers, grad_averager_factory, client_mode, auxiliary,
                              batch_size_per_step)

        self.dht, self.run_id = dht, run_id
        self.client_mode, self.auxiliary = client_mode, auxiliary
        self.target_batch_size, self.batch_size_per_step = target_batch_size, batch_size_per_step
        self.matchmaking_time, self.averaging_timeout = matchmaking_time, averaging_timeout
        self.allreduce_timeout = averaging_timeout if allreduce_timeout is None else allreduce_timeout
        self.next_chunk_timeout = matchmaking_time if next_chunk_timeout is None else next_chunk_timeout
        self.load_state_timeout, self.shutdown_timeout = load_state_timeout, shutdown_timeout
        self.offload_optimizer = offload_optimizer
        self.delay_optimizer_step, self.delay_grad_averaging = delay_optimizer_step, delay_grad_averaging
        self.delay_state_averaging, self.average_state_every = delay_state_averaging, average_state_every
        self.status_loglevel = logging.INFO if verbose else logging.DEBUG
        self._grads_round = _Prescheduled("gradient averaging", averaging_timeout, self.status_loglevel)
        self._state_round = _Prescheduled("state averaging", averaging_timeout, self.status_loglevel)

        shared = dict(min_matchmaking_time=matchmaking_time, allreduce_timeout=self.allreduce_timeout,
                      shutdown_timeout=shutdown_timeout, next_chunk_timeout=self.next_chunk_timeout,
                      client_mode=client_mode, auxiliary=auxiliary, start=True)
        self.tracker = self._make_progress_tracker(target_batch_size, performance_ema_alpha=performance_ema_alpha,
                                                   **(tracker_opts or {}))
        self.state_averager = self._make_state_averager(
            optimizer=optimizer, params=params, scheduler=scheduler, compression=state_averaging_compression,
            state_compression=load_state_compression, average_opt_statistics=average_opt_statistics,
            delta_rule_averaging=use_local_updates and delay_state_averaging, extra_tensors=extra_tensors,
            performance_ema_alpha=performance_ema_alpha, **shared, **(averager_opts or {}))
        self.grad_averager: Optional[GradientAverager] = None
        if not use_local_updates:
            self.grad_averager = self._make_gradient_averager(
                grad_averager_factory, reuse_grad_buffers=reuse_grad_buffers, compression=grad_compression,
                **shared, **(averager_opts or {}))
        self._verify_sync_after_switch = True
        self._layout_fingerprint = self._fingerprint()
        self.delay_before_state_averaging = PerformanceEMA(alpha=performance_ema_alpha)
        self._step_supports_amp_scaling = reuse_grad_buffers  # torch AMP consults this flag

    @staticmethod
    def _check_arguments(optimizer, params, scheduler, offload, delay_step, delay_grads, local_updates, reuse_grads,
                         grad_factory, client_mode, auxiliary, batch_size_per_step) -> None:
        if delay_grads and not delay_step:
            raise ValueError("delay_grad_averaging requires delay_optimizer_step")
        if client_mode and auxiliary:
            raise ValueError("a client-mode peer cannot be an auxiliary")
        if auxiliary and batch_size_per_step is not None:
            raise ValueError("auxiliary peers process no batches")
        made_here = callable(optimizer) and not isinstance(optimizer, TorchOptimizer) and params is not None
        ready_made = all(hasattr(optimizer, name) for name in ("param_groups", "step", "zero_grad"))
        if made_here:
            if scheduler is not None and (isinstance(scheduler, LRSchedulerBase) or not callable(scheduler)):
                raise ValueError("with an optimizer factory, pass a scheduler factory: optimizer -> scheduler")
        elif ready_made:
            if offload or delay_step or delay_grads:
                raise ValueError("offloading and delayed updates need Optimizer(..., params=params, "
                                 "optimizer=lambda params: make_optimizer(params))")
        else:
            raise ValueError("pass either (params=..., optimizer=factory) or optimizer=an_initialised_optimizer")
        if local_updates and (reuse_grads or delay_grads or grad_factory is not None):
            raise ValueError("use_local_updates neither accumulates nor averages gradients: reuse_grad_buffers, "
                             "delay_grad_averaging and grad_averager_factory do not apply")

    # ---------------------------------------------------------------------------------------------- factories
    def _make_progress_tracker(self, target_batch_size: int, **kwargs) -> ProgressTracker:
        return ProgressTracker(dht=self.dht, prefix=self.run_id, target_batch_size=target_batch_size,
                               client_mode=self.client_mode, status_loglevel=self.status_loglevel, start=True, **kwargs)

    def _make_state_averager(self, **kwargs) -> TrainingStateAverager:
        return TrainingStateAverager(dht=self.dht, prefix=f"{self.run_id}_state_averager",
                                     offload_optimizer=self.offload_optimizer, custom_gradients=self.offload_optimizer,
                                     status_loglevel=self.status_loglevel, **kwargs)

    def _make_gradient_averager(self, factory: Optional[GradientAveragerFactory], **kwargs) -> GradientAverager:
        factory = GradientAverager if factory is None else factory
        averager = factory(dht=self.dht, prefix=f"{self.run_id}_grad_averager",
                           parameters=self.state_averager.main_parameters, **kwargs)
        if self.offload_optimizer:
            # the offloaded optimizer reads its gradients straight out of the averaged-gradient buffers
            with averager.get_tensors() as averaged:
                shadow = self._inner_parameters()
                if len(shadow) != len(averaged):
                    raise RuntimeError("gradient averager and optimizer disagree about the parameters")
                for p, g in zip(shadow, averaged):
                    p.grad = g if g.dtype == p.dtype else g.to(p.dtype)
        return averager

    def _inner_parameters(self) -> List[torch.Tensor]:
        return [p for group in self.state_averager.optimizer.param_groups for p in group["params"]]

    def _fingerprint(self) -> int:
        """Changes if somebody swaps parameters or (with offloading) the gradient buffers behind our back."""
        inner = self._inner_parameters()
        buffers = tuple(id(p.grad) for p in inner) if self.offload_optimizer else None
        return hash((buffers, tuple(tuple(p.shape) for p in inner)))

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

    @property
    def scheduled_grads(self) -> Optional[StepControl]:
        return self._grads_round.control

    @property
    def scheduled_state(self) -> Optional[StepControl]:
        return self._state_round.control

    def _next_epoch(self) -> int:
        return max(self.local_epoch + 1, self.tracker.global_epoch)

    def _swarm_has_others(self) -> bool:
        return self.tracker.global_progress.num_peers > 1

    # ---------------------------------------------------------------------------------------------- step
    def step(self, closure: Optional[Callable[[], torch.Tensor]] = None, batch_size: Optional[int] = None,
             grad_scaler: Optional[GradScaler] = None):
        """Register one more local batch; run or schedule whatever the swarm's progress calls for.

        Unlike a plain optimizer, most calls only accumulate gradients; the inner optimizer steps once per epoch.
        """
        if grad_scaler is not None and not isinstance(grad_scaler, GradScaler):
            raise ValueError("loss scaling needs hivemind_b200.GradScaler, which knows about collaborative steps")
        if self.auxiliary:
            if closure is not None or batch_size is not None or grad_scaler is not None:
                raise ValueError("auxiliary peers take no closure, batch size or gradient scaler")
        else:
            batch_size = self.batch_size_per_step if batch_size is None else batch_size
            if batch_size is None:
                raise ValueError("set batch_size_per_step at construction or pass batch_size to step()")

        self.state_averager.step(apply_delayed_updates=True)  # adopt whatever finished in the background
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()

        if not self.auxiliary and self._fell_behind():
            logger.log(self.status_loglevel, "This peer is out of sync with the swarm")
            self.load_state_from_peers()
            return loss  # these gradients belong to stale parameters: the epoch starts over

        if self.use_gradient_averaging:
            if not self.auxiliary and not self._book_gradients(batch_size, grad_scaler):
                return loss  # overflow in scaled gradients: the batch was dropped
            self._keep_gradient_round_scheduled()
            self._keep_state_round_scheduled()
        elif not self.auxiliary:
            if grad_scaler is not None:
                with grad_scaler.running_global_step():
                    if not grad_scaler.unscale_(self):
                        raise RuntimeError("the gradient scaler refused to unscale")
            self.tracker.report_local_progress(self.local_epoch, self.local_progress.samples_accumulated + batch_size)
            self._keep_state_round_scheduled()
            self.state_averager.step(increment_epoch=False, optimizer_step=True,
                                     delay_optimizer_step=self.delay_optimizer_step, grad_scaler=grad_scaler)

        if self.tracker.ready_to_update_epoch:
            self._close_epoch(grad_scaler)
        return loss

    def _book_gradients(self, batch_size: int, grad_scaler: Optional[GradScaler]) -> bool:
        if grad_scaler is not None and not grad_scaler.are_grads_finite(self):
            logger.log(self.status_loglevel, "Non-finite scaled gradients: this epoch's local gradients are discarded")
            self.tracker.report_local_progress(self.local_epoch, samples_accumulated=0)
            self.grad_averager.reset_accumulated_grads_()
            return False
        self.grad_averager.accumulate_grads_(batch_size)
        self.tracker.report_local_progress(self.local_epoch, self.grad_averager.local_samples_accumulated)
        return True

    def _keep_gradient_round_scheduled(self) -> None:
        """Matchmaking for gradients starts ``matchmaking_time`` before the epoch is expected to end."""
        time_left = self.tracker.estimated_next_update_time - get_dht_time()
        if time_left > self.matchmaking_time or self._grads_round.usable:
            return
        eta = max(time_left, self.grad_averager.matchmaking_kwargs["min_matchmaking_time"])
        logger.log(self.status_loglevel, f"Looking for a gradient averaging group; the epoch should end in {eta:.2f} s")
        self._grads_round.control = self.grad_averager.schedule_step(timeout=self.averaging_timeout)

    def _keep_state_round_scheduled(self) -> None:
        """Same for parameter averaging, which begins a little after the epoch switch."""
        next_epoch = self._next_epoch()
        if next_epoch % self.average_state_every != 0 or self.state_averager.averaging_in_progress:
            return
        if self.delay_before_state_averaging.num_updates == 0:
            return  # no estimate yet of how long after the switch the round begins
        begins_at = (self.tracker.estimated_next_update_time + self.delay_before_state_averaging.ema_seconds_per_sample
                     + self.state_averager.delay_before_averaging.ema_seconds_per_sample)
        time_left = begins_at - get_dht_time()
        if time_left > self.matchmaking_time or self._state_round.usable:
            return
        eta = max(time_left, self.state_averager.matchmaking_kwargs["min_matchmaking_time"])
        logger.log(self.status_loglevel, f"Looking for a state averaging group; averaging should begin in {eta:.2f} s")
        self._state_round.control = self.state_averager.schedule_step(gather=next_epoch, timeout=self.averaging_timeout)

    # ---------------------------------------------------------------------------------------------- epoch switch
    def _close_epoch(self, grad_scaler: Optional[GradScaler]) -> None:
        """The swarm reached the target batch: average gradients, step, maybe average state, begin the next epoch."""
        if self._layout_fingerprint != self._fingerprint():
            raise RuntimeError("parameters or gradient buffers were replaced while training was running")
        began = time.perf_counter()
        with self.tracker.pause_updates():
            gradients_arrive_later = None
            if self.use_gradient_averaging:
                logger.log(self.status_loglevel, f"Optimizer step {self.local_epoch} begins")
                if self.delay_optimizer_step:
                    self.state_averager.step(wait_for_delayed_updates=True)  # the previous delayed update is over
                round_in_flight = self._start_gradient_round(grad_scaler)
                if round_in_flight is None:
                    self.grad_averager.load_accumulators_into_averager_()  # local gradients it is
                elif self.delay_grad_averaging:
                    def gradients_arrive_later(control=round_in_flight):
                        self._finish_gradient_round(control)
                else:
                    self._finish_gradient_round(round_in_flight)

            next_epoch = self._next_epoch()
            step_now = not self.auxiliary and not self.use_local_updates
            average_state = (self._swarm_has_others() and next_epoch % self.average_state_every == 0
                             and not self.state_averager.averaging_in_progress)
            state_control = None
            if average_state:
                state_control = self._state_round.take()
                self.delay_before_state_averaging.update(task_size=1, interval=time.perf_counter() - began)
            self.state_averager.step(
                increment_epoch=True, wait_for_trigger=gradients_arrive_later, optimizer_step=step_now,
                delay_optimizer_step=self.delay_optimizer_step and step_now, grad_scaler=grad_scaler,
                averaging_round=average_state, delay_averaging=self.delay_state_averaging and not self.auxiliary,
                averaging_control=state_control, averaging_opts=dict(timeout=self.averaging_timeout) if average_state else None)
            if not average_state:
                self._state_round.retire()

            self.tracker.update_epoch(new_epoch=self.state_averager.local_epoch)
            self._verify_sync_after_switch = True
            self._announce_priority()
            if self.use_gradient_averaging and not self.auxiliary:
                self.grad_averager.reset_accumulated_grads_()
            logger.log(self.status_loglevel, f"Epoch {self.local_epoch} begins")

    def _announce_priority(self) -> None:
        """Newcomers download state from whoever is furthest along."""
        if self.client_mode:
            return
        self.state_averager.state_sharing_priority = self.local_epoch
        if self.use_gradient_averaging and not self.auxiliary:
            self.grad_averager.state_sharing_priority = self.local_epoch

    def _start_gradient_round(self, grad_scaler: Optional[GradScaler]) -> Optional[StepControl]:
        """Hand the accumulated gradients to the averager and let the all-reduce begin; returns the round in flight,
        or None if this epoch's step uses local gradients."""
        if grad_scaler is not None:
            with grad_scaler.running_global_step():
                if not grad_scaler.unscale_(self):
                    raise RuntimeError("the gradient scaler refused to unscale")
        had_round = self._grads_round.control is not None
        control = self._grads_round.take()
        if had_round and control is None:
            return None  # the round was spent elsewhere (e.g. while catching up): no second attempt this epoch
        if self._swarm_has_others():
            try:
                return self.grad_averager.step(control=control, reset_accumulators=True, wait=False)
            except BaseException as e:
                logger.exception(e)
        if control is not None and not control.done():
            if self._swarm_has_others():
                logger.log(self.status_loglevel, "Seeing the pre-scheduled gradient round through with zero weight")
                ride_along_with_zero_weight(control, self.averaging_timeout)
            else:
                logger.log(self.status_loglevel, "Nobody else is training: the pre-scheduled round is cancelled")
                self._use_local_gradients()
                control.cancel()
        return None

    def _finish_gradient_round(self, control: StepControl) -> None:
        """Wait for the gradient round (possibly on the state averager's worker thread) and feed the optimizer."""
        try:
            group = control.result(self.averaging_timeout)
            logger.log(self.status_loglevel, f"Averaged gradients with {len(group)} peers")
            self._feed_averaged_gradients()
        except BaseException as e:
            logger.log(self.status_loglevel, f"Gradient averaging failed: {e!r}")
            self._use_local_gradients()

    def _feed_averaged_gradients(self) -> None:
        if not self.offload_optimizer:  # with offloading the optimizer's .grad ARE the averaged buffers
            with torch.no_grad(), self.grad_averager.get_tensors() as averaged:
                inner = self._inner_parameters()
                if len(inner) != len(averaged):
                    raise RuntimeError("gradient averager and optimizer disagree about the parameters")
                for p, g in zip(inner, averaged):
                    if p.grad is None:
                        p.grad = g.to(p.device, p.dtype, copy=True)
                    else:
                        p.grad.copy_(g, non_blocking=True)
        self.grad_averager.notify_used_averaged_gradients()

    def _use_local_gradients(self) -> None:
        logger.log(self.status_loglevel, "This step uses the peer's own gradients")
        self.grad_averager.load_accumulators_into_averager_()
        self._feed_averaged_gradients()

    def zero_grad(self, set_to_none: bool = True):
        """Reset model gradients; forbidden with ``reuse_grad_buffers=True`` (accumulation lives in param.grad)."""
        if self.use_gradient_averaging and self.grad_averager.reuse_grad_buffers:
            raise ValueError("with reuse_grad_buffers=True the optimizer clears gradients itself; do not call zero_grad")
        for group in self.param_groups:
            for p in group["params"]:
                if set_to_none:
                    p.grad = None
                elif p.grad is not None:
                    p.grad.zero_()

    # ---------------------------------------------------------------------------------------------- synchronisation
    def _fell_behind(self) -> bool:
        """Right after an epoch switch the epochs must agree; otherwise a lag of one is normal (the others have just
        switched and this peer is about to), more than one is not."""
        if self._verify_sync_after_switch and self.tracker.fetched_global_progress_this_epoch.is_set():
            self._verify_sync_after_switch = False
            return self.local_epoch != self.tracker.global_epoch
        return self.local_epoch < self.tracker.global_epoch - 1

    def is_synchronized_with_peers(self) -> bool:
        return self.local_epoch >= self.tracker.global_epoch - 1

    def load_state_from_peers(self, **kwargs) -> None:
        """Download parameters, optimizer statistics, epoch and LR schedule position from the freshest peer."""
        self._grads_round.retire()
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
                    logger.exception(f"Downloading the state failed ({e!r}); trying again")
            if self.local_epoch == self.tracker.global_epoch - 1:
                logger.log(self.status_loglevel, f"Joining the swarm at epoch {self.tracker.global_epoch}")
                self.state_averager.local_epoch = self.tracker.global_epoch
            self.tracker.report_local_progress(local_epoch=self.local_epoch, samples_accumulated=0)
            self._announce_priority()
            if self.use_gradient_averaging:
                self.grad_averager.reset_accumulated_grads_()

    # ---------------------------------------------------------------------------------------------- torch.optim API
    def state_dict(self) -> dict:
        state = self.state_averager.optimizer.state_dict()
        state["state"]["local_epoch"] = self.local_epoch
        return state

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
        model, cursor, groups = self.state_averager.main_parameters, 0, []
        for inner in self.state_averager.optimizer.param_groups:
            count = len(inner["params"])
            groups.append(dict(inner, params=model[cursor:cursor + count]))
            cursor += count
        if cursor != len(model):
            raise RuntimeError("the optimizer's parameter groups changed during training")
        return tuple(groups)

    def add_param_group(self, param_group: dict) -> None:
        raise ValueError(f"{type(self).__name__} takes all of its parameter groups at construction")

    def __repr__(self):
        return f"{type(self).__name__}(prefix={self.run_id}, epoch={self.local_epoch})"

    def shutdown(self):
        logger.log(self.status_loglevel, "Leaving the swarm")
        self.tracker.shutdown(self.shutdown_timeout)
        self.state_averager.step(wait_for_delayed_updates=True)
        self._grads_round.retire()
        self._state_round.retire()
        self.state_averager.shutdown()
        if self.grad_averager is not None:
            self.grad_averager.shutdown()
        logger.log(self.status_loglevel, f"{type(self).__name__} has shut down")

    def __del__(self):
        try:
            if self._owner_pid == os.getpid() and self.is_alive():
                self.shutdown()
        except Exception:
            pass

"""``GradientAverager``: accumulates local gradients over micro-batches and averages them with peers.

Three sets of buffers, as in the reference (hivemind/optim/grad_averager.py:18-239):
 (1) ``param.grad`` of the model, (2) local accumulators (or (1) itself with ``reuse_grad_buffers=True``),
 (3) the averaged tensors that take part in all-reduce.
Differences by design: (3) lives on the parameters' device — for CUDA models in a peer-mappable fp32 arena that the
device butterfly averages in place — and accumulate / scale / zero are single multi-tensor kernels
(``ops/csrc/multi_tensor.cu``) instead of per-parameter loops with a device-to-host copy.
"""
from __future__ import annotations

import contextlib
from typing import Iterable, Iterator, Optional, Sequence

import torch

from hivemind_b200.averaging import DecentralizedAverager, StepControl
from hivemind_b200.dht import DHT
from hivemind_b200.ops import multi_tensor as mt
from hivemind_b200.utils import DHTExpiration, get_logger

logger = get_logger(__name__)
TGradientAverager = "GradientAverager"


class GradientAverager(DecentralizedAverager):
    """
    :param parameters: parameters whose gradients are averaged
    :param dht: a running DHT
    :param prefix: averager namespace (unique per run and per tensor set)
    :param reuse_grad_buffers: accumulate directly in ``param.grad`` (the user must not zero grads between
      micro-batches) instead of separate accumulators
    :param accumulate_grads_on: device of the separate accumulators (default: same as the gradients)
    :param client_mode: send-only peer
    :param warn: warn when averaged gradients are overwritten before being used
    :param averaged_grads: pre-allocated buffers for the averaged gradients (default: allocated here)
    :param kwargs: forwarded to ``DecentralizedAverager``
    """

    def __init__(self, parameters: Iterable[torch.nn.Parameter], *, dht: DHT, prefix: str,
                 reuse_grad_buffers: bool = False, accumulate_grads_on: Optional[torch.device] = None,
                 client_mode: bool = None, warn: bool = True, averaged_grads: Sequence[torch.Tensor] = (), **kwargs):
        if reuse_grad_buffers and accumulate_grads_on is not None:
            logger.warning("Setting 'accumulate_grads_on' has no effect if reuse_grad_buffers=True")
        client_mode = client_mode if client_mode is not None else dht.client_mode
        self.parameters = tuple(parameters)
        self.reuse_grad_buffers = reuse_grad_buffers
        self.warn = warn
        self.local_samples_accumulated = 0
        self.local_times_accumulated = 0
        self._anchor_batch_size = None
        self._local_accumulators = None
        if not reuse_grad_buffers:
            self._local_accumulators = tuple(torch.zeros_like(grad, dtype=torch.float32, device=accumulate_grads_on)
                                             for grad in self._grads_from_parameters())
        self._accumulators_used_in_step = False
        self._new_averaged_grads = False
        with torch.no_grad():
            if not averaged_grads:
                averaged_grads = tuple(torch.zeros_like(grad, dtype=torch.float32) for grad in self._grads_from_parameters())
            elif any(param_grad.size() != grad.size() for param_grad, grad in zip(self._grads_from_parameters(), averaged_grads)):
                raise ValueError("Averaged gradients don't have same shape as gradients from parameters")
        super().__init__(averaged_tensors=averaged_grads, dht=dht, prefix=prefix, client_mode=client_mode, **kwargs)

    def _grads_from_parameters(self) -> Iterator[torch.Tensor]:
        """Gradient buffers of the parameters (created as zeros where missing)."""
        for param in self.parameters:
            if param.grad is None:
                param.grad = torch.zeros_like(param)
            yield param.grad

    @torch.no_grad()
    def _grad_accumulators(self) -> Iterator[torch.Tensor]:
        assert (self._local_accumulators is None) == self.reuse_grad_buffers
        yield from self._grads_from_parameters() if self.reuse_grad_buffers else self._local_accumulators

    @torch.no_grad()
    def accumulate_grads_(self, batch_size: int) -> None:
        """Add the current ``param.grad`` (a mean over ``batch_size`` samples) to the accumulators.

        Micro-batches are weighted by their size relative to the first one after a reset, so the accumulated
        value stays a sample-weighted sum in units of the first batch.
        """
        if self._accumulators_used_in_step and self.warn:
            logger.warning("[warn=True] Gradient accumulators were not reset since the last averaging round. Please "
                           "call .reset_accumulated_grads_ after every step or use .step(reset_accumulators=True)")
            self._accumulators_used_in_step = False  # warn once per round
        if self._anchor_batch_size is None:
            self._anchor_batch_size = batch_size  # remember the first batch size to scale the rest
        self.local_samples_accumulated += batch_size
        self.local_times_accumulated += 1
        if self.reuse_grad_buffers:
            pass  # autograd already added this micro-batch to param.grad
        else:
            alpha = float(batch_size) / self._anchor_batch_size
            grads = list(self._grads_from_parameters())
            accs = list(self._grad_accumulators())
            same_device = all(a.device == g.device for a, g in zip(accs, grads))
            if same_device:
                mt.axpy_(accs, grads, alpha)
            else:
                for acc, grad in zip(accs, grads):
                    acc.add_(grad.to(acc.device, acc.dtype), alpha=alpha)

    def schedule_step(self, scheduled_time: Optional[DHTExpiration] = None, **kwargs) -> StepControl:
        """Begin matchmaking ahead of time; pass the returned control to ``step`` when gradients are ready."""
        assert kwargs.get("weight") is None, "setting weight in schedule_step is not supported"
        return super().step(scheduled_time=scheduled_time, wait=False, require_trigger=True, **kwargs)

    def step(self, weight: Optional[float] = None, reset_accumulators: bool = True,
             control: Optional[StepControl] = None, timeout: Optional[float] = None, wait: bool = True, **kwargs):
        """Average the accumulated gradients with peers.

        :param weight: averaging weight (default: number of locally accumulated samples)
        :param reset_accumulators: zero the accumulators once they are loaded into the averager
        :param control: a pre-scheduled step from ``schedule_step``
        :param wait: block until the round is finished
        """
        if control is None:
            control = self.schedule_step(timeout=timeout, **kwargs)
        elif len(kwargs) > 0:
            raise RuntimeError(f"Averaging with a pre-scheduled group, parameters {kwargs} will have no effect")
        assert not control.triggered, f"This {type(control)} instance was already used"
        if self._new_averaged_grads and self.warn:
            logger.warning("[warn=True] Starting new averaging round, but previous round results were not used. "
                           "This may be a sign of incorrect optimizer behavior")
        self.load_accumulators_into_averager_()
        self._accumulators_used_in_step = True
        self._new_averaged_grads = True
        control.weight = self.local_samples_accumulated if weight is None else weight
        if reset_accumulators:
            self.reset_accumulated_grads_()
        control.allow_allreduce()
        return control.result(timeout) if wait else control

    @torch.no_grad()
    def load_accumulators_into_averager_(self) -> None:
        """averaged_grads = accumulators / number of accumulated micro-batches (one fused kernel on GPU)."""
        if self.local_times_accumulated == 0:
            logger.warning("Averaging gradients before accumulating any; averaged gradients are zeros")
        grad_scale = (1.0 / self.local_times_accumulated) if self.local_times_accumulated != 0 else 0.0
        with self.get_tensors() as averaged_grads:
            accs = list(self._grad_accumulators())
            if all(a.device == g.device for a, g in zip(accs, averaged_grads)):
                mt.scale_copy_(list(averaged_grads), accs, grad_scale)
            else:
                for grad_acc, averaged_grad in zip(accs, averaged_grads):
                    averaged_grad.copy_(grad_acc.to(averaged_grad.device, averaged_grad.dtype) * grad_scale)

    @torch.no_grad()
    def reset_accumulated_grads_(self) -> None:
        self._accumulators_used_in_step = False
        self.local_samples_accumulated = self.local_times_accumulated = 0
        self._anchor_batch_size = None
        mt.zero_(list(self._grad_accumulators()))

    @contextlib.contextmanager
    @torch.no_grad()
    def use_averaged_gradients(self):
        """Temporarily point ``param.grad`` at the averaged gradients (for the inner optimizer's step)."""
        self._new_averaged_grads = False
        with self.get_tensors() as averaged_grads:
            assert len(averaged_grads) == len(self.parameters)
            old_grads = [param.grad for param in self.parameters]
            try:
                for param, new_grad in zip(self.parameters, averaged_grads):
                    if new_grad.device == param.device and new_grad.dtype == param.dtype:
                        param.grad = new_grad
                    else:
                        param.grad = new_grad.to(param.device, param.dtype)
                yield averaged_grads
            finally:
                for param, old_grad in zip(self.parameters, old_grads):
                    param.grad = old_grad

    def notify_used_averaged_gradients(self) -> None:
        """Tell the averager that the results were consumed through ``get_tensors`` directly."""
        self._new_averaged_grads = False

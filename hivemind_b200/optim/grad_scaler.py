"""Loss scaling that cooperates with ``Optimizer(reuse_grad_buffers=True)``.

With gradients accumulated in ``param.grad`` across micro-batches, the usual AMP routine (unscale, step, update after
every backward) would unscale partially accumulated gradients. This scaler (behaviour of
hivemind/optim/grad_scaler.py:25-127): unscales only inside a global step, lets the scale grow only right after a
global step (it still shrinks on overflow at any time), and allows low-precision master parameters.
"""
from __future__ import annotations

import contextlib
import threading
from copy import deepcopy
from typing import Dict, Optional

import torch
from torch.amp.grad_scaler import GradScaler as TorchGradScaler
from torch.amp.grad_scaler import OptState, _refresh_per_optimizer_state
from torch.optim import Optimizer as TorchOptimizer

from hivemind_b200.utils.logging import get_logger

logger = get_logger(__name__)


class GradScaler(TorchGradScaler):
    """See the module docstring. State on top of torch's scaler:

    * ``_inside_global_step`` - set by ``running_global_step()``; only then are gradients really unscaled and the
      wrapped optimizer really stepped through the scaler;
    * ``_stepped`` - a global step went through since the last ``update()``: the scale may grow;
    * ``_handover`` - torch keys its per-optimizer records by ``id(optimizer)``; the collaborative optimizer is
      unscaled under its own id, its inner torch optimizer is stepped under another, so the record is carried over;
    * ``_partial`` - optimizers whose records describe a local (accumulating) step and must be forgotten at the next
      ``update()`` that does not change the scale.
    """

    def __init__(self, *args, **kwargs):
        names_device = bool(args and isinstance(args[0], str)) or "device" in kwargs
        if not names_device:
            args = ("cuda" if torch.cuda.is_available() else "cpu", *args)
        super().__init__(*args, **kwargs)
        self._inside_global_step = False
        self._stepped = False
        self._handover: Dict[int, dict] = {}
        self._partial = set()
        self._lock = threading.RLock()

    @contextlib.contextmanager
    def running_global_step(self):
        """Inside this context ``unscale_`` and ``step`` act for real (the collaborative optimizer enters it)."""
        with self._lock:
            outer = self._inside_global_step
            self._inside_global_step = True
            try:
                yield
            finally:
                self._inside_global_step = outer

    @staticmethod
    def _is_collaborative(optimizer) -> bool:
        from hivemind_b200.optim.optimizer import Optimizer

        return isinstance(optimizer, Optimizer)

    @staticmethod
    def _overflows(found_inf_per_device: Dict[torch.device, torch.Tensor]) -> float:
        return sum(flag.item() for flag in found_inf_per_device.values())

    def unscale_(self, optimizer: TorchOptimizer) -> bool:
        """True if the gradients were unscaled (global step); otherwise only overflow was looked for."""
        assert self._is_collaborative(optimizer), "this scaler is meant for hivemind_b200.Optimizer"
        with self._lock:
            if not self._inside_global_step:
                self._check_inf_per_device(optimizer)  # gradients keep their scale while they accumulate
                self._partial.add(id(optimizer))
                return False
            super().unscale_(optimizer)
            self._handover[id(optimizer.opt)] = deepcopy(self._per_optimizer_states[id(optimizer)])
            return True

    def _global_step(self, inner: TorchOptimizer, *args, **kwargs) -> None:
        if self._stepped:
            logger.warning("Please call grad_scaler.update() after each step")
        record = self._handover.pop(id(inner), None)
        if record is not None:
            self._per_optimizer_states[id(inner)] = record
        stage = self._per_optimizer_states[id(inner)]["stage"]
        assert stage == OptState.UNSCALED, "the collaborative optimizer unscales before it steps its inner optimizer"
        if self.are_grads_finite(inner, use_cached=True):
            super().step(inner, *args, **kwargs)
        else:
            logger.warning("Skipping global step due to gradient over/underflow")
        self._stepped = True

    def step(self, optimizer: TorchOptimizer, *args, **kwargs) -> bool:
        """True if this was the inner optimizer's step of a global step."""
        if self._inside_global_step and not self._is_collaborative(optimizer):
            with self._lock:
                self._global_step(optimizer, *args, **kwargs)
            return True
        # A local step of the collaborative optimizer: it accumulates and reports progress. The optimizer is handed this
        # scaler explicitly (torch's own ``step`` does the same for optimizers whose ``step`` takes ``grad_scaler``,
        # but announces that it will stop doing so).
        if not self._enabled:
            optimizer.step(*args, **kwargs)
            return False
        record = self._per_optimizer_states[id(optimizer)]
        if record["stage"] is OptState.STEPPED:
            raise RuntimeError("step() has already been called since the last update().")
        optimizer.step(*args, **{**kwargs, "grad_scaler": self})
        record["stage"] = OptState.STEPPED
        self._partial.add(id(optimizer))
        return False

    def update(self, new_scale: Optional[float] = None) -> bool:
        """Change the scale only after a global step or on overflow; True if torch's update ran."""
        with self._lock:
            overflow = any(self._overflows(record["found_inf_per_device"]) for record in self._per_optimizer_states.values())
            if self._stepped or overflow:
                super().update(new_scale)
                self._stepped = False
                return True
            while self._partial:
                self._per_optimizer_states[self._partial.pop()] = _refresh_per_optimizer_state()
            return False

    def _unscale_grads_(self, optimizer: TorchOptimizer, inv_scale: torch.Tensor, found_inf: torch.Tensor,
                        allow_fp16: bool) -> Dict[torch.device, torch.Tensor]:
        # master parameters may be fp16 / bf16 here
        return super()._unscale_grads_(optimizer, inv_scale, found_inf, allow_fp16=True)

    def are_grads_finite(self, optimizer: TorchOptimizer, use_cached: bool = False) -> bool:
        flags = self._found_inf_per_device(optimizer) if use_cached else self._check_inf_per_device(optimizer)
        return not self._overflows(flags)

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
    def __init__(self, *args, **kwargs):
        if args and isinstance(args[0], str) or "device" in kwargs:
            super().__init__(*args, **kwargs)
        else:
            super().__init__("cuda" if torch.cuda.is_available() else "cpu", *args, **kwargs)
        self._is_running_global_step = False
        self._is_ready_to_update = False
        self._inner_optimizer_states = {}
        self._optimizer_states_to_reset = set()
        self._lock = threading.RLock()

    @contextlib.contextmanager
    def running_global_step(self):
        """Inside this context ``unscale_`` and ``step`` act for real (the collaborative optimizer enters it)."""
        with self._lock:
            previous, self._is_running_global_step = self._is_running_global_step, True
            try:
                yield
            finally:
                self._is_running_global_step = previous

    @staticmethod
    def _is_collaborative(optimizer) -> bool:
        from hivemind_b200.optim.optimizer import Optimizer

        return isinstance(optimizer, Optimizer)

    def unscale_(self, optimizer: TorchOptimizer) -> bool:
        with self._lock:
            assert self._is_collaborative(optimizer), "this scaler is meant for hivemind_b200.Optimizer"
            if self._is_running_global_step:
                super().unscale_(optimizer)
                # the inner optimizer will look for its own record when ``step`` is called on it
                self._inner_optimizer_states[id(optimizer.opt)] = deepcopy(self._per_optimizer_states[id(optimizer)])
                return True
            self._check_inf_per_device(optimizer)  # only record overflow; gradients stay scaled
            self._optimizer_states_to_reset.add(id(optimizer))
            return False

    def step(self, optimizer: TorchOptimizer, *args, **kwargs) -> bool:
        if self._is_running_global_step and not self._is_collaborative(optimizer):
            with self._lock:
                if self._is_ready_to_update:
                    logger.warning("Please call grad_scaler.update() after each step")
                saved = self._inner_optimizer_states.pop(id(optimizer), None)
                if saved is not None:
                    self._per_optimizer_states[id(optimizer)] = saved
                assert self._per_optimizer_states[id(optimizer)]["stage"] == OptState.UNSCALED, \
                    "InternalError: Optimizer should have called .unscale internally before invoking grad_scaler.step"
                if self.are_grads_finite(optimizer, use_cached=True):
                    super().step(optimizer, *args, **kwargs)
                else:
                    logger.warning("Skipping global step due to gradient over/underflow")
                self._is_ready_to_update = True
                return True
        super().step(optimizer)
        self._optimizer_states_to_reset.add(id(optimizer))
        return False

    def update(self, new_scale: Optional[float] = None) -> bool:
        with self._lock:
            total_infs = 0
            for optimizer_state in self._per_optimizer_states.values():
                total_infs += sum(v.item() for v in optimizer_state["found_inf_per_device"].values())
            if self._is_ready_to_update or total_infs != 0:
                super().update(new_scale)
                self._is_ready_to_update = False
                return True
            for opt_id in self._optimizer_states_to_reset:
                self._per_optimizer_states[opt_id] = _refresh_per_optimizer_state()
            self._optimizer_states_to_reset.clear()
            return False

    def _unscale_grads_(self, optimizer: TorchOptimizer, inv_scale: torch.Tensor, found_inf: torch.Tensor,
                        allow_fp16: bool) -> Dict[torch.device, torch.Tensor]:
        return super()._unscale_grads_(optimizer, inv_scale, found_inf, allow_fp16=True)

    def are_grads_finite(self, optimizer: TorchOptimizer, use_cached: bool = False) -> bool:
        found = self._found_inf_per_device(optimizer) if use_cached else self._check_inf_per_device(optimizer)
        return not sum(v.item() for v in found.values())

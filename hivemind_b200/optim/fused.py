"""Fused optimizers: ``torch.optim.Optimizer`` subclasses whose step is one or two multi-tensor kernels.

``FusedLAMB`` follows the LAMB variant that the reference's ALBERT example trains with
(``torch_optimizer.Lamb(lr, betas, eps, weight_decay, clamp_value, debias)``,
examples/albert/run_trainer.py:240-248): Adam moments, update ``m / (sqrt(v) + eps) + wd * p``, per-tensor trust
ratio ``clamp(|p|, 0, clamp_value) / |update|`` (1 when either norm is zero), optional bias correction.
``FusedAdam`` matches ``torch.optim.Adam`` / ``AdamW``; ``FusedSGD`` matches ``torch.optim.SGD``.
State dict keys equal those of the PyTorch classes (``step``, ``exp_avg``, ``exp_avg_sq``, ``momentum_buffer``), so
checkpoints and peer-to-peer state downloads stay interchangeable. CPU tensors run the same math in PyTorch.
"""
from __future__ import annotations

from typing import Iterable, List, Tuple

import torch

from hivemind_b200.ops import multi_tensor as mt


def _bump_versions(params: Iterable[torch.Tensor]) -> None:
    """Kernels write through raw pointers; tell autograd (and bf16 weight caches) that the tensors changed."""
    for p in params:
        torch.autograd.graph.increment_version(p)


class _FusedBase(torch.optim.Optimizer):
    def _collect(self, group) -> Tuple[List[torch.Tensor], List[torch.Tensor]]:
        params, grads = [], []
        for p in group["params"]:
            if p.grad is None:
                continue
            if p.grad.is_sparse:
                raise RuntimeError(f"{type(self).__name__} does not support sparse gradients")
            params.append(p)
            grads.append(p.grad if p.grad.is_contiguous() else p.grad.contiguous())
        return params, grads

    def _advance_steps(self, params: List[torch.Tensor], grads: List[torch.Tensor]):
        """Advance every parameter's own step counter and batch the parameters by the new value: a parameter that
        sat out some steps (its gradient was None) must get the bias correction of ITS step count, so each batch
        becomes one multi-tensor launch. Normally there is exactly one batch. Yields (step, params, grads)."""
        batches = {}
        for p, g in zip(params, grads):
            state = self.state[p]
            value = state.get("step", 0)
            value = int(value.item()) if isinstance(value, torch.Tensor) else int(value)
            state["step"] = value + 1
            entry = batches.setdefault(value + 1, ([], []))
            entry[0].append(p)
            entry[1].append(g)
        return [(step, ps, gs) for step, (ps, gs) in sorted(batches.items())]


class FusedLAMB(_FusedBase):
    def __init__(self, params, lr: float = 1e-3, betas: Tuple[float, float] = (0.9, 0.999), eps: float = 1e-6,
                 weight_decay: float = 0.0, clamp_value: float = 10.0, debias: bool = False):
        if lr <= 0 or eps < 0 or not 0 <= betas[0] < 1 or not 0 <= betas[1] < 1 or weight_decay < 0 or clamp_value < 0:
            raise ValueError("invalid LAMB hyper-parameters")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, clamp_value=clamp_value,
                                      debias=debias))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            params, grads = self._collect(group)
            if not params:
                continue
            for p in params:
                state = self.state[p]
                if "exp_avg" not in state:
                    state["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    state["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
                if "_update" not in self.__dict__.setdefault("_scratch", {}).setdefault(id(p), {}):
                    self._scratch[id(p)]["_update"] = torch.empty_like(p, dtype=torch.float32)
            for step, ps, gs in self._advance_steps(params, grads):
                mt.lamb_step_(ps, gs, [self.state[p]["exp_avg"] for p in ps], [self.state[p]["exp_avg_sq"] for p in ps],
                              [self._scratch[id(p)]["_update"] for p in ps], step=step, lr=group["lr"],
                              betas=group["betas"], eps=group["eps"], weight_decay=group["weight_decay"],
                              clamp_value=group["clamp_value"], debias=group["debias"])
            _bump_versions(params)
        return loss


class FusedAdam(_FusedBase):
    def __init__(self, params, lr: float = 1e-3, betas: Tuple[float, float] = (0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, decoupled_weight_decay: bool = False):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                      decoupled_weight_decay=decoupled_weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            params, grads = self._collect(group)
            if not params:
                continue
            for p in params:
                state = self.state[p]
                if "exp_avg" not in state:
                    state["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    state["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
            for step, ps, gs in self._advance_steps(params, grads):
                mt.adam_step_(ps, gs, [self.state[p]["exp_avg"] for p in ps], [self.state[p]["exp_avg_sq"] for p in ps],
                              step=step, lr=group["lr"], betas=group["betas"], eps=group["eps"],
                              weight_decay=group["weight_decay"], decoupled=group["decoupled_weight_decay"])
            _bump_versions(params)
        return loss


class FusedAdamW(FusedAdam):
    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 1e-2):
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, decoupled_weight_decay=True)


class FusedSGD(_FusedBase):
    def __init__(self, params, lr: float = 1e-3, momentum: float = 0.0, dampening: float = 0.0,
                 weight_decay: float = 0.0, nesterov: bool = False):
        if nesterov and (momentum <= 0 or dampening != 0):
            raise ValueError("Nesterov momentum requires a momentum and zero dampening")
        super().__init__(params, dict(lr=lr, momentum=momentum, dampening=dampening, weight_decay=weight_decay,
                                      nesterov=nesterov))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            params, grads = self._collect(group)
            if not params:
                continue
            options = dict(lr=group["lr"], momentum=group["momentum"], dampening=group["dampening"],
                           weight_decay=group["weight_decay"], nesterov=group["nesterov"])
            if group["momentum"] == 0:
                mt.sgd_step_(params, grads, None, first_step=False, **options)
            else:
                # a momentum buffer starts as a copy of the first gradient its parameter sees; parameters whose
                # buffers already exist must not be reset because a late-comer in the same group gets its first
                fresh = [i for i, p in enumerate(params) if "momentum_buffer" not in self.state[p]]
                seasoned = [i for i, p in enumerate(params) if "momentum_buffer" in self.state[p]]
                for i in fresh:
                    self.state[params[i]]["momentum_buffer"] = torch.zeros_like(params[i], dtype=torch.float32)
                for first, chosen in ((True, fresh), (False, seasoned)):
                    if chosen:
                        mt.sgd_step_([params[i] for i in chosen], [grads[i] for i in chosen],
                                     [self.state[params[i]]["momentum_buffer"] for i in chosen], first_step=first, **options)
            _bump_versions(params)
        return loss

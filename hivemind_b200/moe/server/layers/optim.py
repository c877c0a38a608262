"""Optimizer wrappers for experts.

``OptimizerWrapper`` delegates the whole ``torch.optim.Optimizer`` interface to an inner optimizer (attribute access
falls through, so state, param_groups, hooks and schedulers see the inner object); ``ClippingWrapper`` clips the
global gradient norm before every step, as the reference's wrapper does for ``--clip_grad_norm``
(hivemind/moe/server/layers/optim.py:4-57). On a GPU the norm and the scaling are two launches of the multi-tensor
kernels in ``ops/csrc/multi_tensor.cu`` for all parameters together.
"""
from typing import Iterable, List

import torch

from hivemind_b200.ops import multi_tensor as mt

_DELEGATED = ("defaults", "state", "param_groups")


class OptimizerWrapper(torch.optim.Optimizer):
    """Behaves like ``optim``; subclasses override the methods they want to change."""

    def __init__(self, optim: torch.optim.Optimizer):
        # deliberately no Optimizer.__init__: there are no parameters of our own, everything lives in ``optim``
        object.__setattr__(self, "optim", optim)

    def __getattribute__(self, name: str):
        if name in _DELEGATED:
            return getattr(object.__getattribute__(self, "optim"), name)
        return object.__getattribute__(self, name)

    def __repr__(self) -> str:
        return f"{type(self).__name__}({self.optim!r})"

    def __getstate__(self):
        return self.optim.__getstate__()

    def __setstate__(self, state) -> None:
        self.optim.__setstate__(state)

    def step(self, *args, **kwargs):
        return self.optim.step(*args, **kwargs)

    def zero_grad(self, *args, **kwargs):
        return self.optim.zero_grad(*args, **kwargs)

    def state_dict(self) -> dict:
        return self.optim.state_dict()

    def load_state_dict(self, state_dict: dict) -> None:
        self.optim.load_state_dict(state_dict)

    def add_param_group(self, param_group: dict) -> None:
        self.optim.add_param_group(param_group)


def _gradients(groups: Iterable[dict]) -> List[torch.Tensor]:
    return [p.grad for group in groups for p in group["params"] if p.grad is not None]


class ClippingWrapper(OptimizerWrapper):
    """Clips gradients to a global L2 norm of ``clip_grad_norm`` before each step of the wrapped optimizer."""

    def __init__(self, optim: torch.optim.Optimizer, clip_grad_norm: float):
        super().__init__(optim)
        self.clip_grad_norm = clip_grad_norm

    def step(self, *args, **kwargs):
        grads = _gradients(self.param_groups)
        fusable = grads and len({g.device for g in grads}) == 1 and all(
            g.is_floating_point() and g.is_contiguous() for g in grads)
        if fusable:
            mt.clip_grad_norm_(grads, self.clip_grad_norm)
        elif grads:
            torch.nn.utils.clip_grad_norm_([p for group in self.param_groups for p in group["params"]],
                                           self.clip_grad_norm)
        return super().step(*args, **kwargs)

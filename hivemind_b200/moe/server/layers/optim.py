"""Optimizer wrappers for experts (reference: hivemind/moe/server/layers/optim.py:4-57).

``ClippingWrapper`` clips the global gradient norm before every step; on GPU the norm and the scaling are the
multi-tensor kernels of ``ops/csrc/multi_tensor.cu`` (two launches for all parameters)."""
import torch

from hivemind_b200.ops import multi_tensor as mt


class OptimizerWrapper(torch.optim.Optimizer):
    """Forwards everything to the wrapped optimizer; subclasses override what they need."""

    def __init__(self, optim: torch.optim.Optimizer):
        object.__init__(self)
        self.optim = optim

    @property
    def defaults(self):
        return self.optim.defaults

    @property
    def state(self):
        return self.optim.state

    def __getstate__(self):
        return self.optim.__getstate__()

    def __setstate__(self, state):
        self.optim.__setstate__(state)

    def __repr__(self):
        return f"{self.__class__.__name__}({repr(self.optim)})"

    def state_dict(self):
        return self.optim.state_dict()

    def load_state_dict(self, state_dict: dict) -> None:
        return self.optim.load_state_dict(state_dict)

    def step(self, *args, **kwargs):
        return self.optim.step(*args, **kwargs)

    def zero_grad(self, *args, **kwargs):
        return self.optim.zero_grad(*args, **kwargs)

    @property
    def param_groups(self):
        return self.optim.param_groups

    def add_param_group(self, param_group: dict) -> None:
        return self.optim.add_param_group(param_group)


class ClippingWrapper(OptimizerWrapper):
    """A wrapper that clips gradients to ``clip_grad_norm`` (global L2 norm) before each optimizer step."""

    def __init__(self, optim: torch.optim.Optimizer, clip_grad_norm):
        super().__init__(optim)
        self.clip_grad_norm = clip_grad_norm

    def step(self, *args, **kwargs):
        grads = [p.grad for group in self.param_groups for p in group["params"] if p.grad is not None]
        if grads and all(g.is_contiguous() and g.is_floating_point() for g in grads) and len({g.device for g in grads}) == 1:
            mt.clip_grad_norm_(grads, self.clip_grad_norm)
        else:
            parameters = tuple(param for group in self.param_groups for param in group["params"])
            torch.nn.utils.clip_grad_norm_(parameters, self.clip_grad_norm)
        return super().step(*args, **kwargs)

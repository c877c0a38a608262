"""``det_dropout``: an expert with dropout whose keep-mask is an INPUT of the expert.

A server recomputes the forward pass during backward (see ``ModuleBackend.backward``), so a random mask drawn inside
the expert would differ between the two passes. The client draws the mask and sends it along; the same behaviour as
the reference's deterministic dropout expert (hivemind/moe/server/layers/dropout.py:7-53).
"""
import torch
from torch import nn

from hivemind_b200.moe.server.layers.custom_experts import register_expert_class


class _MaskedScale(torch.autograd.Function):
    """y = x * mask / keep_prob, with the mask treated as a constant."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, mask: torch.Tensor, inverse_keep: float) -> torch.Tensor:
        scale = mask.to(x.dtype) * inverse_keep
        ctx.save_for_backward(scale)
        return x * scale

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        (scale,) = ctx.saved_tensors
        return grad_output * scale, None, None


class DeterministicDropout(nn.Module):
    """Dropout with a caller-supplied keep-mask (1 = keep); identity in eval mode."""

    def __init__(self, drop_prob: float):
        super().__init__()
        assert 0.0 <= drop_prob < 1.0
        self.keep_prob = 1.0 - drop_prob

    def forward(self, x: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        if not self.training:
            return x
        return _MaskedScale.apply(x, mask, 1.0 / self.keep_prob)


DeterministicDropoutFunction = _MaskedScale  # the name used by the reference


def dropout_sample_input(batch_size: int, hid_dim: int):
    return torch.empty((batch_size, hid_dim)), torch.randint(0, 1, (batch_size, hid_dim))


@register_expert_class("det_dropout", dropout_sample_input)
class DeterministicDropoutNetwork(nn.Module):
    """dropout(x, mask) -> Linear(h, 2h) -> ReLU -> Linear(2h, h)."""

    def __init__(self, hid_dim: int, dropout_prob: float = 0.2):
        super().__init__()
        self.dropout = DeterministicDropout(dropout_prob)
        self.linear_in = nn.Linear(hid_dim, 2 * hid_dim)
        self.linear_out = nn.Linear(2 * hid_dim, hid_dim)

    def forward(self, x: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        hidden = torch.relu(self.linear_in(self.dropout(x, mask)))
        return self.linear_out(hidden)

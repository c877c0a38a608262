"""``RemoteSwitchMixtureOfExperts``: Switch-Transformer routing over the swarm.

Top-1 routing by default (``k_best=1``), multiplicative input jitter, random "grid dropout" of coordinates, expert
probability = product of per-dimension softmaxes, a residual connection, and a load-balancing auxiliary loss built
from an exponential moving average of how often each coordinate was used
(reference: hivemind/moe/client/switch_moe.py:16-226; Fedus et al., arXiv:2101.03961).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch

from hivemind_b200.moe.client.expert import DUMMY, RemoteExpert
from hivemind_b200.moe.client.moe import RemoteMixtureOfExperts, _RemoteCallMany, gather_expert_scores
from hivemind_b200.moe.expert_uid import UID_DELIMITER
from hivemind_b200.p2p.control import P2PDaemonError
from hivemind_b200.utils import nested_flatten, nested_pack
from hivemind_b200.utils.logging import get_logger

logger = get_logger(__name__)


class RemoteSwitchMixtureOfExperts(RemoteMixtureOfExperts):
    """
    :param utilization_alpha: EMA factor of the per-coordinate utilisation estimate
    :param grid_dropout: probability of *keeping* each grid coordinate in a forward pass
    :param jitter_eps: gate inputs are multiplied by noise uniform in ``[1 - eps, 1 + eps]``
    :returns: ``(outputs + input, balancing_loss)`` from ``forward``
    Other parameters as in ``RemoteMixtureOfExperts``; by default no expert is required to answer
    (``k_min = backward_k_min = 0``, ``allow_zero_outputs=True``): a token whose expert is gone passes through.
    """

    def __init__(self, *, grid_size: Tuple[int, ...], utilization_alpha: float = 0.9, grid_dropout: float = 1.0,
                 jitter_eps: float = 1e-2, k_best: int = 1, k_min: int = 0, backward_k_min: int = 0,
                 allow_zero_outputs: bool = True, **kwargs):
        super().__init__(grid_size=grid_size, k_best=k_best, k_min=k_min, backward_k_min=backward_k_min,
                         allow_zero_outputs=allow_zero_outputs, **kwargs)
        uniform = torch.cat([torch.full((size,), 1.0 / size, dtype=torch.float) for size in grid_size])
        self.register_buffer("grid_utilization", uniform)
        self.utilization_alpha, self.grid_dropout, self.jitter_eps = utilization_alpha, grid_dropout, jitter_eps

    def forward(self, input: torch.Tensor, *args: torch.Tensor, **kwargs: torch.Tensor):
        grid_sizes = tuple(self.beam_search.grid_size)
        gate_input = input if input.ndim == 2 else input.mean(dim=tuple(range(1, input.ndim - 1)))
        jitter = torch.empty_like(gate_input).uniform_(1 - self.jitter_eps, 1 + self.jitter_eps)
        gate_input = gate_input * jitter

        grid_scores = self.proj(gate_input).split_with_sizes(grid_sizes, dim=-1)
        kept = [torch.rand(size, device=gate_input.device) < self.grid_dropout for size in grid_sizes]
        grid_scores = [scores.masked_fill(~keep, float("-inf")) for scores, keep in zip(grid_scores, kept)]
        grid_softmax = [torch.softmax(scores, dim=-1) for scores in grid_scores]

        chosen_experts: List[List[RemoteExpert]] = self.beam_search.batch_find_best_experts(
            [scores.detach().float().cpu().numpy() for scores in grid_scores], self.k_best)
        if self._expert_info is None:
            try:
                self._expert_info = next(expert.info for row in chosen_experts for expert in row)
            except StopIteration:
                raise RuntimeError("No responding experts found during beam search. Check that UID prefixes and "
                                   "the grid size are consistent with running Server instances.")
            except P2PDaemonError as e:
                logger.warning(f"Failed to get RemoteSwitchMixtureOfExperts.output_shape: {e}")

        expert_mask, *expert_outputs = _RemoteCallMany.apply(
            DUMMY, chosen_experts, self.k_min, self.backward_k_min, self.timeout_after_k_min, self.forward_timeout,
            self.backward_timeout, self.detect_anomalies, self.allow_zero_outputs, self.info, self.max_rows_per_call,
            *nested_flatten(((input, *args), kwargs)))

        batch_utilization = self._compute_batch_utilization(chosen_experts, expert_mask)
        self.grid_utilization = (self.utilization_alpha * self.grid_utilization
                                 + (1 - self.utilization_alpha) * batch_utilization)

        expert_probs = self.compute_expert_scores(grid_softmax, chosen_experts)
        expert_probs = torch.where(expert_mask, expert_probs, torch.zeros((), device=expert_probs.device,
                                                                          dtype=expert_probs.dtype))
        mixed = [(expert_probs[..., None] * tensor.flatten(start_dim=2)).view(tensor.shape).sum(dim=1)
                 for tensor in expert_outputs]
        packed = nested_pack(mixed, self.info["outputs_schema"])

        # balancing loss: per dimension, mean(probability mass per coordinate * routed fraction) * size^2
        utilization = self.grid_utilization.split_with_sizes(grid_sizes)
        balancing_loss = torch.stack([
            torch.mean(dim_softmax.mean(0) * dim_utilization) * size ** 2
            for dim_softmax, dim_utilization, size in zip(grid_softmax, utilization, grid_sizes)]).sum()

        if isinstance(packed, torch.Tensor):
            packed = packed + input
        else:
            packed = list(packed)
            packed[0] = packed[0] + input
            packed = type(self.info["outputs_schema"])(packed) if isinstance(self.info["outputs_schema"], tuple) else packed
        return packed, balancing_loss

    @torch.no_grad()
    def _compute_batch_utilization(self, batch_experts: List[List[RemoteExpert]], expert_mask: torch.Tensor
                                   ) -> torch.Tensor:
        """Fraction of answered calls that used each coordinate, concatenated over dimensions."""
        counts = [torch.zeros(size, dtype=self.grid_utilization.dtype) for size in self.beam_search.grid_size]
        prefix_len = len(self.beam_search.uid_prefix)
        for sample, slot in expert_mask.nonzero().cpu().tolist():
            coords = batch_experts[sample][slot].uid[prefix_len:].split(UID_DELIMITER)
            for coord, dim_counts in zip(coords, counts):
                dim_counts[int(coord)] += 1
        normalised = [torch.nn.functional.normalize(dim_counts, p=1, dim=0) for dim_counts in counts]
        return torch.cat(normalised).to(self.grid_utilization.device)

    def compute_expert_scores(self, grid_probs: Sequence[torch.Tensor], batch_experts: List[List[RemoteExpert]]
                              ) -> torch.Tensor:
        """Probability of each chosen expert = product of its coordinates' probabilities (``-inf`` padding)."""
        return gather_expert_scores(grid_probs, batch_experts, len(self.beam_search.uid_prefix), product=True)

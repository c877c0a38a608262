"""``RemoteMixtureOfExperts``: a layer that routes every sample to its ``k_best`` live experts across the swarm.

Behaviour (reference: hivemind/moe/client/moe.py:28-440): a learned projection scores each grid coordinate; beam
search over the DHT finds the best live experts per sample; the layer calls them, tolerating failures (an expert
that errs or misses the deadline is masked out; the call fails only if fewer than ``k_min`` experts answered for
some sample), and returns the softmax-weighted mixture of the answers. Gradients flow to the inputs through the
experts' own backward RPCs and to the gate through the mixture weights.

Difference from the reference's wire pattern: it issues one single-row RPC per (sample, expert) pair; here the rows
that go to the same expert are stacked into one request (split only above ``max_rows_per_call``), so a batch costs
one message per distinct expert rather than ``batch * k`` messages. On CUDA inputs the masked softmax and the
weighted combine of the ``[batch, k, ...]`` answers run as one fused kernel (``ops.moe.masked_softmax_combine``).
"""
from __future__ import annotations

import time
from concurrent.futures import Future
from queue import Empty, Queue
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
from torch.autograd.function import once_differentiable

from hivemind_b200.dht import DHT
from hivemind_b200.moe.client.beam_search import MoEBeamSearcher
from hivemind_b200.moe.client.expert import DUMMY, RemoteExpert, expert_backward, expert_forward, get_server_stub
from hivemind_b200.moe.client.remote_expert_worker import RemoteExpertWorker
from hivemind_b200.moe.expert_uid import UID_DELIMITER
from hivemind_b200.p2p.control import P2PDaemonError
from hivemind_b200.utils import nested_flatten, nested_pack
from hivemind_b200.utils.logging import get_logger

logger = get_logger(__name__)


class RemoteMixtureOfExperts(nn.Module):
    """
    :param in_features: size of the last input dimension (the gate's input)
    :param grid_size: number of coordinates in each dimension of the expert grid
    :param dht: DHT used to find experts
    :param uid_prefix: common prefix of expert uids, e.g. ``"ffn_expert."``
    :param k_best: mix this many best-scoring experts per sample
    :param k_min: every sample needs at least this many answers, otherwise forward raises ``TimeoutError``
    :param forward_timeout / backward_timeout: total deadline of each phase in seconds (None = unbounded)
    :param timeout_after_k_min: once every sample has ``k_min`` answers, wait at most this long for the rest
    :param backward_k_min: minimum number of experts per sample that must return gradients
    :param detect_anomalies: treat non-finite inputs as an error and non-finite answers as failures
    :param allow_zero_outputs: return zeros instead of raising when no expert answered at all
    :param max_rows_per_call: rows of one expert's share of the batch sent in one request
    """

    def __init__(self, *, in_features: int, grid_size: Tuple[int, ...], dht: DHT, uid_prefix: str, k_best: int,
                 k_min: int = 1, forward_timeout: Optional[float] = None, timeout_after_k_min: Optional[float] = None,
                 backward_k_min: int = 1, backward_timeout: Optional[float] = None, detect_anomalies: bool = False,
                 allow_zero_outputs: bool = False, max_rows_per_call: int = 1024, **dht_kwargs):
        super().__init__()
        self.dht = dht
        self.beam_search = MoEBeamSearcher(dht, uid_prefix, grid_size, **dht_kwargs)
        self.k_best, self.k_min, self.backward_k_min = k_best, k_min, backward_k_min
        self.forward_timeout, self.backward_timeout = forward_timeout, backward_timeout
        self.timeout_after_k_min = timeout_after_k_min
        self.detect_anomalies, self.allow_zero_outputs = detect_anomalies, allow_zero_outputs
        self.max_rows_per_call = max_rows_per_call
        self.proj = nn.Linear(in_features, self.beam_search.total_grid_size)  # logits of all dimensions at once
        self._expert_info: Optional[Dict[str, Any]] = None

    def forward(self, input: torch.Tensor, *args: torch.Tensor, **kwargs: torch.Tensor):
        """
        :param input: batch-first tensor; the gate sees its mean over all dimensions but the first and the last
        :param args / kwargs: further batch-first inputs passed to every expert
        :returns: the mixture of the experts' outputs, same nested structure as one expert's output
        """
        gate_input = input if input.ndim == 2 else input.mean(dim=tuple(range(1, input.ndim - 1)))
        grid_scores = self.proj(gate_input).split_with_sizes(tuple(self.beam_search.grid_size), dim=-1)
        chosen_experts: List[List[RemoteExpert]] = self.beam_search.batch_find_best_experts(
            [scores.detach().float().cpu().numpy() for scores in grid_scores], self.k_best)
        if self._expert_info is None:
            try:
                self._expert_info = next(expert.info for row in chosen_experts for expert in row)
            except StopIteration:
                raise RuntimeError("No responding experts found during beam search. Check that UID prefixes and "
                                   "the grid size are consistent with running Server instances.")
            except P2PDaemonError as e:
                logger.warning(f"Failed to get RemoteMixtureOfExperts.output_shape: {e}")

        expert_mask, *expert_outputs = _RemoteCallMany.apply(
            DUMMY, chosen_experts, self.k_min, self.backward_k_min, self.timeout_after_k_min, self.forward_timeout,
            self.backward_timeout, self.detect_anomalies, self.allow_zero_outputs, self.info, self.max_rows_per_call,
            *nested_flatten(((input, *args), kwargs)))
        # expert_outputs: tensors of shape [batch, max_experts, *output_shape]; mask marks the answers that arrived

        expert_logits = self.compute_expert_scores(grid_scores, chosen_experts)
        mixed = [_mix(expert_logits, expert_mask, tensor) for tensor in expert_outputs]
        return nested_pack(mixed, self.info["outputs_schema"])

    def compute_expert_scores(self, grid_scores: Sequence[torch.Tensor], batch_experts: List[List[RemoteExpert]]
                              ) -> torch.Tensor:
        """
        Sum each chosen expert's coordinate scores (differentiable w.r.t. ``grid_scores``).

        :returns: ``float[batch, max experts per sample]``, padded with ``-inf`` where a row has fewer experts
        """
        return gather_expert_scores(grid_scores, batch_experts, len(self.beam_search.uid_prefix), product=False)

    @property
    def info(self) -> Dict[str, Any]:
        """Schemas of the experts in this grid (taken from whichever expert is found first)."""
        if self._expert_info is None:
            device = self.proj.weight.device
            probe = self.proj(torch.randn(1, self.proj.in_features, device=device)).detach().cpu()
            probe_scores = probe.split_with_sizes(tuple(self.beam_search.grid_size), dim=-1)
            found = self.beam_search.find_best_experts([s[0] for s in probe_scores], beam_size=1)
            if not found:
                raise RuntimeError("No experts found in the DHT under prefix " + self.beam_search.uid_prefix)
            self._expert_info = found[0].info
        return self._expert_info


def gather_expert_scores(grid_values: Sequence[torch.Tensor], batch_experts: List[List[RemoteExpert]], prefix_len: int,
                         product: bool) -> torch.Tensor:
    """
    Combine each chosen expert's per-dimension values (sum of logits, or product of probabilities) into
    ``[batch, max experts per sample]``, ``-inf`` where a row has fewer experts; differentiable w.r.t. ``grid_values``.
    """
    device = grid_values[0].device
    batch_size = len(batch_experts)
    width = max((len(row) for row in batch_experts), default=0)
    rows, cols, coords = [], [], []
    for i, row in enumerate(batch_experts):
        for j, expert in enumerate(row):
            rows.append(i)
            cols.append(j)
            coords.append([int(c) for c in expert.uid[prefix_len:].split(UID_DELIMITER)])
    scores = torch.full((batch_size, width), float("-inf"), device=device, dtype=grid_values[0].dtype)
    if not rows:
        return scores
    row_index = torch.as_tensor(rows, device=device)
    col_index = torch.as_tensor(cols, device=device)
    coord_index = torch.as_tensor(coords, device=device)  # [n, ndim]
    flat = None
    for d, dim_values in enumerate(grid_values):
        picked = dim_values[row_index, coord_index[:, d]]
        flat = picked if flat is None else (flat * picked if product else flat + picked)
    return scores.index_put((row_index, col_index), flat)


def _mix(expert_logits: torch.Tensor, expert_mask: torch.Tensor, outputs: torch.Tensor) -> torch.Tensor:
    """softmax over the answered experts of each row, then the weighted sum of their outputs."""
    if outputs.is_cuda and outputs.dtype in (torch.float32, torch.bfloat16, torch.float16):
        from hivemind_b200.ops.moe import masked_softmax_combine

        return masked_softmax_combine(expert_logits, expert_mask, outputs)
    masked = torch.where(expert_mask, expert_logits, torch.full((1,), float("-inf"), device=expert_logits.device,
                                                                dtype=expert_logits.dtype))
    weights = torch.softmax(masked, dim=1)
    weights = torch.where(expert_mask.any(dim=1, keepdim=True), weights, torch.zeros_like(weights))
    return (weights[..., None] * outputs.flatten(start_dim=2)).view(outputs.shape).sum(dim=1)


class _Call:
    """One request to one expert: which (sample, slot) pairs its rows belong to."""
    __slots__ = ("expert", "samples", "slots")

    def __init__(self, expert: RemoteExpert):
        self.expert, self.samples, self.slots = expert, [], []


def _group_calls(experts_per_sample: List[List[RemoteExpert]], max_rows: int,
                 pairs: Optional[Sequence[Tuple[int, int]]] = None) -> List[_Call]:
    """Group (sample, slot) pairs by expert, in chunks of at most ``max_rows`` rows."""
    if pairs is None:
        pairs = [(i, j) for i, row in enumerate(experts_per_sample) for j in range(len(row))]
    open_calls: Dict[Tuple[str, Any], _Call] = {}
    calls: List[_Call] = []
    for i, j in pairs:
        expert = experts_per_sample[i][j]
        key = (expert.uid, expert.peer_id)
        call = open_calls.get(key)
        if call is None or len(call.samples) >= max_rows:
            call = open_calls[key] = _Call(expert)
            calls.append(call)
        call.samples.append(i)
        call.slots.append(j)
    return calls


class _RemoteCallMany(torch.autograd.Function):
    """
    Calls many experts on (subsets of) a batch and survives individual failures. An expert that failed in forward
    gets zero outputs and ``mask[i, j] = False``; one that failed in backward contributes zero gradient.
    """

    @classmethod
    def forward(cls, ctx, dummy, experts_per_sample: List[List[RemoteExpert]], k_min: int, backward_k_min: int,
                timeout_after_k_min: Optional[float], forward_timeout: Optional[float],
                backward_timeout: Optional[float], detect_anomalies: bool, allow_zero_outputs: bool,
                info: Dict[str, Any], max_rows_per_call: int, *flat_inputs: torch.Tensor) -> Tuple[torch.Tensor, ...]:
        assert not torch.is_grad_enabled()
        num_samples = len(experts_per_sample)
        max_experts = max(map(len, experts_per_sample)) if experts_per_sample else 0
        device = flat_inputs[0].device
        flat_inputs_cpu = []
        for tensor in flat_inputs:
            if detect_anomalies and not tensor.isfinite().all():
                raise ValueError("One of inputs has nan/inf values")
            flat_inputs_cpu.append(tensor.detach().cpu())
        assert all(len(t) == num_samples for t in flat_inputs_cpu)

        forward_compressions = [descr.compression for descr in nested_flatten(info["forward_schema"])]
        calls = _group_calls(experts_per_sample, max_rows_per_call)
        pending: Dict[Future, _Call] = {}
        for call in calls:
            index = torch.as_tensor(call.samples, dtype=torch.long)
            rows = [t.index_select(0, index) for t in flat_inputs_cpu]
            stub = get_server_stub(call.expert.p2p, call.expert.peer_id)
            future = RemoteExpertWorker.run_coroutine(expert_forward(call.expert.uid, rows, forward_compressions, stub),
                                                      return_future=True)
            pending[future] = call

        done = cls._collect_responses(pending, num_samples, k_min, forward_timeout, timeout_after_k_min,
                                      detect_anomalies)
        answered = [0] * num_samples
        for call, _ in done:
            for i in call.samples:
                answered[i] += 1
        routed = {i for call in calls for i in call.samples}
        if any(answered[i] < k_min for i in routed):
            raise TimeoutError(f"Forward pass: less than {k_min} responded within timeout")
        if not done and not allow_zero_outputs:
            raise RuntimeError("Forward pass: 0 experts responded within timeout and allow_zero_outputs is False")

        outputs_schema = info["outputs_schema"] if isinstance(info["outputs_schema"], tuple) else (info["outputs_schema"],)
        outputs = tuple(descr.make_zeros(num_samples, max_experts, device=device)
                        for descr in nested_flatten(outputs_schema))
        mask = torch.zeros([num_samples, max_experts], dtype=torch.bool, device=device)
        alive_i: List[int] = []
        alive_j: List[int] = []
        for call, tensors in done:
            alive_i.extend(call.samples)
            alive_j.extend(call.slots)
        batch_inds = torch.as_tensor(alive_i, dtype=torch.long, device=device)
        expert_inds = torch.as_tensor(alive_j, dtype=torch.long, device=device)
        if done:
            for k, output in enumerate(outputs):
                stacked = torch.cat([tensors[k] for _, tensors in done], dim=0)
                output[batch_inds, expert_inds] = stacked.to(device=output.device, dtype=output.dtype)
            mask[batch_inds, expert_inds] = True

        ctx.save_for_backward(batch_inds, expert_inds, *flat_inputs_cpu)
        ctx._saved_non_tensors = (info, backward_k_min, backward_timeout, timeout_after_k_min, experts_per_sample,
                                  detect_anomalies, max_rows_per_call)
        return (mask,) + outputs

    @classmethod
    @once_differentiable
    def backward(cls, ctx, *raw_grads: torch.Tensor) -> Tuple[Optional[torch.Tensor], ...]:
        assert not torch.is_grad_enabled()
        (info, backward_k_min, backward_timeout, timeout_after_k_min, experts_per_sample, detect_anomalies,
         max_rows_per_call) = ctx._saved_non_tensors
        alive_ii, alive_jj, *flat_inputs_cpu = ctx.saved_tensors
        mask_grad, *flat_grad_outputs = raw_grads
        device = flat_grad_outputs[0].device
        grads_cpu = []
        for tensor in flat_grad_outputs:
            if detect_anomalies and not tensor.isfinite().all():
                raise ValueError("One of gradients has nan/inf values")
            grads_cpu.append(tensor.cpu())
        num_samples, max_experts = mask_grad.shape
        pairs = list(zip(alive_ii.cpu().tolist(), alive_jj.cpu().tolist()))
        backward_compressions = [descr.compression
                                 for descr in nested_flatten((info["forward_schema"], info["outputs_schema"]))]

        calls = _group_calls(experts_per_sample, max_rows_per_call, pairs)
        pending: Dict[Future, _Call] = {}
        for call in calls:
            rows_index = torch.as_tensor(call.samples, dtype=torch.long)
            slots_index = torch.as_tensor(call.slots, dtype=torch.long)
            payload = tuple(t.index_select(0, rows_index) for t in flat_inputs_cpu) + \
                tuple(g[rows_index, slots_index] for g in grads_cpu)
            stub = get_server_stub(call.expert.p2p, call.expert.peer_id)
            future = RemoteExpertWorker.run_coroutine(
                expert_backward(call.expert.uid, payload, backward_compressions, stub), return_future=True)
            pending[future] = call

        done = cls._collect_responses(pending, num_samples, backward_k_min, backward_timeout, timeout_after_k_min,
                                      detect_anomalies)
        answered = [0] * num_samples
        for call, _ in done:
            for i in call.samples:
                answered[i] += 1
        if any(answered[i] < backward_k_min for i, _ in pairs):
            raise TimeoutError(f"Backward pass: less than {backward_k_min} experts responded within timeout")

        grad_inputs = [descr.make_zeros(num_samples, device=device) for descr in nested_flatten(info["forward_schema"])]
        for call, tensors in done:
            rows_index = torch.as_tensor(call.samples, dtype=torch.long, device=device)
            for grad_input, part in zip(grad_inputs, tensors):
                grad_input.index_add_(0, rows_index, part.to(device=device, dtype=grad_input.dtype))
        return (DUMMY, None, None, None, None, None, None, None, None, None, None, *grad_inputs)

    @staticmethod
    def _collect_responses(pending: Dict[Future, _Call], num_samples: int, k_min: int, timeout_total: Optional[float],
                           timeout_after_k_min: Optional[float], detect_anomalies: bool
                           ) -> List[Tuple[_Call, Tuple[torch.Tensor, ...]]]:
        """Wait until every routed sample has ``k_min`` answers, then ``timeout_after_k_min`` more; cancel the rest."""
        timeout_total = float("inf") if timeout_total is None else timeout_total
        timeout_after_k_min = float("inf") if timeout_after_k_min is None else timeout_after_k_min
        successes = [0] * num_samples
        waiting = {i for call in pending.values() for i in call.samples}  # samples with fewer than k_min answers
        if k_min <= 0:
            waiting.clear()
        deadline = time.perf_counter() + timeout_total
        if not waiting:
            deadline = min(deadline, time.perf_counter() + timeout_after_k_min)
        finished: "Queue[Future]" = Queue()
        outstanding = set(pending.keys())
        results: List[Tuple[_Call, Tuple[torch.Tensor, ...]]] = []
        try:
            for future in outstanding:
                future.add_done_callback(finished.put)
            for _ in range(len(pending)):
                wait = None if deadline == float("inf") else max(0.0, deadline - time.perf_counter())
                future = finished.get(timeout=wait)
                outstanding.discard(future)
                tensors = _process_dispatched_task(future, detect_anomalies)
                if tensors is None:
                    continue
                call = pending[future]
                results.append((call, tuple(tensors)))
                for i in call.samples:
                    successes[i] += 1
                    if successes[i] >= k_min:
                        waiting.discard(i)
                if not waiting:
                    deadline = min(deadline, time.perf_counter() + timeout_after_k_min)
        except Empty:
            pass  # the deadline passed: normal when some experts are slow or gone
        finally:
            for future in outstanding:
                future.cancel()
        return results


def _process_dispatched_task(task: Future, detect_anomalies: bool) -> Optional[Tuple[torch.Tensor, ...]]:
    if task.cancelled() or task.exception():
        logger.warning(f"Task {task} failed: {None if task.cancelled() else task.exception()!r}")
        return None
    outputs = task.result()
    if detect_anomalies and any(not tensor.isfinite().all() for tensor in outputs):
        logger.error(f"Task {task} failed: output tensor contains nan/inf values")
        return None
    return outputs

"""``DeviceMixtureOfExperts``: the mixture-of-experts layer for experts that live on this box's GPUs.

``RemoteMixtureOfExperts`` reaches experts through RPC, one message per expert; when clients and experts are
processes on the same NVLink domain the same computation is done on the device: the gate's top-k runs as a kernel
over the table of live experts (the role of beam search over the DHT: hivemind/moe/client/beam_search.py:263-352),
token rows are sorted by expert into one packed buffer (the role of the per-row RPC fan-out and the server's
re-batching: hivemind/moe/client/moe.py:227-243, hivemind/moe/server/task_pool.py:161-192), experts run tcgen05
GEMMs over their contiguous rows, and one kernel applies the masked softmax and the weighted sum
(hivemind/moe/client/moe.py:129-137). With a process group, experts are sharded over ranks (expert ``e`` lives on
rank ``e // experts_per_rank``) and rows travel by all-to-all; every rank is a client and a server at once.

Fault-tolerance semantics carry over: an expert absent from the ``alive`` table is never chosen, a token with fewer
than ``k_min`` live experts raises, and a token with no expert yields zeros (or the residual for Switch).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn

from hivemind_b200.moe.server.layers import name_to_block
from hivemind_b200.ops import moe as moe_ops
from hivemind_b200.ops.grouped_ffn import GroupedFeedforward
from hivemind_b200.utils.profiling import device_range


class _GroupedExperts(torch.autograd.Function):
    """
    Run expert ``e`` on rows ``offsets[e]:offsets[e+1]`` of the packed buffer. Each expert keeps its own small
    autograd graph from forward; backward replays them, so parameter gradients accumulate straight into ``.grad``
    (fp32, through the GEMM's reduce-add epilogue) and no slicing op sits in the outer graph.
    """

    @staticmethod
    def forward(ctx, packed: torch.Tensor, bounds: Sequence[int], experts: Sequence[nn.Module], train_experts: bool):
        out = torch.empty_like(packed)
        graphs = []
        need_graph = packed.requires_grad or train_experts
        for e, module in enumerate(experts):
            lo, hi = bounds[e], bounds[e + 1]
            if hi <= lo:
                continue
            rows = packed[lo:hi].detach()
            if need_graph:
                rows.requires_grad_(packed.requires_grad)
                with torch.enable_grad():
                    result = module(rows)
                graphs.append((lo, hi, rows, result))
                out[lo:hi].copy_(result.detach())
            else:
                out[lo:hi].copy_(module(rows))
        if bounds[len(experts)] < packed.shape[0]:
            out[bounds[len(experts)]:].zero_()
        ctx.graphs = graphs
        return out

    @staticmethod
    def backward(ctx, grad_out: torch.Tensor):
        grad_in = torch.zeros_like(grad_out)
        for lo, hi, rows, result in ctx.graphs:
            torch.autograd.backward(result, grad_out[lo:hi])
            if rows.grad is not None:
                grad_in[lo:hi].copy_(rows.grad)
        ctx.graphs = None
        return grad_in, None, None, None


class DeviceMixtureOfExperts(nn.Module):
    """
    :param in_features: hidden size of tokens and experts
    :param grid_size: expert grid; experts are numbered row-major over it
    :param k_best: experts mixed per token (at most 8)
    :param expert_cls: a registered expert class name (``"ffn"`` by default)
    :param k_min: every token needs this many live experts, otherwise ``forward`` raises ``RuntimeError``
      (checked only if ``check_k_min``; the check costs a device-to-host read)
    :param switch: Switch-style routing — probabilities multiply across grid dimensions, jitter, grid dropout, residual
      connection; ``forward`` then returns ``(output, balancing_loss)``
    :param group: process group over which experts are sharded (None = all experts on this device)
    :param compute_dtype: dtype of the rows sent to experts (bf16 on CUDA by default)
    :param exchange: how rows reach experts on other ranks: ``"all_to_all"`` (NCCL / gloo collectives) or ``"peer"``
      (kernels that pull rows straight out of the other GPUs' memory over NVLink; CUDA only, one box)
    :param max_tokens: for ``exchange="peer"``: the most tokens one forward pass will carry (sizes the arenas)
    """

    def __init__(self, *, in_features: int, grid_size: Sequence[int], k_best: int, expert_cls: str = "ffn",
                 k_min: int = 0, check_k_min: bool = False, switch: bool = False, jitter_eps: float = 1e-2,
                 grid_dropout: float = 1.0, utilization_alpha: float = 0.9, group: Optional[dist.ProcessGroup] = None,
                 compute_dtype: Optional[torch.dtype] = None, train_experts: bool = True,
                 exchange: str = "all_to_all", max_tokens: int = 0, exchange_timeout: float = 10.0):
        super().__init__()
        assert 1 <= k_best <= moe_ops.MAX_K and 1 <= len(grid_size) <= 3
        self.grid_size = tuple(int(g) for g in grid_size)
        self.num_experts = 1
        for g in self.grid_size:
            self.num_experts *= g
        self.k_best, self.k_min, self.check_k_min = k_best, k_min, check_k_min
        self.switch, self.jitter_eps, self.grid_dropout = switch, jitter_eps, grid_dropout
        self.utilization_alpha = utilization_alpha
        self.group = group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        assert self.num_experts % self.world == 0, "experts must divide evenly over ranks"
        self.experts_per_rank = self.num_experts // self.world
        self.first_expert = self.rank * self.experts_per_rank
        self.compute_dtype = compute_dtype
        self.train_experts = train_experts
        assert exchange in ("all_to_all", "peer")
        self.exchange_kind, self.max_tokens, self.exchange_timeout = exchange, max_tokens, exchange_timeout
        self._exchange = None  # PeerExpertExchange, created at the first CUDA forward
        self.proj = nn.Linear(in_features, sum(self.grid_size))
        # "ffn" experts share one set of stacked parameters and run as grouped GEMMs; any other registered class
        # runs expert by expert over its contiguous rows
        self.grouped = expert_cls == "ffn"
        if self.grouped:
            self.experts = GroupedFeedforward(self.experts_per_rank, in_features)
        else:
            self.experts = nn.ModuleList([name_to_block[expert_cls](in_features) for _ in range(self.experts_per_rank)])
        self.register_buffer("alive", torch.ones(self.num_experts, dtype=torch.uint8))
        uniform = torch.cat([torch.full((size,), 1.0 / size) for size in self.grid_size])
        self.register_buffer("grid_utilization", uniform)

    # ------------------------------------------------------------------------------------------------ liveness

    def set_alive(self, expert_ids: Sequence[int], alive: bool = True) -> None:
        """Mark experts as present or gone (what DHT expirations do for remote experts)."""
        self.alive[torch.as_tensor(list(expert_ids), dtype=torch.int64)] = 1 if alive else 0

    def expert_uid(self, expert_id: int, prefix: str = "expert.") -> str:
        coords = moe_ops.expert_coordinates(torch.tensor([expert_id]), self.grid_size)[0].tolist()
        return prefix + ".".join(str(c) for c in coords)

    # ------------------------------------------------------------------------------------------------- forward

    def forward(self, x: torch.Tensor):
        shape = x.shape
        tokens = x.reshape(-1, shape[-1])
        gate_in = tokens
        if self.switch and self.training and self.jitter_eps > 0:
            gate_in = tokens * torch.empty_like(tokens).uniform_(1 - self.jitter_eps, 1 + self.jitter_eps)
        scores = self.proj(gate_in.to(self.proj.weight.dtype)).float()
        if self.switch and self.grid_dropout < 1.0 and self.training:
            kept = torch.rand(scores.shape[1], device=scores.device) < self.grid_dropout
            scores = scores.masked_fill(~kept, float("-inf"))
        mode = "prob" if self.switch else "sum"
        with device_range("moe.gate"):
            idx, _ = moe_ops.gate_topk(scores, self.grid_size, self.k_best, self.alive, mode)
            gate = moe_ops.expert_values(scores, idx, self.grid_size, mode)
        if self.check_k_min and self.k_min > 0:
            if int(((idx >= 0).sum(1) < self.k_min).any()):
                raise RuntimeError(f"some tokens have fewer than {self.k_min} live experts")

        dtype = self.compute_dtype or (torch.bfloat16 if tokens.is_cuda else tokens.dtype)
        rows = tokens.to(dtype)
        align = moe_ops.TILE_ROWS if (self.grouped and self.world == 1) else 1
        with device_range("moe.dispatch"):
            routed = moe_ops.dispatch(rows, idx, self.num_experts, align=align)
        with device_range("moe.experts"):
            answers, row_ok = self._run_experts(routed)
        keep = None
        if row_ok is not None:  # rows whose expert host did not answer in time count as failed experts
            keep = row_ok[routed.pos.clamp(min=0).long()] & (routed.pos >= 0)
        residual = rows if self.switch else None
        with device_range("moe.combine"):
            mixed = moe_ops.combine(answers, routed.pos, gate, "prob" if self.switch else "softmax", keep=keep,
                                    residual=residual)
        out = mixed.to(x.dtype).view(shape)
        if not self.switch:
            return out
        return out, self._balancing_loss(scores, idx)

    def _run_experts(self, routed: moe_ops.Dispatch) -> torch.Tensor:
        if self.world > 1 and self.exchange_kind == "peer" and routed.packed.is_cuda:
            from hivemind_b200.parallel.expert_exchange import PeerExchangeExperts

            exchange = self._get_exchange(routed.packed)
            answers, ok = PeerExchangeExperts.apply(routed.packed, routed.offsets, exchange,
                                                    lambda rows, gathered: self._run_local(gathered))
            return answers, ok.bool()
        if self.world > 1:
            return _AllToAllExperts.apply(routed.packed, routed.counts, self), None
        return self._run_local(routed), None

    def _get_exchange(self, packed: torch.Tensor):
        if self._exchange is None:
            from hivemind_b200.parallel.expert_exchange import PeerExpertExchange

            assert self.max_tokens > 0, 'exchange="peer" needs max_tokens (the largest batch of tokens per forward)'

            def all_descriptors(mine):
                gathered = [None] * self.world
                dist.all_gather_object(gathered, mine, group=self.group)
                return gathered

            self._exchange = PeerExpertExchange(
                rank=self.rank, world=self.world, experts_per_rank=self.experts_per_rank, hidden=packed.shape[1],
                max_rows=self.max_tokens * self.k_best, device=packed.device, dtype=packed.dtype,
                exchange_descriptors=all_descriptors, timeout=self.exchange_timeout)
        return self._exchange

    def _run_local(self, routed: moe_ops.Dispatch) -> torch.Tensor:
        """Apply this rank's experts to the rows that a dispatch over ``len(self.experts)`` experts assigned them."""
        if self.grouped:
            return self.experts(routed.packed, routed)  # no host synchronisation: empty tiles are skipped on the device
        bounds = routed.offsets.tolist()  # one small device-to-host read: per-expert launches need the row counts
        return _GroupedExperts.apply(routed.packed, bounds, list(self.experts), self.train_experts)

    def run_single_expert(self, local_index: int, rows: torch.Tensor) -> torch.Tensor:
        """Expert ``local_index`` of this rank applied to ``rows`` directly (for tests and debugging)."""
        if not self.grouped:
            return self.experts[local_index](rows)
        e = self.experts
        compute = rows.to(e.w1.dtype)
        hidden = torch.nn.functional.gelu(torch.nn.functional.linear(compute, e.w1[local_index], e.b1[local_index]),
                                          approximate="tanh")
        out = torch.nn.functional.linear(hidden, e.w2[local_index], e.b2[local_index])
        out = torch.nn.functional.layer_norm(compute + out, (e.hid_dim,), e.gamma[local_index], e.beta[local_index], 1e-12)
        return out.to(rows.dtype)

    def _balancing_loss(self, scores: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
        """Switch load balancing: per dimension, mean(probability mass * routed fraction) * size^2, summed."""
        parts = scores.split_with_sizes(self.grid_size, dim=-1)
        softmaxes = [torch.softmax(p, dim=-1) for p in parts]
        with torch.no_grad():
            coords = moe_ops.expert_coordinates(idx, self.grid_size)
            routed = (idx >= 0)
            used = []
            for d, size in enumerate(self.grid_size):
                hist = torch.bincount(coords[..., d][routed], minlength=size).float()
                used.append(hist / hist.sum().clamp(min=1.0))
            batch_utilization = torch.cat(used)
            if self.training:
                self.grid_utilization.mul_(self.utilization_alpha).add_((1 - self.utilization_alpha) * batch_utilization)
        utilization = self.grid_utilization.split_with_sizes(self.grid_size)
        return torch.stack([torch.mean(sm.mean(0) * u) * size ** 2
                            for sm, u, size in zip(softmaxes, utilization, self.grid_size)]).sum()


class _AllToAllExperts(torch.autograd.Function):
    """
    Expert-parallel step over a process group: rows sorted by global expert id are exchanged so that each rank
    receives the rows of its own experts from every rank, runs them, and sends the answers back the same way.
    """

    @staticmethod
    def forward(ctx, packed: torch.Tensor, counts: torch.Tensor, layer: DeviceMixtureOfExperts):
        world, per_rank, group = layer.world, layer.experts_per_rank, layer.group
        device = packed.device
        # counts of every (source rank, local expert): one small all-to-all, then one host read for the split sizes
        sent = counts.view(world, per_rank).to(torch.int64)
        received = torch.empty_like(sent)
        dist.all_to_all_single(received, sent, group=group)
        sent_host, received_host = sent.cpu(), received.cpu()
        send_splits = sent_host.sum(1).tolist()
        recv_splits = received_host.sum(1).tolist()
        incoming = torch.empty(sum(recv_splits), packed.shape[1], dtype=packed.dtype, device=device)
        dist.all_to_all_single(incoming, packed[:sum(send_splits)].contiguous(), recv_splits, send_splits, group=group)
        # regroup (source, expert)-ordered rows by expert with the dispatch kernel (k = 1)
        local_expert = torch.repeat_interleave(
            torch.arange(per_rank, device=device, dtype=torch.int32).repeat(world),
            received.reshape(-1).to(device), output_size=sum(recv_splits)).view(-1, 1)
        with torch.enable_grad():
            incoming.requires_grad_(packed.requires_grad)
            regrouped = moe_ops.dispatch(incoming, local_expert, per_rank,
                                         align=moe_ops.TILE_ROWS if layer.grouped else 1)
            answers = layer._run_local(regrouped)
            back = moe_ops.combine(answers, regrouped.pos, None, "sum")
        outgoing = torch.zeros_like(packed)
        dist.all_to_all_single(outgoing[:sum(send_splits)], back.detach(), send_splits, recv_splits, group=group)
        ctx.saved = (incoming, back, send_splits, recv_splits, group)
        return outgoing

    @staticmethod
    def backward(ctx, grad_out: torch.Tensor):
        incoming, back, send_splits, recv_splits, group = ctx.saved
        grad_back = torch.empty_like(back)
        dist.all_to_all_single(grad_back, grad_out[:sum(send_splits)].contiguous(), recv_splits, send_splits, group=group)
        torch.autograd.backward(back, grad_back)
        grad_in = torch.zeros_like(grad_out)
        grad_incoming = incoming.grad if incoming.grad is not None else torch.zeros_like(incoming)
        dist.all_to_all_single(grad_in[:sum(send_splits)], grad_incoming, send_splits, recv_splits, group=group)
        ctx.saved = None
        return grad_in, None, None

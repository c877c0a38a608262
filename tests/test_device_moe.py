"""Device mixture-of-experts: routing ops against dense PyTorch oracles (CPU formulas and, on a GPU, the kernels),
the layer against a per-token loop, and the expert-parallel all-to-all path against the single-rank layer."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hivemind_b200.ops import moe as moe_ops
from hivemind_b200.parallel.expert_parallel import DeviceMixtureOfExperts


def _dense_mixture(layer, x, scores, idx, mode):
    gate = moe_ops.expert_values(scores, idx, layer.grid_size, mode)
    if mode == "sum":
        weights = torch.softmax(gate.masked_fill(idx < 0, float("-inf")), 1).nan_to_num(0.0)
    else:
        weights = gate
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            if e >= 0:
                out[t] = out[t] + weights[t, j] * layer.experts[e](x[t:t + 1])[0]
    return out


def test_gate_topk_reference_properties():
    torch.manual_seed(0)
    grid = (3, 4, 2)
    scores = torch.randn(40, sum(grid))
    alive = torch.rand(24) > 0.4
    idx, val = moe_ops.gate_topk(scores, grid, 5, alive)
    assert idx.shape == (40, 5) and (val[:, :-1] >= val[:, 1:]).all()
    assert alive[idx[idx >= 0].long()].all()
    assert torch.allclose(val, moe_ops.expert_values(scores, idx, grid), atol=1e-6)
    full = sum(s.reshape([40] + [g if i == d else 1 for i, g in enumerate(grid)])
               for d, s in enumerate(scores.split_with_sizes(grid, 1))).reshape(40, -1)
    full[:, ~alive] = float("-inf")
    assert torch.allclose(val[:, 0], full.max(1).values)
    # fewer live experts than k -> padded with -1
    few = torch.zeros(24, dtype=torch.bool)
    few[[3, 7]] = True
    idx2, val2 = moe_ops.gate_topk(scores, grid, 4, few)
    assert (idx2[:, 2:] == -1).all() and (val2[:, 2:] == float("-inf")).all() and set(idx2[:, :2].unique().tolist()) == {3, 7}
    pidx, pval = moe_ops.gate_topk(scores, grid, 2, alive, mode="prob")
    assert (pval >= 0).all() and (pval <= 1).all()
    assert torch.allclose(pval, moe_ops.expert_values(scores, pidx, grid, "prob"), atol=1e-6)


def test_dispatch_combine_autograd_cpu():
    torch.manual_seed(1)
    tokens, k, experts, hidden = 33, 3, 7, 8
    idx = torch.randint(-1, experts, (tokens, k), dtype=torch.int32)
    x = torch.randn(tokens, hidden, requires_grad=True)
    gate = torch.randn(tokens, k, requires_grad=True)
    routed = moe_ops.dispatch(x, idx, experts)
    assert int(routed.offsets[-1]) == int((idx >= 0).sum())
    for e in range(experts):
        rows = routed.packed[routed.offsets[e]:routed.offsets[e + 1]]
        tok = (routed.src[routed.offsets[e]:routed.offsets[e + 1]] // k).long()
        assert torch.equal(rows, x[tok].detach()) and (idx.reshape(-1)[routed.src[routed.offsets[e]:routed.offsets[e + 1]].long()] == e).all()
    answers = routed.packed * 3.0
    out = moe_ops.combine(answers, routed.pos, gate, "softmax", residual=x)
    out.pow(2).sum().backward()
    x2, g2 = x.detach().clone().requires_grad_(True), gate.detach().clone().requires_grad_(True)
    w = torch.softmax(g2.masked_fill(idx < 0, float("-inf")), 1).nan_to_num(0.0)
    ref = x2 + (w.sum(1, keepdim=True) * 3.0 * x2)
    ref.pow(2).sum().backward()
    assert torch.allclose(out, ref, atol=1e-5) and torch.allclose(x.grad, x2.grad, atol=1e-4)
    assert torch.allclose(gate.grad, g2.grad, atol=1e-4)


@pytest.mark.parametrize("switch", [False, True])
def test_layer_matches_per_token_loop(switch):
    torch.manual_seed(2)
    layer = DeviceMixtureOfExperts(in_features=16, grid_size=(2, 3), k_best=1 if switch else 3, switch=switch,
                                   jitter_eps=0.0)
    layer.set_alive([1], False)
    x = torch.randn(9, 16, requires_grad=True)
    result = layer(x)
    out, aux = result if switch else (result, None)
    scores = layer.proj(x).float()
    mode = "prob" if switch else "sum"
    idx, _ = moe_ops.gate_topk(scores, layer.grid_size, layer.k_best, layer.alive, mode)
    assert not (idx == 1).any()
    ref = _dense_mixture(layer, x, scores, idx, mode) + (x if switch else 0)
    assert torch.allclose(out, ref, atol=1e-5)
    (out.pow(2).sum() + (aux if switch else 0)).backward()
    assert x.grad.norm() > 0 and layer.proj.weight.grad.norm() > 0
    used = sorted(set(idx[idx >= 0].tolist()))
    assert all(layer.experts[e].ffn.weight.grad is not None for e in used)
    if switch:
        assert aux > 0 and abs(float(layer.grid_utilization.sum()) - 2.0) < 1e-4
    strict = DeviceMixtureOfExperts(in_features=16, grid_size=(4,), k_best=2, k_min=2, check_k_min=True)
    strict.set_alive([0, 1, 2], False)
    with pytest.raises(RuntimeError):
        strict(x)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _expert_parallel_worker(rank, world, port, results):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(100)  # same full model everywhere, then every rank keeps its shard of experts
        full = DeviceMixtureOfExperts(in_features=16, grid_size=(2, 2), k_best=2)
        sharded = DeviceMixtureOfExperts(in_features=16, grid_size=(2, 2), k_best=2, group=dist.group.WORLD)
        sharded.proj.load_state_dict(full.proj.state_dict())
        for i, expert in enumerate(sharded.experts):
            expert.load_state_dict(full.experts[sharded.first_expert + i].state_dict())
        torch.manual_seed(200 + rank)  # every rank is a client with its own tokens
        x = torch.randn(11 + rank, 16, requires_grad=True)
        out = sharded(x)
        out.pow(2).sum().backward()
        x_ref = x.detach().clone().requires_grad_(True)
        ref = full(x_ref)
        ref.pow(2).sum().backward()
        ok = torch.allclose(out, ref, atol=1e-5) and torch.allclose(x.grad, x_ref.grad, atol=1e-4)
        # expert gradients: the sharded expert saw rows of all ranks, the full model only this rank's; sum over ranks
        local = torch.stack([e.ffn.weight.grad for e in sharded.experts])
        expected = torch.stack([full.experts[sharded.first_expert + i].ffn.weight.grad
                                if full.experts[sharded.first_expert + i].ffn.weight.grad is not None
                                else torch.zeros_like(e.ffn.weight) for i, e in enumerate(sharded.experts)])
        every = [torch.zeros(4, *expected.shape[1:]) for _ in range(world)]
        mine = torch.stack([full.experts[i].ffn.weight.grad if full.experts[i].ffn.weight.grad is not None
                            else torch.zeros_like(full.experts[i].ffn.weight) for i in range(4)])
        dist.all_gather(every, mine)
        total = sum(every)[sharded.first_expert:sharded.first_expert + len(sharded.experts)]
        ok = ok and torch.allclose(local, total, atol=1e-4)
        results.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_expert_parallel_matches_single_rank():
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_expert_parallel_worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(results.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(30)
    assert got == {0: True, 1: True}


# ------------------------------------------------------------------------------------------------------ GPU


@pytest.mark.gpu
@pytest.mark.parametrize("grid,k,mode", [((8, 8), 4, "sum"), ((64,), 1, "prob"), ((4, 4, 4), 8, "sum"), ((16, 4), 2, "prob")])
def test_gate_topk_kernel(grid, k, mode):
    torch.manual_seed(0)
    scores = torch.randn(1000, sum(grid), device="cuda")
    if mode == "prob":
        scores[:, 1] = float("-inf")  # a dropped coordinate
    n = 1
    for g in grid:
        n *= g
    alive = torch.rand(n, device="cuda") > 0.3
    idx, val = moe_ops.gate_topk(scores, grid, k, alive, mode)
    ridx, rval = moe_ops.gate_topk_reference(scores.cpu(), grid, k, alive.cpu(), mode)
    assert torch.allclose(val.cpu(), rval, atol=1e-5, rtol=1e-5)
    # ids may differ only where values tie
    differs = idx.cpu() != ridx
    assert (val.cpu()[differs] - rval[differs]).abs().max() < 1e-5 if differs.any() else True
    assert alive[idx[idx >= 0].long()].all()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_dispatch_combine_kernels(dtype):
    torch.manual_seed(1)
    tokens, k, experts, hidden = 777, 4, 13, 256
    idx = torch.randint(-1, experts, (tokens, k), dtype=torch.int32, device="cuda")
    x = torch.randn(tokens, hidden, device="cuda", dtype=dtype, requires_grad=True)
    gate = torch.randn(tokens, k, device="cuda", requires_grad=True)
    keep = torch.rand(tokens, k, device="cuda") > 0.2
    routed = moe_ops.dispatch(x, idx, experts)
    counts = torch.bincount(idx[idx >= 0].long(), minlength=experts)
    assert torch.equal(routed.counts.long(), counts) and int(routed.offsets[-1]) == int(counts.sum())
    total = int(routed.offsets[-1])
    src = routed.src[:total].long()
    assert torch.equal(routed.packed[:total], x.detach()[src // k])
    expert_of_row = torch.repeat_interleave(torch.arange(experts, device="cuda"), counts)
    assert torch.equal(idx.reshape(-1)[src].long(), expert_of_row)
    answers = (routed.packed.float() * (1 + expert_of_row.float()[:, None] / experts)).to(dtype)
    answers = torch.cat([answers[:total], torch.zeros(tokens * k - total, hidden, device="cuda", dtype=dtype)]) \
        if answers.shape[0] != tokens * k else answers
    answers = answers.detach().requires_grad_(True)
    for mode in ("softmax", "prob", "sum"):
        for t in (x, gate, answers):
            t.grad = None
        out = moe_ops.combine(answers, routed.pos, gate, mode, keep=keep, residual=x)
        probe = torch.randn_like(out)
        (out.float() * probe.float()).sum().backward()
        ref_y = answers.detach().float().cpu().requires_grad_(True)
        ref_g = gate.detach().cpu().requires_grad_(True)
        ref_x = x.detach().float().cpu().requires_grad_(True)
        ref, _ = moe_ops._combine_reference(ref_y, routed.pos.cpu(), ref_g, keep.cpu(), ref_x,
                                            {"softmax": 0, "prob": 1, "sum": 2}[mode])
        (ref * probe.float().cpu()).sum().backward()
        tol = 3e-2 if dtype == torch.bfloat16 else 1e-4
        assert torch.allclose(out.float().cpu(), ref, atol=tol, rtol=tol), mode
        assert torch.allclose(answers.grad.float().cpu(), ref_y.grad, atol=tol, rtol=tol), mode
        if mode != "sum":
            scale = ref_g.grad.abs().max().item() + 1e-6
            assert (gate.grad.cpu() - ref_g.grad).abs().max().item() <= (5e-2 if dtype == torch.bfloat16 else 1e-3) * scale, mode
    # backward of dispatch: the sum over a token's routed slots
    x.grad = None
    routed.packed.backward(torch.ones_like(routed.packed))
    assert torch.allclose(x.grad.float(), (idx >= 0).sum(1, keepdim=True).float().expand(-1, hidden))


@pytest.mark.gpu
def test_masked_softmax_combine_kernel():
    torch.manual_seed(3)
    logits = torch.randn(64, 4, device="cuda", requires_grad=True)
    mask = torch.rand(64, 4, device="cuda") > 0.3
    mask[5] = False
    outputs = torch.randn(64, 4, 96, device="cuda", requires_grad=True)
    mixed = moe_ops.masked_softmax_combine(logits, mask, outputs)
    mixed.pow(2).sum().backward()
    l2, o2 = logits.detach().clone().requires_grad_(True), outputs.detach().clone().requires_grad_(True)
    w = torch.softmax(l2.masked_fill(~mask, float("-inf")), 1).nan_to_num(0.0)
    ref = (w[..., None] * o2).sum(1)
    ref.pow(2).sum().backward()
    assert torch.allclose(mixed, ref, atol=1e-5) and (mixed[5] == 0).all()
    assert torch.allclose(logits.grad, l2.grad, atol=1e-4) and torch.allclose(outputs.grad, o2.grad, atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("switch", [False, True])
def test_layer_on_gpu_matches_fp32_oracle(switch):
    torch.manual_seed(4)
    layer = DeviceMixtureOfExperts(in_features=256, grid_size=(4, 4), k_best=1 if switch else 4, switch=switch,
                                   jitter_eps=0.0).cuda()
    layer.set_alive([3, 9], False)
    x = torch.randn(512, 256, device="cuda", requires_grad=True)
    result = layer(x)
    out = result[0] if switch else result
    out.float().pow(2).mean().backward()
    oracle = DeviceMixtureOfExperts(in_features=256, grid_size=(4, 4), k_best=layer.k_best, switch=switch, jitter_eps=0.0)
    oracle.load_state_dict({k: v.cpu() for k, v in layer.state_dict().items()})
    x_ref = x.detach().cpu().requires_grad_(True)
    ref_result = oracle(x_ref)
    ref = ref_result[0] if switch else ref_result
    ref.pow(2).mean().backward()
    assert (out.float().cpu() - ref).abs().max() < 0.06 and (out.float().cpu() - ref).pow(2).mean().sqrt() < 0.01
    assert torch.allclose(x.grad.cpu(), x_ref.grad, atol=2e-3, rtol=0.1)
    g_gpu, g_ref = layer.experts[0].ffn.weight.grad.cpu(), oracle.experts[0].ffn.weight.grad
    assert (g_gpu - g_ref).norm() <= 0.05 * g_ref.norm() + 1e-6

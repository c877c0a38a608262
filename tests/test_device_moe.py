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
                out[t] = out[t] + weights[t, j] * layer.run_single_expert(e, x[t:t + 1])[0]
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
    assert all(layer.experts.w1.grad[e].norm() > 0 for e in used)
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
        lo, hi = sharded.first_expert, sharded.first_expert + sharded.experts_per_rank
        with torch.no_grad():
            for name, param in sharded.experts.named_parameters():
                param.copy_(dict(full.experts.named_parameters())[name][lo:hi])
        torch.manual_seed(200 + rank)  # every rank is a client with its own tokens
        x = torch.randn(11 + rank, 16, requires_grad=True)
        out = sharded(x)
        out.pow(2).sum().backward()
        x_ref = x.detach().clone().requires_grad_(True)
        ref = full(x_ref)
        ref.pow(2).sum().backward()
        ok = torch.allclose(out, ref, atol=1e-5) and torch.allclose(x.grad, x_ref.grad, atol=1e-4)
        # expert gradients: a sharded expert saw the rows of all ranks, the full model only this rank's: sum over ranks
        mine = full.experts.w1.grad.clone()
        every = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        ok = ok and torch.allclose(sharded.experts.w1.grad, sum(every)[lo:hi], atol=1e-4)
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
    answers = torch.zeros(tokens * k, hidden, device="cuda", dtype=dtype)
    answers[:total] = (routed.packed[:total].float() * (1 + expert_of_row.float()[:, None] / experts)).to(dtype)
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
    g_gpu, g_ref = layer.experts.w1.grad.cpu(), oracle.experts.w1.grad
    assert (g_gpu - g_ref).norm() <= 0.05 * g_ref.norm() + 1e-6


@pytest.mark.gpu
def test_aligned_dispatch_kernel():
    torch.manual_seed(5)
    tokens, k, experts, hidden = 1000, 2, 9, 128
    idx = torch.randint(-1, experts, (tokens, k), dtype=torch.int32, device="cuda")
    idx[idx == 4] = -1  # an expert with no rows
    x = torch.randn(tokens, hidden, device="cuda", dtype=torch.bfloat16)
    routed = moe_ops.dispatch(x, idx, experts, align=128)
    counts = torch.bincount(idx[idx >= 0].long(), minlength=experts)
    padded = (counts + 127) // 128 * 128
    assert torch.equal(routed.counts.long(), counts)
    assert torch.equal(routed.offsets.long(), torch.cat([torch.zeros(1, device="cuda", dtype=torch.long), padded.cumsum(0)]))
    offsets = routed.offsets.tolist()
    for e in range(experts):
        lo, n, hi = offsets[e], int(counts[e]), offsets[e + 1]
        src = routed.src[lo:lo + n].long()
        assert (idx.reshape(-1)[src] == e).all() and torch.equal(routed.packed[lo:lo + n], x[src // k])
        assert (routed.src[lo + n:hi] == -1).all() and (routed.packed[lo + n:hi] == 0).all()
        assert (routed.tile_group[lo // 128:hi // 128] == e).all()
    assert (routed.tile_group[offsets[-1] // 128:] == -1).all()
    assert torch.equal(routed.packed[routed.pos[idx >= 0].long()], x[(idx >= 0).nonzero()[:, 0]])


@pytest.mark.gpu
def test_grouped_gemm_modes():
    from hivemind_b200.ops.gemm import check_kernel_errors
    from hivemind_b200.ops.grouped_ffn import tc_gemm_grouped

    torch.manual_seed(6)
    groups, n, k = 5, 384, 256
    rows_per_group = [256, 0, 128, 384, 128]
    table = torch.tensor([g for g, r in enumerate(rows_per_group) for _ in range(r // 128)] + [-1, -1],
                         dtype=torch.int32, device="cuda")
    m = table.numel() * 128
    a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(groups, n, k, device="cuda", dtype=torch.bfloat16) / 16
    bias = torch.randn(groups, n, device="cuda")
    out = torch.full((m, n), 7.0, device="cuda", dtype=torch.bfloat16)
    aux = torch.full((m, n), 7.0, device="cuda", dtype=torch.bfloat16)
    tc_gemm_grouped(a, b.view(groups * n, k), out, table, mode=1, num_groups=groups, m=m, n=n, k=k, bias=bias, gelu=True,
                    aux=aux)
    check_kernel_errors()
    for t, g in enumerate(table.tolist()):
        rows = slice(t * 128, (t + 1) * 128)
        if g < 0:
            assert (out[rows] == 7.0).all() and (aux[rows] == 7.0).all()  # skipped tiles are not touched
            continue
        pre = a[rows].float() @ b[g].float().t() + bias[g]
        assert torch.allclose(aux[rows].float(), pre, atol=0.06, rtol=0.02)
        assert torch.allclose(out[rows].float(), torch.nn.functional.gelu(pre, approximate="tanh"), atol=0.06, rtol=0.02)
    # the same with B stored [k][n] per group (the data-gradient layout)
    bt = b.transpose(1, 2).contiguous()  # [groups, k, n]
    out2 = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
    tc_gemm_grouped(a, bt.view(groups * k, n), out2, table, mode=1, num_groups=groups, m=m, n=n, k=k, b_mn=True)
    for t, g in enumerate(table.tolist()):
        if g >= 0:
            ref = a[t * 128:(t + 1) * 128].float() @ b[g].float().t()
            assert torch.allclose(out2[t * 128:(t + 1) * 128].float(), ref, atol=0.06, rtol=0.02)
    # mode 2: per-group contraction ranges, accumulated into fp32
    offsets = torch.tensor([0, 256, 256, 384, 768, 896], dtype=torch.int32, device="cuda")
    left = torch.randn(m, 256, device="cuda", dtype=torch.bfloat16)   # [K rows][M]
    right = torch.randn(m, 384, device="cuda", dtype=torch.bfloat16)  # [K rows][N]
    acc = torch.ones(groups, 256, 384, device="cuda")
    tc_gemm_grouped(left, right, acc, offsets, mode=2, num_groups=groups, m=256, n=384, k=m, a_mn=True, b_mn=True,
                    reduce_add=True)
    check_kernel_errors()
    for g in range(groups):
        lo, hi = int(offsets[g]), int(offsets[g + 1])
        ref = 1.0 + left[lo:hi].float().t() @ right[lo:hi].float()
        assert torch.allclose(acc[g], ref, atol=0.05, rtol=0.01), g


@pytest.mark.gpu
def test_grouped_ffn_matches_fp32_reference():
    from hivemind_b200.ops.grouped_ffn import GroupedFeedforward

    torch.manual_seed(7)
    experts, hidden, tokens, k = 6, 256, 700, 2
    module = GroupedFeedforward(experts, hidden).cuda()
    oracle = GroupedFeedforward(experts, hidden)
    oracle.load_state_dict({name: value.cpu() for name, value in module.state_dict().items()})
    idx = torch.randint(-1, experts, (tokens, k), dtype=torch.int32, device="cuda")
    idx[idx == 2] = -1
    x = torch.randn(tokens, hidden, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    routed = moe_ops.dispatch(x, idx, experts, align=128)
    y = module(routed.packed, routed)
    probe = torch.randn_like(y) * (routed.src >= 0).unsqueeze(1)  # pad rows receive no gradient, as after combine
    (y.float() * probe.float()).sum().backward()
    x_ref = x.detach().float().cpu().requires_grad_(True)
    routed_ref = moe_ops.dispatch(x_ref, idx.cpu(), experts, align=128)
    # the kernel's row order inside an expert is arbitrary: compare token by token through pos
    y_ref = oracle(routed_ref.packed, routed_ref)
    sel = (idx >= 0).cpu()
    got = y.float().cpu()[routed.pos.cpu()[sel].long()]
    want = y_ref[routed_ref.pos[sel].long()]
    assert (got - want).abs().max() < 0.08 and (got - want).pow(2).mean().sqrt() < 0.012
    probe_ref = torch.zeros_like(y_ref)
    probe_ref[routed_ref.pos[sel].long()] = probe.float().cpu()[routed.pos.cpu()[sel].long()]
    (y_ref * probe_ref).sum().backward()
    assert (x.grad.float().cpu() - x_ref.grad).norm() <= 0.03 * x_ref.grad.norm()
    for name in ("w1", "b1", "w2", "b2", "gamma", "beta"):
        g_gpu, g_ref = getattr(module, name).grad.cpu(), getattr(oracle, name).grad
        assert (g_gpu - g_ref).norm() <= 0.03 * g_ref.norm() + 1e-5, name
        assert g_gpu[2].abs().max() == 0  # the expert without rows gets no gradient


def _cli_server_roundtrip(tmp_path, device):
    """An expert server (a child process started through the CLI) called from CUDA client tensors.

    The server runs in its own process on purpose: a client layer blocks autograd's CUDA worker thread while it waits
    for the experts' backward pass, and a server in the same process would need that very thread for its own backward.
    """
    import re
    import signal
    import subprocess
    import sys
    import time

    from hivemind_b200.dht import DHT
    from hivemind_b200.moe import RemoteMixtureOfExperts

    env = dict(os.environ, PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))), PYTHONUNBUFFERED="1")
    log_path = tmp_path / "server.log"
    with open(log_path, "w") as log:
        proc = subprocess.Popen([sys.executable, "-m", "hivemind_b200.hivemind_cli.run_server", "--expert_uids", "gpu.0",
                                 "gpu.1", "gpu.2", "gpu.3", "--hidden_dim", "256", "--device", device, "--optimizer", "sgd",
                                 "--num_handlers", "2", "--host_maddrs", "/ip4/127.0.0.1/tcp/0"],
                                stderr=log, stdout=log, env=env, cwd=str(tmp_path))
    try:
        maddr, deadline = None, time.time() + 120
        while time.time() < deadline and proc.poll() is None:
            text = log_path.read_text()
            found = re.search(r"Running DHT node on \['(/ip4/127\.0\.0\.1/tcp/\d+/p2p/\S+?)'", text)
            if found and " Started" in text:
                maddr = found.group(1)
                break
            time.sleep(0.5)
        assert maddr is not None, log_path.read_text()[-2000:]
        dht = DHT(initial_peers=[maddr], start=True)
        try:
            moe = RemoteMixtureOfExperts(in_features=256, grid_size=(4,), dht=dht, uid_prefix="gpu.", k_best=2,
                                         forward_timeout=60, backward_timeout=60).to(device)
            x = torch.randn(32, 256, device=device, requires_grad=True)
            out = None
            for attempt in range(20):  # declarations reach the DHT a moment after the server reports "Started"
                try:
                    out = moe(x)
                    break
                except RuntimeError:
                    time.sleep(0.5)
            assert out is not None and out.shape == x.shape and out.device.type == device and out.isfinite().all()
            out.pow(2).mean().backward()
            assert x.grad is not None and x.grad.isfinite().all() and moe.proj.weight.grad.norm() > 0
        finally:
            dht.shutdown()
    finally:
        proc.send_signal(signal.SIGTERM)
        try:
            proc.wait(30)
        except subprocess.TimeoutExpired:
            proc.kill()


def test_cli_server_roundtrip_cpu(tmp_path):
    _cli_server_roundtrip(tmp_path, "cpu")


@pytest.mark.gpu
def test_server_with_experts_on_gpu(tmp_path):
    _cli_server_roundtrip(tmp_path, "cuda")


@pytest.mark.gpu
def test_peer_exchange_stages_emulated_on_one_gpu():
    """Three ranks of the peer-memory exchange on one GPU, stage by stage (no launch ever waits for a later one)."""
    from hivemind_b200.parallel.expert_exchange import BACKWARD, FORWARD, PeerExpertExchange

    torch.manual_seed(8)
    world, per_rank, hidden, k = 3, 2, 128, 2
    experts = world * per_rank
    dev = torch.device("cuda", 0)
    tokens = [50, 0, 300]  # one client sends nothing
    exchanges = [PeerExpertExchange(rank=r, world=world, experts_per_rank=per_rank, hidden=hidden, max_rows=300 * k,
                                    device=dev, timeout=1.0) for r in range(world)]
    descriptors = [e.descriptor for e in exchanges]
    for e in exchanges:
        e.connect(descriptors)
    xs = [torch.randn(t, hidden, device=dev, dtype=torch.bfloat16) for t in tokens]
    idxs = [torch.randint(-1, experts, (t, k), dtype=torch.int32, device=dev) for t in tokens]
    routed = [moe_ops.dispatch(x, idx, experts) for x, idx in zip(xs, idxs)]
    for phase in (FORWARD, BACKWARD):
        for r, e in enumerate(exchanges):
            e.client_publish(routed[r].packed * (1 if phase == FORWARD else -1), routed[r].offsets if phase == FORWARD else None,
                             phase, epoch=1)
        torch.cuda.synchronize()
        gathered = [e.server_gather(phase, epoch=1) for e in exchanges]
        torch.cuda.synchronize()
        for d, g in enumerate(gathered):
            assert int(g.status[0]) == 0
            offs = g.offsets.tolist()
            assert all(o % 128 == 0 for o in offs)
            for el in range(per_rank):
                ge = d * per_rank + el
                want = torch.cat([(routed[s].packed * (1 if phase == FORWARD else -1))[int(routed[s].offsets[ge]):int(routed[s].offsets[ge + 1])]
                                  for s in range(world)])
                got = g.packed[offs[el]:offs[el] + want.shape[0]]
                assert torch.equal(got, want), (phase, d, el)
                assert (g.packed[offs[el] + want.shape[0]:offs[el + 1]] == 0).all()
                assert (g.tile_group[offs[el] // 128:offs[el + 1] // 128] == el).all()
            assert (g.tile_group[offs[-1] // 128:] == -1).all()
        # the "experts": scale every row by (1 + global expert id)
        for d, (e, g) in enumerate(zip(exchanges, gathered)):
            offs = g.offsets.tolist()
            answers = torch.zeros_like(g.packed)
            for el in range(per_rank):
                answers[offs[el]:offs[el + 1]] = g.packed[offs[el]:offs[el + 1]] * (1 + d * per_rank + el)
            e.server_publish(answers, phase, epoch=1)
        torch.cuda.synchronize()
        for r, e in enumerate(exchanges):
            total = int(routed[r].offsets[-1])
            out, ok = e.client_pull(routed[r].offsets, routed[r].packed.shape[0], phase, epoch=1)
            torch.cuda.synchronize()
            scale = 1 + torch.repeat_interleave(torch.arange(experts, device=dev), routed[r].counts.long())
            want = (routed[r].packed[:total] * (1 if phase == FORWARD else -1)).float() * scale[:, None]
            assert torch.allclose(out[:total].float(), want, rtol=1e-2, atol=1e-2) and ok[:total].all()
    # a server that never answers: the client gives up after the timeout and reports the rows as failed
    exchanges[0].client_publish(routed[0].packed, routed[0].offsets, FORWARD, epoch=2)
    out, ok = exchanges[0].client_pull(routed[0].offsets, routed[0].packed.shape[0], FORWARD, epoch=2)
    torch.cuda.synchronize()
    total = int(routed[0].offsets[-1])
    assert not ok[:total].any() and (out[:total] == 0).all()
    for e in exchanges:
        e.close()


@pytest.mark.gpu
def test_client_that_the_servers_gave_up_on_gets_failed_rows_not_somebody_elses():
    """Host-side injection: client 2 skips its publish step, so every server's bounded wait for its flag runs out and
    lays it out with zero rows. When that client later pulls, the segment lengths that the servers published tell it
    that none of its rows were taken: ok = 0 and zeros, instead of rows of the clients that were served."""
    from hivemind_b200.parallel.expert_exchange import FORWARD, PeerExpertExchange

    torch.manual_seed(9)
    world, per_rank, hidden, k = 3, 2, 128, 2
    experts = world * per_rank
    dev = torch.device("cuda", 0)
    exchanges = [PeerExpertExchange(rank=r, world=world, experts_per_rank=per_rank, hidden=hidden, max_rows=200 * k,
                                    device=dev, timeout=0.3) for r in range(world)]
    for e in exchanges:
        e.connect([x.descriptor for x in exchanges])
    xs = [torch.randn(100, hidden, device=dev, dtype=torch.bfloat16) for _ in range(world)]
    idxs = [torch.randint(0, experts, (100, k), dtype=torch.int32, device=dev) for _ in range(world)]
    routed = [moe_ops.dispatch(x, idx, experts) for x, idx in zip(xs, idxs)]
    late = 2
    for r, e in enumerate(exchanges):
        if r != late:
            e.client_publish(routed[r].packed, routed[r].offsets, FORWARD, epoch=1)
    torch.cuda.synchronize()
    gathered = [e.server_gather(FORWARD, epoch=1) for e in exchanges]  # each waits 0.3 s for the late client, then goes on
    torch.cuda.synchronize()
    assert all(int(g.status[0]) == 1 << late for g in gathered)
    for e, g in zip(exchanges, gathered):
        e.server_publish(g.packed * 2, FORWARD, epoch=1)
    # the late client publishes after the servers have moved on, then pulls
    exchanges[late].client_publish(routed[late].packed, routed[late].offsets, FORWARD, epoch=1)
    torch.cuda.synchronize()
    for r, e in enumerate(exchanges):
        total = int(routed[r].offsets[-1])
        out, ok = e.client_pull(routed[r].offsets, routed[r].packed.shape[0], FORWARD, epoch=1)
        torch.cuda.synchronize()
        if r == late:
            assert not ok[:total].any() and (out[:total] == 0).all()
        else:
            assert ok[:total].all()
            assert torch.allclose(out[:total].float(), routed[r].packed[:total].float() * 2, rtol=1e-2, atol=1e-2)
    for e in exchanges:
        e.close()

"""Device butterfly across processes (one per GPU) through the full DecentralizedAverager: matchmaking over the DHT,
IPC handle exchange in the gather blob, kernels over peer-mapped memory. Needs at least two GPUs."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

CHILD = r'''
import os, sys, time, json, torch
sys.path.insert(0, os.environ["REPO_ROOT"])
rank, world = int(sys.argv[1]), int(sys.argv[2])
codec_name = sys.argv[3]
import hivemind_b200 as hivemind
from hivemind_b200.averaging import DecentralizedAverager
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
if rank == 0:
    dht = hivemind.DHT(start=True)
    with open(os.environ["MADDR_FILE"] + ".tmp", "w") as f:
        json.dump([str(m) for m in dht.get_visible_maddrs()], f)
    os.rename(os.environ["MADDR_FILE"] + ".tmp", os.environ["MADDR_FILE"])
else:
    while not os.path.exists(os.environ["MADDR_FILE"]):
        time.sleep(0.05)
    dht = hivemind.DHT(initial_peers=json.load(open(os.environ["MADDR_FILE"])), start=True)
torch.manual_seed(100 + rank)
tensors = [torch.randn(300000, device=dev), torch.randn(257, 129, device=dev)]
original = [t.clone() for t in tensors]
codec = getattr(hivemind, codec_name)()
averager = DecentralizedAverager(tensors, dht, start=True, prefix="mgpu", target_group_size=world,
                                 min_matchmaking_time=3.0, request_timeout=1.0, compression=codec,
                                 part_size_bytes=2 ** 16, sender_timeout=5.0)
assert averager._device_endpoint is not None
weight = 1.0 + rank
gathered = averager.step(weight=weight, gather=dict(rank=rank), timeout=60)
torch.cuda.synchronize()
assert len(gathered) == world
with averager.get_tensors() as out:
    result = [t.cpu() for t in out]
torch.save(dict(original=[t.cpu() for t in original], result=result, weight=weight), os.environ["OUT_PREFIX"] + f"{rank}.pt.tmp")
os.rename(os.environ["OUT_PREFIX"] + f"{rank}.pt.tmp", os.environ["OUT_PREFIX"] + f"{rank}.pt")
# groupmates may still be pulling deltas out of this process's arena: leave (and free GPU memory) only when all are done
deadline = time.time() + 120
while time.time() < deadline and not all(os.path.exists(os.environ["OUT_PREFIX"] + f"{r}.pt") for r in range(world)):
    time.sleep(0.05)
averager.shutdown(); dht.shutdown()
print("child done", rank, flush=True)
'''


@pytest.mark.parametrize("codec_name,tol", [("NoCompression", 1e-5), ("Float16Compression", 5e-3),
                                            ("Uniform8BitQuantization", 0.05)])
def test_two_processes_average_over_ipc(tmp_path, codec_name, tol):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, REPO_ROOT=os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
               MADDR_FILE=str(tmp_path / "maddrs.json"), OUT_PREFIX=str(tmp_path / "out"), NCCL_NVLS_ENABLE="0")
    script = tmp_path / "child.py"
    script.write_text(CHILD)
    procs = [subprocess.Popen([sys.executable, str(script), str(r), str(world), codec_name], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outputs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outputs.append(out)
    assert all(p.returncode == 0 for p in procs), "\n".join(o[-2000:] for o in outputs)
    data = [torch.load(str(tmp_path / f"out{r}.pt")) for r in range(world)]
    total_w = sum(d["weight"] for d in data)
    for k in range(2):
        ref = sum(d["original"][k] * d["weight"] for d in data) / total_w
        spread = ref.std().item() + 1e-6
        for d in data:
            rms = (d["result"][k] - ref).pow(2).mean().sqrt().item()
            assert rms <= tol * max(spread, 1.0), (codec_name, k, rms)


STALL_CHILD = CHILD.replace(
    'weight = 1.0 + rank',
    'weight = 1.0\nif rank == world - 1:\n    averager._device_endpoint.fault_publish_half = True  # host-side injection'
).replace('part_size_bytes=2 ** 16, sender_timeout=5.0', 'part_size_bytes=2 ** 16, sender_timeout=1.0')


def test_peer_that_stalls_after_half_of_its_parts_is_excluded_from_the_rest(tmp_path):
    """The fault variant of the averaging benchmark, injected on the host: the last rank launches its send items only
    for the first half of the parts it owes, then carries on with its reduce and apply work. The other ranks wait
    ``sender_timeout`` (1 s) once, ban it, and finish with the survivors' average for the parts it never published;
    nobody hangs and every process leaves between rounds. NVLS is off and the kernels use plain peer loads."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, REPO_ROOT=os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
               MADDR_FILE=str(tmp_path / "maddrs.json"), OUT_PREFIX=str(tmp_path / "out"), NCCL_NVLS_ENABLE="0")
    script = tmp_path / "child.py"
    script.write_text(STALL_CHILD)
    procs = [subprocess.Popen([sys.executable, str(script), str(r), str(world), "NoCompression"], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outputs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outputs.append(out)
    assert all(p.returncode == 0 for p in procs), "\n".join(o[-2000:] for o in outputs)
    data = [torch.load(str(tmp_path / f"out{r}.pt")) for r in range(world)]
    stalled = world - 1
    everybody = [sum(d["original"][k] for d in data) / world for k in range(2)]
    survivors = [sum(d["original"][k] for r, d in enumerate(data) if r != stalled) / max(world - 1, 1) for k in range(2)]
    saw_exclusion = False
    for r, d in enumerate(data):
        if r == stalled:
            continue
        for k in range(2):
            got = d["result"][k]
            with_all = (got - everybody[k]).abs() < 1e-4
            without = (got - survivors[k]).abs() < 1e-4
            if world == 2:  # the only survivor keeps its own values where the other one never showed up
                without = (got - d["original"][k]).abs() < 1e-6
            assert bool((with_all | without).all()), (r, k)
            saw_exclusion = saw_exclusion or bool((without & ~with_all).any())
    assert saw_exclusion, "the stalled rank was averaged in everywhere"


MOE_CHILD = r'''
import os, sys, torch
import torch.distributed as dist
sys.path.insert(0, os.environ["REPO_ROOT"])
from hivemind_b200.parallel.expert_parallel import DeviceMixtureOfExperts
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
layers = {}
for kind in ("all_to_all", "peer"):
    torch.manual_seed(7)  # same gate everywhere; every rank keeps the experts of its own shard of a common draw
    layer = DeviceMixtureOfExperts(in_features=256, grid_size=(2, 4), k_best=2, group=dist.group.WORLD, exchange=kind,
                                   max_tokens=512, exchange_timeout=5.0).cuda()
    layers[kind] = layer
layers["peer"].load_state_dict(layers["all_to_all"].state_dict())
torch.manual_seed(500 + rank)
x = torch.randn(300 + 50 * rank, 256, device="cuda")
outs, grads, wgrads = {}, {}, {}
for kind, layer in layers.items():
    xi = x.clone().requires_grad_(True)
    out = layer(xi)
    out.float().pow(2).mean().backward()
    torch.cuda.synchronize()
    outs[kind], grads[kind], wgrads[kind] = out.detach().float(), xi.grad.float(), layer.experts.w1.grad.clone()
ok = (outs["peer"] - outs["all_to_all"]).abs().max().item() < 2e-2
ok = ok and (grads["peer"] - grads["all_to_all"]).norm().item() <= 0.02 * grads["all_to_all"].norm().item() + 1e-6
ok = ok and (wgrads["peer"] - wgrads["all_to_all"]).norm().item() <= 0.02 * wgrads["all_to_all"].norm().item() + 1e-6
flag = torch.tensor([1.0 if ok else 0.0], device="cuda")
dist.all_reduce(flag, op=dist.ReduceOp.MIN)
dist.barrier()
torch.cuda.synchronize()
print("moe child", rank, "ok" if ok else "MISMATCH", float(flag), flush=True)
dist.destroy_process_group()
sys.exit(0 if float(flag) == 1.0 else 1)
'''


def test_moe_peer_exchange_matches_all_to_all(tmp_path):
    """Expert-parallel layer over 2-4 GPUs: rows pulled over NVLink by our kernels vs the NCCL all-to-all path."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = min(torch.cuda.device_count(), 4)
    script = tmp_path / "moe_child.py"
    script.write_text(MOE_CHILD)
    import socket
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    env = dict(os.environ, REPO_ROOT=os.path.dirname(os.path.dirname(os.path.abspath(__file__))), NCCL_NVLS_ENABLE="0",
               MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE=str(world))
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r), LOCAL_RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outputs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outputs.append(out)
    assert all(p.returncode == 0 for p in procs), "\n".join(o[-2000:] for o in outputs)


POWERSGD_CHILD = r'''
import os, sys, time, json, torch
sys.path.insert(0, os.environ["REPO_ROOT"])
rank, world = int(sys.argv[1]), int(sys.argv[2])
import hivemind_b200 as hivemind
from hivemind_b200.optim import PowerSGDGradientAverager
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
if rank == 0:
    dht = hivemind.DHT(start=True)
    with open(os.environ["MADDR_FILE"] + ".tmp", "w") as f:
        json.dump([str(m) for m in dht.get_visible_maddrs()], f)
    os.rename(os.environ["MADDR_FILE"] + ".tmp", os.environ["MADDR_FILE"])
else:
    while not os.path.exists(os.environ["MADDR_FILE"]):
        time.sleep(0.05)
    dht = hivemind.DHT(initial_peers=json.load(open(os.environ["MADDR_FILE"])), start=True)
torch.manual_seed(0)  # the same low-rank factors on every rank; the ranks differ by a scale and a sample count
u, v = torch.randn(256, 8).to(dev), torch.randn(8, 128).to(dev)
scales, samples = [1.0 + r for r in range(world)], [8 + 10 * r for r in range(world)]
params = [torch.nn.Parameter(torch.zeros(256, 128, device=dev)), torch.nn.Parameter(torch.zeros(64, device=dev))]
averager = PowerSGDGradientAverager(params, averager_rank=8, dht=dht, prefix="psgd_gpu", target_group_size=world,
                                    min_matchmaking_time=3.0, request_timeout=1.0, min_compression_ratio=0.0,
                                    q_init="normal", sender_timeout=5.0, start=True)
assert averager._p_endpoint is not None and averager._q_endpoint is not None, "the device path must be active"
torch.manual_seed(10 + rank)  # different starting Q on every rank, as in a real swarm
for q in averager._qs:
    q.copy_(torch.randn_like(q))
mean_scale = sum(s * n for s, n in zip(scales, samples)) / sum(samples)
ok = True
for round_index in range(2):  # the second round reuses the arenas and starts from the error feedback of the first
    params[0].grad = scales[rank] * (u @ v)
    params[1].grad = torch.full((64,), scales[rank], device=dev)
    control = averager.schedule_step(timeout=60)
    averager.accumulate_grads_(batch_size=samples[rank])
    averager.step(control=control, wait=True, timeout=60)
    torch.cuda.synchronize()
    expected = mean_scale * (u @ v)
    with averager.use_averaged_gradients():
        got_w, got_b = params[0].grad.clone(), params[1].grad.clone()
    if round_index == 0:
        err_w = ((got_w - expected).norm() / expected.norm()).item()
        err_b = (got_b - mean_scale).abs().max().item()
        residual = ((averager._ms[0] - (scales[rank] - mean_scale) * (u @ v)).norm() / expected.norm()).item()
        ok = ok and err_w < 2e-2 and err_b < 1e-4 and residual < 2e-2
        print("powersgd child", rank, "round 0", err_w, err_b, residual, flush=True)
    else:
        # every rank adds its residual (scale - mean) u v to the same new gradient: the average is again mean_scale u v
        err_w = ((got_w - expected).norm() / expected.norm()).item()
        ok = ok and err_w < 4e-2
        print("powersgd child", rank, "round 1", err_w, flush=True)
    averager.reset_accumulated_grads_()
with open(os.environ["OUT_PREFIX"] + f"{rank}.done", "w") as f:
    f.write("ok" if ok else "mismatch")
deadline = time.time() + 120
while time.time() < deadline and not all(os.path.exists(os.environ["OUT_PREFIX"] + f"{r}.done") for r in range(world)):
    time.sleep(0.05)
averager.shutdown(); dht.shutdown()
sys.exit(0 if ok else 1)
'''


def test_powersgd_factors_average_over_peer_memory(tmp_path):
    """PowerSGDGradientAverager with its P and Q arenas on two GPUs: gradients that share a rank-8 subspace are
    recovered as their sample-weighted mean, and the error feedback keeps what the mean does not explain."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    env = dict(os.environ, REPO_ROOT=os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
               MADDR_FILE=str(tmp_path / "maddrs.json"), OUT_PREFIX=str(tmp_path / "out"), NCCL_NVLS_ENABLE="0")
    script = tmp_path / "powersgd_child.py"
    script.write_text(POWERSGD_CHILD)
    procs = [subprocess.Popen([sys.executable, str(script), str(r), str(world)], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outputs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outputs.append(out)
    assert all(p.returncode == 0 for p in procs), "\n".join(o[-2000:] for o in outputs)

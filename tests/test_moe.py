"""Mixture-of-experts on CPU: DHT declarations, beam search, remote calls, fault tolerance, checkpoints, training.

Modelled on the reference's tests/test_moe.py, test_dht_experts.py, test_expert_backend.py, test_custom_experts.py,
test_connection_handler.py and the MoE parts of test_training.py.
"""
import asyncio
import random
import time

import numpy as np
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from hivemind_b200.dht import DHT
from hivemind_b200.moe import (ModuleBackend, RemoteExpert, RemoteMixtureOfExperts, RemoteSwitchMixtureOfExperts,
                               Server, background_server, declare_experts, get_experts)
from hivemind_b200.moe.client.beam_search import MoEBeamSearcher
from hivemind_b200.moe.client.expert import DUMMY, create_remote_experts
from hivemind_b200.moe.client.moe import _RemoteCallMany
from hivemind_b200.moe.client.remote_expert_worker import RemoteExpertWorker
from hivemind_b200.moe.expert_uid import ExpertInfo, is_valid_prefix, is_valid_uid, split_uid
from hivemind_b200.moe.server.checkpoints import load_experts, store_experts
from hivemind_b200.moe.server.connection_handler import ConnectionHandler
from hivemind_b200.moe.server.layers import name_to_block
from hivemind_b200.moe.server.server import _generate_uids
from hivemind_b200.moe.server.task_pool import TaskPool
from hivemind_b200.p2p import PeerID
from hivemind_b200.proto import runtime_pb2
from hivemind_b200.compression import deserialize_torch_tensor, serialize_torch_tensor
from hivemind_b200.utils import BatchTensorDescriptor, MSGPackSerializer, get_dht_time


def _swarm(n):
    peers = [DHT(start=True)]
    maddrs = peers[0].get_visible_maddrs()
    peers += [DHT(initial_peers=maddrs, start=True) for _ in range(n - 1)]
    return peers


def test_uid_patterns():
    valid = ["expert.1", "expert.0", "expert.0.0.1", "expert.1337", "ffn.12.34.56.78.90", "transformer.3.2.1.0",
             "transformer_encoder.2", "transformer::encoder.2", "T®@nsf0rmE®🤗.321", "🤗.321", "0.1.2", "00.1.2"]
    for uid in valid:
        assert is_valid_uid(uid), uid
    for uid in ["", ".", "ffn.-1", "transformer.---", "a.b", "expert.1.", ".5", "ffn.01", "ffn", "expert.1..2",
                "ffn.1 2", "ffn.1.2.", "ffn.1..2"]:
        assert not is_valid_uid(uid), uid
    for prefix in ["expert.", "e.1.", "ffn.12.34.", "🤗."]:
        assert is_valid_prefix(prefix), prefix
    for prefix in ["", ".", "expert", "ffn.1", "ffn..", "ffn.-1.", ".1."]:
        assert not is_valid_prefix(prefix), prefix
    assert split_uid("ffn.3.7") == ("ffn.3.", 7) and split_uid("ffn.3.") == ("ffn.", 3)


def test_store_get_experts():
    peers = _swarm(6)
    try:
        first, other = peers[1], peers[4]
        uids = [f"my_expert.{i}" for i in range(30)]
        for start in range(0, len(uids), 10):
            assert all(declare_experts(first, uids[start:start + 10], get_dht_time() + 30).values())
        found = get_experts(other, random.sample(uids, 5) + ["foo", "bar"])
        assert all(isinstance(e, RemoteExpert) and e.peer_id == first.peer_id for e in found[:-2])
        assert found[-2] is None and found[-1] is None
        declare_experts(other, ["my_other_expert.1337"], get_dht_time() + 30)
        missing, present = get_experts(first, ["foobar", "my_other_expert.1337"])
        assert missing is None and present.peer_id == other.peer_id
        future = get_experts(first, ["my_expert.3"], return_future=True)
        assert future.result(10)[0].uid == "my_expert.3"
    finally:
        for peer in peers:
            peer.shutdown()


def test_beam_search_against_brute_force():
    peers = _swarm(5)
    grid = (8, 8, 8)
    try:
        rng = random.Random(0)
        experts = sorted({"expert." + ".".join(str(rng.randrange(d)) for d in grid) for _ in range(48)})
        for i in range(0, len(experts), 8):
            declare_experts(rng.choice(peers), experts[i:i + 8], get_dht_time() + 60)
        searcher = MoEBeamSearcher(peers[2], "expert.", grid, num_workers=4)
        for trial in range(3):
            scores = [np.random.RandomState(trial * 10 + d).randn(size).astype(np.float32) for d, size in enumerate(grid)]
            found = searcher.find_best_experts(scores, beam_size=48)
            total = {uid: sum(float(scores[d][int(c)]) for d, c in enumerate(uid.split(".")[1:])) for uid in experts}
            assert {e.uid for e in found} <= set(experts)
            found_scores = [total[e.uid] for e in found]
            assert found_scores == sorted(found_scores, reverse=True)
            # a beam as wide as the number of experts must return the best expert first
            assert found[0].uid == max(total, key=total.get)
        batch = [np.random.randn(5, size).astype(np.float32) for size in grid]
        rows = searcher.batch_find_best_experts(batch, beam_size=4)
        assert len(rows) == 5 and all(0 < len(row) <= 4 for row in rows)
        first = ".".join(experts[0].split(".")[:2]) + "."
        succ = searcher.get_active_successors([first, "expert.999."])
        assert succ["expert.999."] == {} and len(succ[first]) > 0
        beam = searcher.get_initial_beam([float(i) for i in range(8)], beam_size=3)
        assert len(beam) == 3 and beam[0][0] >= beam[1][0] >= beam[2][0]
    finally:
        for peer in peers:
            peer.shutdown()


def test_dht_single_node_and_flat_experts():
    dht = DHT(start=True)
    try:
        searcher = MoEBeamSearcher(dht, "expert.", grid_size=(10,))
        assert all(declare_experts(dht, ["expert.1", "expert.2", "expert.3"], get_dht_time() + 30).values())
        assert len(declare_experts(dht, ["ffn.1", "ffn.2"], get_dht_time() + 30)) == 4
        assert len(declare_experts(dht, ["e.1.2.3", "e.1.2.5", "e.2.0"], get_dht_time() + 30)) == 7
        for uid in ("ffn.1", "ffn.2", "e.1.2.3", "e.2.0"):
            assert get_experts(dht, [uid])[0].uid == uid
        successors = searcher.get_active_successors(["e.1.2.", "e.2.", "e.4.5."])
        assert set(successors["e.1.2."]) == {3, 5} and successors["e.4.5."] == {}
        assert successors["e.2."][0] == ExpertInfo("e.2.0", dht.peer_id)
        beam = searcher.get_initial_beam((3, 2, 1, 0, -1, -2, -3, -4, -5, -6), beam_size=3)
        assert len(beam) == 3 and all(prefix in ("expert.1.", "expert.2.", "expert.3.") for _, prefix, _ in beam)
        best = searcher.find_best_experts([(0.0, 3.0, 1.0, 2.0, 0, 0, 0, 0, 0, 0)], beam_size=2)
        assert [e.uid for e in best] == ["expert.1", "expert.3"]
    finally:
        dht.shutdown()


def test_negative_caching():
    peers = _swarm(4)
    try:
        writer, reader = peers[0], peers[-1]
        declare_experts(writer, ["ffn.1.2.3", "ffn.3.4.5"], get_dht_time() + 30)
        searcher = MoEBeamSearcher(reader, "ffn.", (10, 10, 10), negative_caching=True, cache_expiration=30)
        beam = searcher.get_initial_beam(scores=[0.1, 0.2, 0.3, 0.4, 0.5, 0, 0, 0, 0, 0], beam_size=3)
        assert {prefix for _, prefix, _ in beam} == {"ffn.1.", "ffn.3."}
        time.sleep(0.5)
        # the misses (ffn.4., ffn.2., ffn.0. ...) were written back as "nothing here" records
        seen = reader.get("ffn.4.", latest=True)
        assert seen is not None and isinstance(seen.value, dict) and seen.value[-1].value is None
    finally:
        for peer in peers:
            peer.shutdown()


def test_generate_uids():
    uids = _generate_uids(20, "ffn.[0:4].[10:20]")
    assert len(set(uids)) == 20 and all(is_valid_uid(u) and 10 <= int(u.split(".")[2]) < 20 for u in uids)
    assert _generate_uids(3, None) == ["expert.0", "expert.1", "expert.2"]
    with pytest.raises(ValueError):
        _generate_uids(1, "ffn.[0-4]")


def test_task_pool_batching():
    calls = []

    def double(x):
        calls.append(len(x))
        return (x * 2,)

    pool = TaskPool(double, max_batch_size=8, name="double", min_batch_size=4, timeout=0.2)
    futures = [pool.submit_task(torch.full((3, 2), float(i))) for i in range(3)]
    assert pool.priority < float("inf")  # 9 rows >= min_batch_size
    uid, batch = pool.load_batch_to_runtime()
    assert batch[0].shape == (6, 2)  # two whole tasks fit under max_batch_size, the third does not
    pool.send_outputs_from_runtime(uid, list(double(*batch)))
    assert torch.equal(futures[1].result(1)[0], torch.full((3, 2), 2.0)) and not futures[2].done()
    assert pool.priority == float("inf")  # 3 rows < min_batch_size and the timeout has not passed
    time.sleep(0.25)
    assert pool.priority < float("inf")
    oversized = pool.submit_task(torch.zeros(9, 2))
    with pytest.raises(ValueError):
        oversized.result(1)
    pool.shutdown()
    with pytest.raises(RuntimeError):
        futures[2].result(1)


def test_remote_module_call(hidden_dim=16):
    with background_server(num_experts=1, device="cpu", expert_cls="ffn", num_handlers=1, hidden_dim=hidden_dim,
                           optim_cls=None) as info:
        dht = DHT(initial_peers=info.addrs, start=True)
        try:
            real, fake = create_remote_experts(
                [ExpertInfo("expert.0", info.peer_id), ExpertInfo("oiasfjiasjf", info.peer_id)], dht)
            x = torch.randn(3, hidden_dim, requires_grad=True)
            out1, out2 = real(x), real(x)
            assert torch.allclose(out1, out2)
            (out1.pow(2).sum()).backward()
            assert x.grad is not None and x.grad.norm() > 0
            with pytest.raises(Exception):
                real(torch.randn(3, 11))  # wrong hidden size fails on the server, the error comes back
            with pytest.raises(Exception):
                fake(x)
        finally:
            dht.shutdown()


def test_call_many_fault_tolerance(hidden_dim=16):
    with background_server(num_experts=5, device="cpu", expert_cls="ffn", num_handlers=2, hidden_dim=hidden_dim,
                           optim_cls=None) as info:
        dht = DHT(initial_peers=info.addrs, start=True)
        try:
            x = torch.randn(4, hidden_dim, requires_grad=True)
            e0, e1, e2, e3, e4 = create_remote_experts([ExpertInfo(f"expert.{i}", info.peer_id) for i in range(5)], dht)
            e5 = RemoteExpert(ExpertInfo("thisshouldnotexist", info.peer_id), e0.p2p)
            chosen = [[e0, e1, e2], [e2, e4], [e1, e5, e3], []]
            mask, out = _RemoteCallMany.apply(DUMMY, chosen, 1, 1, None, 10.0, 10.0, False, True, e1.info, 1024, x)
            assert mask.shape == (4, 3) and out.shape == (4, 3, hidden_dim)
            assert np.array_equal(mask.numpy(), [[1, 1, 1], [1, 1, 0], [1, 0, 1], [0, 0, 0]])
            reference = torch.zeros_like(out)
            for i, row in enumerate(chosen):
                for j, expert in enumerate(row):
                    if mask[i, j]:
                        reference[i, j] = expert(x[i:i + 1])[0]
            assert torch.allclose(out, reference, atol=1e-5, rtol=0)
            probe = torch.randn_like(out)
            (out * probe).sum().backward()
            grad_many = x.grad.clone()
            x.grad = None
            (reference * probe).sum().backward()
            assert torch.allclose(grad_many, x.grad, atol=1e-5, rtol=0)
            # k_min larger than the number of live experts of sample 1 -> TimeoutError
            with pytest.raises(TimeoutError):
                _RemoteCallMany.apply(DUMMY, chosen[:3], 3, 1, None, 10.0, 10.0, False, True, e1.info, 1024, x[:3])
        finally:
            dht.shutdown()


def test_moe_layers_and_determinism(hidden_dim=16):
    uids = [f"ffn.{i}.{j}.{k}" for i in (0, 3) for j in (1, 2) for k in (0, 5)]
    with background_server(expert_uids=uids, device="cpu", expert_cls="ffn", num_handlers=2, hidden_dim=hidden_dim,
                           optim_cls=None) as info:
        dht = DHT(initial_peers=info.addrs, start=True)
        try:
            moe = RemoteMixtureOfExperts(in_features=hidden_dim, grid_size=(4, 4, 8), dht=dht, k_best=3, uid_prefix="ffn.")
            x = torch.randn(6, hidden_dim, requires_grad=True)
            out = moe(x)
            assert out.shape == (6, hidden_dim)
            out.pow(2).sum().backward()
            assert x.grad.norm() > 0 and moe.proj.weight.grad.norm() > 0
            out2 = moe(x)
            assert torch.allclose(out, out2, atol=1e-5)
            # 3-d inputs: the gate sees the mean over the middle dimension
            moe_info = moe.info
            assert moe_info["keyword_names"] == () or moe_info["keyword_names"] == []

            switch = RemoteSwitchMixtureOfExperts(in_features=hidden_dim, grid_size=(4, 4, 8), dht=dht,
                                                  uid_prefix="ffn.", jitter_eps=0, grid_dropout=1.0)
            y, balancing_loss = switch(x)
            assert y.shape == x.shape and balancing_loss.ndim == 0 and balancing_loss > 0
            (y.sum() + balancing_loss).backward()
            assert abs(float(switch.grid_utilization.sum()) - 3.0) < 1e-4
        finally:
            dht.shutdown()


def test_no_experts():
    dht = DHT(start=True)
    try:
        moe = RemoteSwitchMixtureOfExperts(in_features=8, grid_size=(4, 4), dht=dht, uid_prefix="expert.",
                                           forward_timeout=0.1, backward_timeout=0.1, allow_zero_outputs=True)
        with pytest.raises(RuntimeError):
            moe(torch.randn(3, 8))
    finally:
        dht.shutdown()


def test_compute_expert_scores():
    dht = DHT(start=True)
    try:
        moe = RemoteMixtureOfExperts(dht=dht, in_features=16, grid_size=(40,), k_best=4, k_min=1,
                                     timeout_after_k_min=1, uid_prefix="expert.")
        moe._expert_info = {}
        gx, gy = torch.randn(4, 5, requires_grad=True), torch.randn(4, 3, requires_grad=True)
        ii = [[4, 0, 2], [3, 1, 1, 1, 3], [0], [3, 2]]
        jj = [[2, 2, 1], [0, 1, 2, 0, 1], [0], [1, 2]]
        peer = PeerID(b"\x00" * 34)
        experts = [[RemoteExpert(ExpertInfo(f"expert.{i}.{j}", peer), None) for i, j in zip(ri, rj)]
                   for ri, rj in zip(ii, jj)]
        logits = moe.compute_expert_scores([gx, gy], experts)
        assert logits.shape == (4, 5)
        logits[logits.isfinite()].sum().backward()
        assert gx.grad.norm() > 0 and gy.grad.norm() > 0
        for b in range(4):
            for e in range(5):
                if e < len(ii[b]):
                    assert torch.allclose(logits[b, e], gx[b, ii[b][e]] + gy[b, jj[b][e]], atol=1e-6)
                else:
                    assert logits[b, e] == float("-inf")
    finally:
        dht.shutdown()


def test_client_anomaly_detection(hidden_dim=16):
    backends = {}
    for i in range(4):
        module = name_to_block["ffn"](hidden_dim)
        backends[f"expert.{i}"] = ModuleBackend(name=f"expert.{i}", module=module,
                                                optimizer=torch.optim.SGD(module.parameters(), lr=0.0),
                                                args_schema=(BatchTensorDescriptor(hidden_dim),),
                                                outputs_schema=BatchTensorDescriptor(hidden_dim), max_batch_size=16)
    with torch.no_grad():
        backends["expert.3"].module.ffn_bias.fill_(float("nan")) if hasattr(backends["expert.3"].module, "ffn_bias") \
            else next(backends["expert.3"].module.parameters()).fill_(float("nan"))
    dht = DHT(start=True)
    server = Server(dht, backends, num_connection_handlers=1, device="cpu", start=True)
    client = DHT(initial_peers=dht.get_visible_maddrs(), start=True)
    try:
        moe = RemoteMixtureOfExperts(in_features=hidden_dim, grid_size=(3,), dht=client, k_best=3, uid_prefix="expert.",
                                     detect_anomalies=True)
        x = torch.randn(2, hidden_dim)
        assert moe(x).isfinite().all()
        bad = x.clone()
        bad[0, 0] = float("inf")
        with pytest.raises(ValueError):
            moe(bad)
        moe_all = RemoteMixtureOfExperts(in_features=hidden_dim, grid_size=(4,), dht=client, k_best=4,
                                         uid_prefix="expert.", detect_anomalies=True)
        assert moe_all(x).isfinite().all()  # the NaN expert is masked out
        moe_blind = RemoteMixtureOfExperts(in_features=hidden_dim, grid_size=(4,), dht=client, k_best=4,
                                           uid_prefix="expert.", detect_anomalies=False)
        assert not moe_blind(x).isfinite().all()
    finally:
        client.shutdown()
        server.shutdown()


def test_connection_handler_rpcs(hidden_dim=16):
    module = name_to_block["ffn"](hidden_dim)
    backend = ModuleBackend(name="expert.0", module=module, args_schema=(BatchTensorDescriptor(hidden_dim),),
                            outputs_schema=BatchTensorDescriptor(hidden_dim), max_batch_size=4096,
                            optimizer=torch.optim.SGD(module.parameters(), lr=0.0))
    dht = DHT(start=True)
    server = Server(dht, {"expert.0": backend}, num_connection_handlers=1, device="cpu", start=True)
    client = DHT(initial_peers=dht.get_visible_maddrs(), start=True)
    try:
        async def _exercise():
            p2p = await client.replicate_p2p()
            stub = ConnectionHandler.get_stub(p2p, dht.peer_id)
            info = MSGPackSerializer.loads((await stub.rpc_info(runtime_pb2.ExpertUID(uid="expert.0"))).serialized_info)
            assert info["keyword_names"] in ((), []) and len(info["forward_schema"][0]) == 1
            x = torch.randn(5, hidden_dim)
            reply = await stub.rpc_forward(runtime_pb2.ExpertRequest(uid="expert.0", tensors=[serialize_torch_tensor(x)]))
            y = deserialize_torch_tensor(reply.tensors[0])
            assert torch.allclose(y, module(x), atol=1e-5)
            reply = await stub.rpc_backward(runtime_pb2.ExpertRequest(
                uid="expert.0", tensors=[serialize_torch_tensor(x), serialize_torch_tensor(torch.ones_like(y))]))
            grad = deserialize_torch_tensor(reply.tensors[0])
            xr = x.clone().requires_grad_(True)
            module(xr).sum().backward()
            assert torch.allclose(grad, xr.grad, atol=1e-5)
            with pytest.raises(Exception):
                await stub.rpc_forward(runtime_pb2.ExpertRequest(uid="expert.404", tensors=[serialize_torch_tensor(x)]))
        RemoteExpertWorker.run_coroutine(_exercise())
        # a large batch goes through the streamed RPCs (over the unary payload limit)
        expert = create_remote_experts([ExpertInfo("expert.0", dht.peer_id)], client)[0]
        wide = torch.randn(40000, hidden_dim)  # 2.5 MB > 2 MiB unary limit
        with pytest.raises(Exception):
            expert(wide)  # exceeds max_batch_size on the server: the error is propagated, not a hang
        backend.forward_pool.max_batch_size = backend.backward_pool.max_batch_size = 65536
        out = expert(wide)
        assert torch.allclose(out[:100], module(wide[:100]), atol=1e-5)
    finally:
        client.shutdown()
        server.shutdown()


def test_custom_and_multihead_experts(tmp_path, hidden_dim=16):
    source = tmp_path / "custom_networks.py"
    source.write_text('''
import torch
import torch.nn as nn
from hivemind_b200.moe import register_expert_class

@register_expert_class("perceptron", lambda batch, hid: torch.empty((batch, hid)))
class Perceptron(nn.Module):
    def __init__(self, hid):
        super().__init__()
        self.a, self.b = nn.Linear(hid, 2 * hid), nn.Linear(2 * hid, hid)
    def forward(self, x):
        return self.b(torch.relu(self.a(x)))

@register_expert_class("multihead", lambda batch, hid: (torch.empty((batch, hid)), torch.empty((batch, 2 * hid)),
                                                      torch.empty((batch, 3 * hid))))
class MultiHead(nn.Module):
    def __init__(self, hid):
        super().__init__()
        self.a, self.b, self.c = nn.Linear(hid, hid), nn.Linear(2 * hid, hid), nn.Linear(3 * hid, hid)
    def forward(self, x, y, z):
        return self.a(x) + self.b(y) + self.c(z)
''')
    for cls, make_inputs in (("perceptron", lambda: (torch.randn(3, hidden_dim),)),
                             ("multihead", lambda: (torch.randn(3, hidden_dim), torch.randn(3, 2 * hidden_dim),
                                                    torch.randn(3, 3 * hidden_dim)))):
        with background_server(expert_cls=cls, num_experts=2, device="cpu", hidden_dim=hidden_dim, num_handlers=1,
                               custom_module_path=str(source)) as info:
            dht = DHT(initial_peers=info.addrs, start=True)
            try:
                e0, e1 = create_remote_experts([ExpertInfo("expert.0", info.peer_id), ExpertInfo("expert.1", info.peer_id)], dht)
                inputs = [t.requires_grad_(True) for t in make_inputs()]
                out = e0(*inputs) + e1(*inputs)
                assert out.shape == (3, hidden_dim)
                out.sum().backward()
                assert all(t.grad is not None for t in inputs)
            finally:
                dht.shutdown()


def _example_backends(hidden_dim=16, n=3):
    backends = {}
    for i in range(n):
        module = nn.Linear(hidden_dim, hidden_dim)
        opt = torch.optim.Adam(module.parameters(), lr=0.1)
        sched = torch.optim.lr_scheduler.LambdaLR(opt, lambda step: max(0.0, 1.0 - step / 10))
        backends[f"expert.{i}"] = ModuleBackend(name=f"expert.{i}", module=module, optimizer=opt, scheduler=sched,
                                                args_schema=(BatchTensorDescriptor(hidden_dim),),
                                                outputs_schema=BatchTensorDescriptor(hidden_dim), max_batch_size=4)
    return backends


def test_checkpoints_update_count_and_schedule(tmp_path):
    backends = _example_backends()
    expert = backends["expert.0"]
    store_experts(backends, tmp_path)
    saved = expert.module.weight.detach().clone()
    with torch.no_grad():
        expert.module.weight.add_(1.0)
    time.sleep(0.01)
    store_experts(backends, tmp_path)
    assert len(list((tmp_path / "expert.0").glob("checkpoint_*.pt"))) == 3  # two stamps + checkpoint_last
    with torch.no_grad():
        expert.module.weight.zero_()
    load_experts(backends, tmp_path)
    assert torch.allclose(expert.module.weight, saved + 1.0)

    x = torch.randn(2, 16)
    for _ in range(3):
        expert.backward(x, torch.ones(2, 16))
    assert expert.update_count == 3 and expert.examples_processed == 6
    assert abs(expert.optimizer.param_groups[0]["lr"] - 0.1 * 0.7) < 1e-9
    store_experts(backends, tmp_path)
    expert.backward(x, torch.ones(2, 16))
    load_experts(backends, tmp_path)
    assert expert.scheduler.last_epoch == 3
    assert abs(expert.optimizer.param_groups[0]["lr"] - 0.1 * 0.7) < 1e-9


def test_server_checkpoint_restart(tmp_path, hidden_dim=16):
    with background_server(num_experts=2, expert_pattern="ckpt.[0:64]", device="cpu", hidden_dim=hidden_dim,
                           num_handlers=1, checkpoint_dir=tmp_path, update_period=0.5, optim_cls=None):
        time.sleep(0.1)
    saved = sorted(child.name for child in tmp_path.iterdir())
    assert len(saved) == 2
    with background_server(num_experts=2, expert_pattern="ckpt.[0:64]", device="cpu", hidden_dim=hidden_dim,
                           num_handlers=1, checkpoint_dir=tmp_path, optim_cls=None) as info:
        dht = DHT(initial_peers=info.addrs, start=True)
        try:
            assert all(e is not None for e in get_experts(dht, saved))  # restarted with the same uids
        finally:
            dht.shutdown()


def test_training_through_a_chain_of_remote_experts(max_steps=100, threshold=0.9):
    """Two remote experts stacked inside an ordinary ``nn.Sequential``: gradients cross two RPC hops and both experts
    learn on the server side (the case of hivemind tests/test_training.py::test_training)."""
    from sklearn.datasets import load_digits

    torch.manual_seed(0)
    digits = load_digits(n_class=2)
    features = torch.tensor(digits["data"], dtype=torch.float32)
    labels = torch.tensor(digits["target"])
    with background_server(expert_uids=["expert.0", "expert.1"], device="cpu", hidden_dim=64, num_handlers=1,
                           optim_cls=lambda p: torch.optim.SGD(p, lr=0.05)) as info:
        dht = DHT(initial_peers=info.addrs, start=True)
        try:
            first, second = get_experts(dht, ["expert.0", "expert.1"])
            model = nn.Sequential(second, nn.ReLU(), first, nn.Linear(64, 2))
            opt = torch.optim.SGD(model.parameters(), lr=0.05)
            accuracy = 0.0
            for step in range(max_steps):
                logits = model(features)
                loss = F.cross_entropy(logits, labels)
                opt.zero_grad()
                loss.backward()
                opt.step()
                accuracy = (logits.argmax(1) == labels).float().mean().item()
                if accuracy >= threshold:
                    break
            assert accuracy >= threshold, accuracy
        finally:
            dht.shutdown()


def test_moe_training(max_steps=100, threshold=0.9):
    from sklearn.datasets import load_digits

    torch.manual_seed(0)
    digits = load_digits(n_class=2)
    features = torch.tensor(digits["data"], dtype=torch.float32)
    labels = torch.tensor(digits["target"])
    uids = [f"expert.{i}" for i in range(2)]
    with background_server(expert_uids=uids, device="cpu", optim_cls=lambda p: torch.optim.SGD(p, lr=0.05),
                           hidden_dim=64, num_handlers=1) as info:
        dht = DHT(initial_peers=info.addrs, start=True)
        try:
            moe = RemoteMixtureOfExperts(in_features=64, grid_size=(2,), dht=dht, uid_prefix="expert.", k_best=2)
            head = nn.Linear(64, 2)
            opt = torch.optim.SGD(list(moe.parameters()) + list(head.parameters()), lr=0.05)
            accuracy = 0.0
            for step in range(max_steps):
                logits = head(moe(features))
                loss = F.cross_entropy(logits, labels)
                opt.zero_grad()
                loss.backward()
                opt.step()
                accuracy = (logits.argmax(1) == labels).float().mean().item()
                if accuracy >= threshold:
                    break
            assert accuracy >= threshold, accuracy
        finally:
            dht.shutdown()


def test_switch_training(max_steps=10, threshold=0.9, num_experts=5):
    from sklearn.datasets import load_digits

    torch.manual_seed(0)
    digits = load_digits(n_class=2)
    features = torch.tensor(digits["data"], dtype=torch.float32)
    labels = torch.tensor(digits["target"])
    uids = [f"expert.{i}" for i in range(num_experts)]
    with background_server(expert_uids=uids, device="cpu", optim_cls=lambda p: torch.optim.SGD(p, lr=0.05),
                           hidden_dim=64, num_handlers=1) as info:
        dht = DHT(initial_peers=info.addrs, start=True)
        try:
            moe = RemoteSwitchMixtureOfExperts(in_features=64, grid_size=(num_experts,), dht=dht,
                                               uid_prefix="expert.", k_best=1)
            head = nn.Linear(64, 2)
            opt = torch.optim.SGD(list(moe.parameters()) + list(head.parameters()), lr=0.05)
            accuracy = 0.0
            for step in range(max_steps):
                hidden, balancing_loss = moe(features)
                logits = head(hidden)
                loss = F.cross_entropy(logits, labels) + 0.01 * balancing_loss
                opt.zero_grad()
                loss.backward()
                opt.step()
                accuracy = (logits.argmax(1) == labels).float().mean().item()
                if accuracy >= threshold:
                    break
            assert accuracy >= threshold, accuracy
            assert int((moe.grid_utilization > 0).sum()) > num_experts // 2  # no collapse onto a single expert
        finally:
            dht.shutdown()


def test_remote_expert_worker_concurrency():
    async def nap(i):
        await asyncio.sleep(0.2)
        return i

    started = time.perf_counter()
    futures = [RemoteExpertWorker.run_coroutine(nap(i), return_future=True) for i in range(20)]
    assert [f.result(5) for f in futures] == list(range(20))
    assert time.perf_counter() - started < 1.5


def test_background_servers_share_or_differ_in_identity(tmp_path):
    """Servers started with the same identity file have one peer id, a server without it gets its own
    (the case of hivemind tests/test_start_server.py::test_background_server_identity_path)."""
    from functools import partial

    identity = str(tmp_path / "server.id")
    start = partial(background_server, num_experts=1, device="cpu", hidden_dim=4, num_handlers=1, expert_cls="nop")
    with start(identity_path=identity) as first, start(identity_path=identity) as second, start() as third:
        assert first.peer_id == second.peer_id != third.peer_id
        assert all(str(addr).endswith(info.peer_id.to_base58()) for info in (first, second, third) for addr in info.addrs)

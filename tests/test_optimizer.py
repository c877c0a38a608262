"""Optimizer stack on CPU: gradient averager weighting, state averager, progress tracker, full Optimizer runs.
Cases modelled on the reference's tests/test_optimizer.py."""
import threading
import time

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

import hivemind_b200 as hivemind
from hivemind_b200.optim import GradientAverager, Optimizer, ProgressTracker, TrainingStateAverager
from hivemind_b200.optim.state_averager import dump_optimizer_state, load_optimizer_state


def launch_dht_instances(n):
    first = hivemind.DHT(start=True)
    return [first] + [hivemind.DHT(initial_peers=first.get_visible_maddrs(), start=True) for _ in range(n - 1)]


def test_grad_averager_accumulation_and_weighting():
    dhts = launch_dht_instances(2)
    p1, p2 = nn.Parameter(torch.zeros(3)), nn.Parameter(torch.zeros(3))
    a1 = GradientAverager([p1], dht=dhts[0], prefix="grads", target_group_size=2, min_matchmaking_time=1.0,
                          request_timeout=0.5, reuse_grad_buffers=False, start=True)
    a2 = GradientAverager([p2], dht=dhts[1], prefix="grads", target_group_size=2, min_matchmaking_time=1.0,
                          request_timeout=0.5, reuse_grad_buffers=True, start=True)
    try:
        c1 = a1.schedule_step(timeout=30)
        c2 = a2.schedule_step(timeout=30)
        for _ in range(10):
            p1.grad = None
            F.mse_loss(p1, torch.ones(3)).backward()
            a1.accumulate_grads_(batch_size=2)  # 20 samples in total
            F.mse_loss(p2, -torch.ones(3)).backward()  # accumulates in param.grad
            a2.accumulate_grads_(batch_size=3)  # 30 samples
        g1 = -2 / 3 * torch.ones(3)  # d/dp mean((p-1)^2) at p=0
        g2 = 2 / 3 * torch.ones(3)
        assert a1.local_samples_accumulated == 20 and a1.local_times_accumulated == 10
        assert torch.allclose(next(a2._grad_accumulators()), g2 * 10)
        t1 = threading.Thread(target=lambda: a1.step(control=c1, wait=True, timeout=30))
        t1.start()
        a2.step(control=c2, wait=True, timeout=30)
        t1.join()
        expected = (g1 * 20 + g2 * 30) / 50
        for averager in (a1, a2):
            with averager.use_averaged_gradients() as grads:
                assert torch.allclose(grads[0], expected, atol=1e-6)
            assert averager.local_samples_accumulated == 0
        with a1.use_averaged_gradients():
            assert torch.allclose(p1.grad, expected, atol=1e-6)
        assert not torch.allclose(p1.grad, expected)  # original grad buffers are restored
    finally:
        for x in (a1, a2, *dhts):
            x.shutdown()


def test_optimizer_state_dump_roundtrip():
    model = nn.Linear(4, 3)
    opt = torch.optim.Adam(model.parameters(), lr=0.1)
    model(torch.randn(2, 4)).sum().backward()
    opt.step()
    meta, tensors = dump_optimizer_state(opt)
    assert all(m["type"] in ("tensor", "value") for m in meta) and len(tensors) >= 4
    other = torch.optim.Adam(nn.Linear(4, 3).parameters(), lr=0.5)
    for p in other.param_groups[0]["params"]:
        p.grad = torch.zeros_like(p)
    other.step()
    load_optimizer_state(other, meta, tensors)
    assert other.param_groups[0]["lr"] == 0.1
    for (k1, s1), (k2, s2) in zip(opt.state_dict()["state"].items(), other.state_dict()["state"].items()):
        assert torch.allclose(s1["exp_avg"], s2["exp_avg"])


@pytest.mark.parametrize("offload,reuse", [(False, False), (True, True), (True, False)])
def test_state_averager_step_and_averaging(offload, reuse):
    dhts = launch_dht_instances(2)
    torch.manual_seed(0)
    models = [nn.Linear(3, 2), nn.Linear(3, 2)]
    extras = [torch.full((2,), 1.0), torch.full((2,), 3.0)]
    avgs = [TrainingStateAverager(dht=dht, optimizer=lambda p: torch.optim.SGD(p, lr=0.1), params=list(m.parameters()),
                                  scheduler=lambda opt: torch.optim.lr_scheduler.LambdaLR(opt, lambda e: 1 / (1 + e)),
                                  offload_optimizer=offload, reuse_tensors=reuse, extra_tensors=[e],
                                  prefix="state", target_group_size=2, min_matchmaking_time=1.0, request_timeout=0.5,
                                  start=True)
            for dht, m, e in zip(dhts, models, extras)]
    try:
        before = [[p.detach().clone() for p in m.parameters()] for m in models]
        for m in models:
            m(torch.ones(1, 3)).sum().backward()
        threads = [threading.Thread(target=lambda a=a: a.step(increment_epoch=True, optimizer_step=True, zero_grad=True,
                                                              averaging_round=True, averaging_opts=dict(timeout=30)))
                   for a in avgs]
        [t.start() for t in threads]
        [t.join(60) for t in threads]
        assert all(a.local_epoch == 1 for a in avgs)
        # every peer made one SGD step, then parameters were averaged
        stepped = [[b - 0.1 * torch.ones_like(b) for b in bs] for bs in before]
        for k, (pa, pb) in enumerate(zip(models[0].parameters(), models[1].parameters())):
            expected = (stepped[0][k] + stepped[1][k]) / 2
            assert torch.allclose(pa, expected, atol=1e-6) and torch.allclose(pb, expected, atol=1e-6)
        assert all(torch.allclose(e, torch.full((2,), 2.0)) for e in extras)
        assert abs(avgs[0].optimizer.param_groups[0]["lr"] - 0.05) < 1e-9  # scheduler follows the epoch
        assert all(p.grad is None or float(p.grad.abs().sum()) == 0 for p in models[0].parameters())
    finally:
        for x in (*avgs, *dhts):
            x.shutdown()


def test_progress_tracker_counts_swarm_samples():
    dhts = launch_dht_instances(3)
    trackers = [ProgressTracker(dht, "run", target_batch_size=100, min_refresh_period=0.1, default_refresh_period=0.2,
                                max_refresh_period=0.5, start=True) for dht in dhts]
    try:
        for i, tracker in enumerate(trackers):
            tracker.report_local_progress(0, 10 * (i + 1))
        deadline = time.time() + 15
        while time.time() < deadline and not all(t.global_progress.samples_accumulated >= 60 and
                                                 t.global_progress.num_peers == 3 for t in trackers):
            time.sleep(0.1)
        assert all(t.global_progress.num_peers == 3 for t in trackers)
        assert all(t.global_progress.samples_accumulated == 60 for t in trackers)
        trackers[1].report_local_progress(0, 70)  # 10 + 70 + 30 >= 100
        deadline = time.time() + 15
        while time.time() < deadline and not all(t.ready_to_update_epoch for t in trackers):
            time.sleep(0.1)
        assert all(t.ready_to_update_epoch for t in trackers)
        with trackers[0].pause_updates():
            assert trackers[0].update_epoch() == 1
        deadline = time.time() + 15
        while time.time() < deadline and trackers[2].global_epoch != 1:
            time.sleep(0.1)
        assert trackers[2].global_epoch == 1 and trackers[2].ready_to_update_epoch
    finally:
        for x in (*trackers, *dhts):
            x.shutdown()


def _run_peer(dht, seed, results, epochs, **opt_kwargs):
    torch.manual_seed(seed)
    model = nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 4))
    opt = Optimizer(dht=dht, run_id="test_run", target_batch_size=64, batch_size_per_step=8,
                    params=model.parameters(), optimizer=lambda p: torch.optim.Adam(p, lr=3e-2),
                    matchmaking_time=1.0, averaging_timeout=15.0, verbose=False,
                    averager_opts=dict(request_timeout=0.5, target_group_size=2),
                    tracker_opts=dict(min_refresh_period=0.1, default_refresh_period=0.3, max_refresh_period=0.5),
                    **opt_kwargs)
    gen = torch.Generator().manual_seed(1234)
    w_true = torch.randn(16, 4, generator=gen)
    losses = []
    deadline = time.time() + 120
    while opt.local_epoch < epochs and time.time() < deadline:
        x = torch.randn(8, 16)
        y = (x @ w_true).argmax(-1)
        loss = F.cross_entropy(model(x), y)
        loss.backward()
        opt.step()
        if not (opt.use_gradient_averaging and opt.grad_averager.reuse_grad_buffers):
            opt.zero_grad()
        losses.append(loss.item())
        time.sleep(0.01)
    first_loss, last_loss = sum(losses[:8]) / 8, sum(losses[-8:]) / 8
    results[seed] = (opt.local_epoch, first_loss, last_loss, [p.detach().clone() for p in model.parameters()],
                     opt.state_dict()["state"].get("local_epoch"))
    opt.shutdown()


@pytest.mark.parametrize("mode", ["sync", "delayed", "local_updates"])
def test_optimizer_two_peers_converge_and_stay_in_sync(mode):
    kwargs = dict(sync=dict(), delayed=dict(delay_optimizer_step=True, delay_grad_averaging=True, offload_optimizer=True),
                  local_updates=dict(use_local_updates=True, delay_state_averaging=False))[mode]
    dhts = launch_dht_instances(2)
    results = {}
    try:
        threads = [threading.Thread(target=_run_peer, args=(dht, i, results, 8), kwargs=kwargs) for i, dht in enumerate(dhts)]
        [t.start() for t in threads]
        [t.join(180) for t in threads]
        assert set(results) == {0, 1}
        for epoch, first, last, params, saved_epoch in results.values():
            assert epoch >= 8 and saved_epoch == epoch
            assert last < first
        if mode == "sync" and results[0][0] == results[1][0]:
            # peers that stopped at the same epoch hold (nearly) the same parameters
            for pa, pb in zip(results[0][3], results[1][3]):
                assert torch.allclose(pa, pb, atol=5e-2)
    finally:
        for dht in dhts:
            dht.shutdown()


def test_single_peer_proceeds_with_local_gradients():
    dht = hivemind.DHT(start=True)
    results = {}
    try:
        _run_peer(dht, 0, results, 6)
        assert results[0][0] >= 6 and results[0][2] < results[0][1]
    finally:
        dht.shutdown()


def test_power_sgd_rank1_recovers_rank1_gradients():
    """With rank-1 gradients, rank-1 PowerSGD reproduces the sample-weighted mean (reference: tests/test_optimizer.py:28-87)."""
    from hivemind_b200.optim import PowerSGDGradientAverager

    dhts = launch_dht_instances(2)
    torch.manual_seed(0)
    u, v = torch.randn(12, 1), torch.randn(1, 9)
    params = [[nn.Parameter(torch.zeros(12, 9)), nn.Parameter(torch.zeros(7))] for _ in range(2)]
    avs = [PowerSGDGradientAverager(p, averager_rank=1, dht=dht, prefix="psgd", target_group_size=2,
                                    min_matchmaking_time=1.0, request_timeout=0.5, min_compression_ratio=0.0, start=True)
           for p, dht in zip(params, dhts)]
    try:
        scales, samples = [1.0, 3.0], [8, 18]
        for p, scale in zip(params, scales):
            p[0].grad = scale * (u @ v)
            p[1].grad = torch.full((7,), scale)
        controls = [a.schedule_step(timeout=30) for a in avs]
        for a, n in zip(avs, samples):
            a.accumulate_grads_(batch_size=n)
        threads = [threading.Thread(target=lambda a=a, c=c: a.step(control=c, wait=True, timeout=30)) for a, c in zip(avs, controls)]
        [t.start() for t in threads]
        [t.join(60) for t in threads]
        mean_scale = (scales[0] * samples[0] + scales[1] * samples[1]) / sum(samples)
        for a, scale in zip(avs, scales):
            # error feedback keeps what the average does not explain: local gradient minus averaged gradient
            assert torch.allclose(a._ms[0], (scale - mean_scale) * (u @ v), atol=1e-4)
            with a.use_averaged_gradients() as grads:
                assert torch.allclose(grads[0], mean_scale * (u @ v), atol=1e-4)
                assert torch.allclose(grads[1], torch.full((7,), mean_scale), atol=1e-5)
    finally:
        for x in (*avs, *dhts):
            x.shutdown()


def test_training_averager_averages_parameters_and_statistics():
    """Legacy TrainingAverager: two peers with different parameters / Adam statistics meet in the middle."""
    from hivemind_b200.optim import TrainingAverager

    dht_root = hivemind.DHT(start=True)
    peers, averagers, models = [dht_root, hivemind.DHT(initial_peers=dht_root.get_visible_maddrs(), start=True)], [], []
    try:
        for i, dht in enumerate(peers):
            torch.manual_seed(i)
            model = torch.nn.Linear(8, 4)
            opt = torch.optim.Adam(model.parameters(), lr=0.1)
            model(torch.randn(16, 8)).pow(2).sum().backward()
            opt.step()
            models.append(model)
            averagers.append(TrainingAverager(opt, average_parameters=True, average_gradients=True,
                                              average_opt_statistics=["exp_avg_sq"], dht=dht, prefix="legacy",
                                              target_group_size=2, min_matchmaking_time=1.0, request_timeout=1.0,
                                              start=True))
        expected_weight = (models[0].weight.detach() + models[1].weight.detach()) / 2
        expected_grad = (models[0].weight.grad + models[1].weight.grad) / 2
        results = [None, None]

        def run(i):
            results[i] = averagers[i].step(timeout=30)

        threads = [threading.Thread(target=run, args=(i,)) for i in range(2)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(60)
        assert all(r is not None for r in results)
        for model in models:
            assert torch.allclose(model.weight, expected_weight, atol=1e-5)
            assert torch.allclose(model.weight.grad, expected_grad, atol=1e-5)
        stats = [averagers[i].opt.state[models[i].weight]["exp_avg_sq"] for i in range(2)]
        assert torch.allclose(stats[0], stats[1], atol=1e-6)
    finally:
        for averager in averagers:
            averager.shutdown()
        for dht in reversed(peers):
            dht.shutdown()


def test_grad_scaler_defers_unscale_and_update_to_the_global_step():
    """With reuse_grad_buffers the scaler must not unscale or step between global steps, and must survive overflows."""
    dht = hivemind.DHT(start=True)
    try:
        model = torch.nn.Linear(4, 2)
        opt = hivemind.Optimizer(dht=dht, run_id="scaler", target_batch_size=8, batch_size_per_step=4,
                                 params=model.parameters(), optimizer=lambda p: torch.optim.SGD(p, lr=0.1),
                                 reuse_grad_buffers=True, matchmaking_time=0.5, averaging_timeout=5.0,
                                 tracker_opts=dict(min_refresh_period=0.05, default_refresh_period=0.05,
                                                   max_refresh_period=0.1), verbose=False)
        scaler = hivemind.GradScaler("cpu", init_scale=4.0, growth_interval=1)
        before = model.weight.detach().clone()
        for micro_step in range(2):
            loss = model(torch.ones(4, 4)).sum()
            scaler.scale(loss).backward()
            assert scaler.unscale_(opt) is False  # between global steps gradients stay scaled
            scaler.step(opt)
            scaler.update()
            time.sleep(0.3)
        deadline = time.time() + 20
        while opt.local_epoch < 1 and time.time() < deadline:
            loss = model(torch.ones(4, 4)).sum()
            scaler.scale(loss).backward()
            scaler.unscale_(opt)
            scaler.step(opt)
            scaler.update()
            time.sleep(0.2)
        assert opt.local_epoch >= 1 and not torch.allclose(model.weight, before)
        assert torch.isfinite(model.weight).all()
        # the applied update corresponds to unscaled gradients: |delta| = lr * |grad| = 0.1 * 4 per weight at most x small factor
        assert (model.weight.detach() - before).abs().max() < 2.0
        opt.shutdown()
    finally:
        dht.shutdown()


def test_fused_optimizers_track_parameters_that_join_or_skip_steps():
    """A parameter whose gradient is None in some steps keeps its own momentum buffer and step count, exactly like
    the PyTorch optimizers (which skip such parameters): nobody else's momentum is reset when it joins, and its bias
    correction uses its own number of steps."""
    from hivemind_b200.optim.fused import FusedAdam, FusedSGD

    torch.manual_seed(0)
    for make_ours, make_ref in (
            (lambda ps: FusedSGD(ps, lr=0.1, momentum=0.9), lambda ps: torch.optim.SGD(ps, lr=0.1, momentum=0.9)),
            (lambda ps: FusedAdam(ps, lr=0.05), lambda ps: torch.optim.Adam(ps, lr=0.05))):
        a, b = torch.randn(7, 3), torch.randn(5)
        ours = [a.clone().requires_grad_(), b.clone().requires_grad_()]
        ref = [a.clone().requires_grad_(), b.clone().requires_grad_()]
        opt_ours, opt_ref = make_ours(ours), make_ref(ref)
        for step in range(4):
            grads = [torch.randn_like(a), torch.randn_like(b)]
            for params in (ours, ref):
                params[0].grad = grads[0].clone()
                params[1].grad = grads[1].clone() if step in (1, 3) else None  # joins late, then skips a step
            opt_ours.step()
            opt_ref.step()
        for mine, theirs in zip(ours, ref):
            assert torch.allclose(mine, theirs, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("factory", ["plain", "powersgd"])
def test_grad_averager_refuses_buffers_of_the_wrong_shape(factory):
    """Pre-allocated ``averaged_grads`` have to match the parameters one by one
    (the case of hivemind tests/test_optimizer.py::test_grad_averager_wrong_shape)."""
    from functools import partial

    from hivemind_b200 import DHT
    from hivemind_b200.optim.grad_averager import GradientAverager
    from hivemind_b200.optim.power_sgd_averager import PowerSGDGradientAverager

    make = GradientAverager if factory == "plain" else partial(PowerSGDGradientAverager, averager_rank=1)
    model = torch.nn.ParameterDict({"w": torch.nn.Parameter(torch.zeros(5, 5))})
    dht = DHT(start=True)
    try:
        with pytest.raises(ValueError):
            make(model.parameters(), dht=dht, prefix="wrong_shape", target_group_size=2, reuse_grad_buffers=False,
                 start=True, averaged_grads=[torch.zeros(5, 5, 1)])
    finally:
        dht.shutdown()


def test_user_supplied_gradient_buffers_receive_the_average():
    """Buffers passed as ``averaged_grads`` are the averaged tensors themselves on the CPU path: after a round the
    caller finds the result in the objects it handed in (on CUDA the tensors move into a device arena and
    ``get_tensors()`` is the way to read them, which the averager says in its log)."""
    from hivemind_b200 import DHT

    first = DHT(start=True)
    second = DHT(initial_peers=first.get_visible_maddrs(), start=True)
    models = [torch.nn.Linear(3, 2) for _ in range(2)]
    buffers = [[torch.zeros_like(p) for p in model.parameters()] for model in models]
    averagers = [GradientAverager(model.parameters(), dht=dht, prefix="own_buffers", target_group_size=2,
                                  min_matchmaking_time=1.0, reuse_grad_buffers=False, start=True, averaged_grads=own)
                 for model, dht, own in zip(models, (first, second), buffers)]
    try:
        for index, (model, averager) in enumerate(zip(models, averagers)):
            model(torch.ones(4, 3) * (index + 1)).sum().backward()
            averager.accumulate_grads_(batch_size=4)
        expected = [(a.grad + b.grad) / 2 for a, b in zip(models[0].parameters(), models[1].parameters())]
        controls = [averager.step(wait=False, timeout=30) for averager in averagers]
        for control in controls:
            control.result(60)
        for own in buffers:
            for buffer, reference in zip(own, expected):
                assert torch.allclose(buffer, reference, atol=1e-6), "the caller's own buffer holds the average"
        with averagers[0].use_averaged_gradients():
            for p, reference in zip(models[0].parameters(), expected):
                assert torch.allclose(p.grad, reference, atol=1e-6)
    finally:
        for item in (*averagers, second, first):
            item.shutdown()

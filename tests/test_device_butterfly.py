"""Device butterfly against a CPU oracle built from the reference math: several ranks emulated on one GPU."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from hivemind_b200.averaging.allreduce import AveragingMode
from hivemind_b200.compression import (BlockwiseQuantization, CompressionInfo, Float16Compression, NoCompression,
                                       Quantile8BitQuantization, ScaledFloat16Compression, Uniform8BitQuantization,
                                       deserialize_torch_tensor)

CODECS = [NoCompression(), Float16Compression(), ScaledFloat16Compression(), Uniform8BitQuantization(),
          Quantile8BitQuantization(), BlockwiseQuantization()]
TOL = {"NoCompression": 1e-6, "Float16Compression": 2e-3, "ScaledFloat16Compression": 2e-3,
       "Uniform8BitQuantization": 0.08, "Quantile8BitQuantization": 0.08, "BlockwiseQuantization": 0.08}


def _make_endpoints(n, shapes, codec, part_size_bytes, seed=0):
    from hivemind_b200.parallel.device_butterfly import DeviceEndpoint

    torch.manual_seed(seed)
    dev = torch.device("cuda", 0)
    originals = [[torch.randn(s) * (1 + i) + 0.1 * r for i, s in enumerate(shapes)] for r in range(n)]
    endpoints = []
    for r in range(n):
        tensors = [t.to(dev) for t in originals[r]]
        infos = [CompressionInfo.from_tensor(t, key=i) for i, t in enumerate(tensors)]
        endpoints.append(DeviceEndpoint(tensors, codec, infos, part_size_bytes))
    return endpoints, originals


@pytest.mark.parametrize("codec", CODECS, ids=lambda c: type(c).__name__)
@pytest.mark.parametrize("n", [2, 3, 4])
def test_weighted_average_all_codecs(codec, n):
    from hivemind_b200.parallel.device_butterfly import run_group_emulated

    shapes = [(1000, 37), (5,), (70000,), (123, 4)]
    endpoints, originals = _make_endpoints(n, shapes, codec, part_size_bytes=2 ** 15)
    weights = [0.5 + 0.5 * r for r in range(n)]
    fractions = [1.0 / n] * n
    statuses = run_group_emulated(endpoints, weights=weights, peer_fractions=fractions)
    torch.cuda.synchronize()
    assert all(s.failed_elements == 0 and not s.banned_senders for s in statuses)
    for endpoint in endpoints:
        endpoint.check_canaries()  # no kernel wrote past the end of a region of any arena
    tol = TOL[type(codec).__name__]
    lossy8 = type(codec).__name__ in ("Uniform8BitQuantization", "Quantile8BitQuantization", "BlockwiseQuantization")
    for k in range(len(shapes)):
        ref = sum(w * originals[r][k] for r, w in enumerate(weights)) / sum(weights)
        spread = max(originals[0][k].std().item() if originals[0][k].numel() > 1 else 1.0, 1e-3)
        for r in range(n):
            got = endpoints[r].tensor_views[k].cpu()
            if lossy8:
                # 8-bit codebooks represent outliers by their bin mean, so judge by RMS error, like the
                # reference's MSE thresholds (tests/test_compression.py:33-46), not by the worst element
                rms = (got - ref).pow(2).mean().sqrt().item()
                assert rms <= 0.05 * spread, (type(codec).__name__, k, r, rms, spread)
            else:
                err = (got - ref).abs().max().item()
                assert err <= tol * max(ref.abs().max().item(), spread, 1.0), (type(codec).__name__, k, r, err)
    if isinstance(codec, NoCompression):
        for k in range(len(shapes)):
            assert torch.allclose(endpoints[0].tensor_views[k], endpoints[n - 1].tensor_views[k], atol=1e-5)


def test_modes_fractions_and_alpha():
    from hivemind_b200.parallel.device_butterfly import run_group_emulated

    shapes = [(50000,), (333,)]
    endpoints, originals = _make_endpoints(4, shapes, NoCompression(), part_size_bytes=2 ** 14)
    modes = [AveragingMode.NODE, AveragingMode.AUX, AveragingMode.NODE, AveragingMode.NODE]
    weights = [1.0, 0.0, 2.0, 3.0]
    fractions = [0.5, 0.25, 0.25, 0.0]  # the last peer reduces nothing, the auxiliary one only reduces
    run_group_emulated(endpoints, weights=weights, peer_fractions=fractions, modes=modes, alpha=0.5)
    torch.cuda.synchronize()
    for k in range(len(shapes)):
        ref = (originals[0][k] * 1 + originals[2][k] * 2 + originals[3][k] * 3) / 6
        for r in (0, 2, 3):
            expected = originals[r][k] + 0.5 * (ref - originals[r][k])
            assert torch.allclose(endpoints[r].tensor_views[k].cpu(), expected, atol=1e-5)
        assert torch.allclose(endpoints[1].tensor_views[k].cpu(), originals[1][k])  # auxiliaries keep their data


def test_missing_and_stalled_senders_are_excluded_without_hanging():
    """Host-side fault injection: one rank never publishes, another publishes only half of its parts.
    The waits run out after ``sender_timeout`` and the survivors average among themselves."""
    from hivemind_b200.parallel.device_butterfly import run_group_emulated

    shapes = [(200000,)]
    endpoints, originals = _make_endpoints(4, shapes, Float16Compression(), part_size_bytes=2 ** 14)
    statuses = run_group_emulated(endpoints, weights=[1.0] * 4, peer_fractions=[0.25] * 4, sender_timeout=0.5,
                                  reducer_timeout=1.0, skip_send_of=[3])
    torch.cuda.synchronize()
    ref = (originals[0][0] + originals[1][0] + originals[2][0]) / 3
    for r in range(3):
        assert 3 in statuses[r].banned_senders
        got = endpoints[r].tensor_views[0].cpu()
        # everything except the span reduced by the absent peer is the survivors' average
        assert torch.allclose(got[:150000], ref[:150000], atol=5e-3)
    # the absent peer still reduced its own span with what the others sent, so nobody loses that span either
    assert torch.allclose(endpoints[0].tensor_views[0].cpu()[150000:], ((originals[0][0] + originals[1][0] +
                          originals[2][0] + originals[3][0]) / 4)[150000:], atol=5e-3)


def test_sender_that_stalls_after_half_of_its_parts_is_left_out_of_the_rest():
    """Host-side fault injection: rank 2 publishes only the first half of the parts it sends, then nothing. The
    reducers of its later parts wait ``sender_timeout`` once, ban it, and average the survivors; the parts it did
    publish are averaged over everybody (hivemind/averaging/allreduce.py:317-321 bans a late sender the same way)."""
    from hivemind_b200.parallel.device_butterfly import run_group_emulated

    n, numel = 3, 6 * 16384
    endpoints, originals = _make_endpoints(n, [(numel,)], NoCompression(), part_size_bytes=2 ** 16)
    statuses = run_group_emulated(endpoints, weights=[1.0] * n, peer_fractions=[1.0 / n] * n, sender_timeout=0.5,
                                  reducer_timeout=1.0, publish_only_first_half_of=[2])
    torch.cuda.synchronize()
    everybody = sum(o[0] for o in originals) / n
    survivors = (originals[0][0] + originals[1][0]) / 2
    span = numel // n
    got0 = endpoints[0].tensor_views[0].cpu()
    # rank 2 sends its parts of rank 0's span first (published) and of rank 1's span last (never published)
    assert torch.allclose(got0[:span], everybody[:span], atol=1e-5)
    assert torch.allclose(got0[span:2 * span], survivors[span:2 * span], atol=1e-5)
    assert 2 in statuses[1].banned_senders and 2 not in statuses[0].banned_senders
    # rank 2's own span was reduced by rank 2 itself with what the others sent
    assert torch.allclose(got0[2 * span:], everybody[2 * span:], atol=1e-5)


def test_results_of_a_round_stay_readable_while_their_owner_runs_the_next_round_with_others():
    """Rank 1 is slow: it has not applied the results of round A yet when ranks 0 and 2 run a whole round B with each
    other. Round B writes the other copy of the staging buffers, so rank 1 still finds round A's averages."""
    from hivemind_b200.parallel.device_butterfly import finish_group_emulated, run_group_emulated

    numel = 4 * 16384
    for codec in (NoCompression(), Float16Compression()):
        endpoints, originals = _make_endpoints(3, [(numel,)], codec, part_size_bytes=2 ** 16, seed=7)
        prepared = run_group_emulated(endpoints, weights=[1.0] * 3, peer_fractions=[1 / 3] * 3, group_id=b"round-A",
                                      stop_after_stage=2)
        finish_group_emulated(endpoints, prepared, only=[0, 2])
        torch.cuda.synchronize()
        average_a = sum(o[0] for o in originals) / 3
        tol = 1e-5 if isinstance(codec, NoCompression) else 5e-3
        assert torch.allclose(endpoints[0].tensor_views[0].cpu(), average_a, atol=tol)
        # round B between ranks 0 and 2 with new values; rank 1 is still behind
        for r in (0, 2):
            endpoints[r].tensor_views[0].normal_()
        run_group_emulated([endpoints[0], endpoints[2]], weights=[1.0, 1.0], peer_fractions=[0.5, 0.5], group_id=b"round-B")
        torch.cuda.synchronize()
        statuses = finish_group_emulated(endpoints, prepared, only=[1])
        torch.cuda.synchronize()
        assert statuses[0].failed_elements == 0
        assert torch.allclose(endpoints[1].tensor_views[0].cpu(), average_a, atol=tol)


def test_zero_total_weight_leaves_values_unchanged():
    from hivemind_b200.parallel.device_butterfly import run_group_emulated

    endpoints, originals = _make_endpoints(2, [(40000,)], Float16Compression(), part_size_bytes=2 ** 15)
    run_group_emulated(endpoints, weights=[0.0, 0.0], peer_fractions=[0.5, 0.5], reducer_timeout=1.0)
    torch.cuda.synchronize()
    for r in range(2):
        assert torch.equal(endpoints[r].tensor_views[0].cpu(), originals[r][0])


def test_client_mode_peer_takes_part_with_an_empty_span():
    from hivemind_b200.parallel.device_butterfly import run_group_emulated

    endpoints, originals = _make_endpoints(3, [(50000,)], NoCompression(), part_size_bytes=2 ** 15)
    modes = [AveragingMode.NODE, AveragingMode.CLIENT, AveragingMode.NODE]
    infos = [e.describe() for e in endpoints]
    assert endpoints[1].can_run_with(infos, modes) and endpoints[0].can_run_with(infos, modes)
    run_group_emulated(endpoints, weights=[1.0, 1.0, 2.0], peer_fractions=[0.5, 0.0, 0.5], modes=modes)
    torch.cuda.synchronize()
    ref = (originals[0][0] + originals[1][0] + 2 * originals[2][0]) / 4
    for r in range(3):
        assert torch.allclose(endpoints[r].tensor_views[0].cpu(), ref, atol=1e-5)


def test_canaries_report_a_write_past_a_region():
    """The guard zones after each arena region: intact after a round, reported once something overwrites one
    (here the host does the overwriting with an ordinary fill of a slice that it owns)."""
    from hivemind_b200.parallel.device_butterfly import GUARD_BYTES, run_group_emulated

    endpoints, _ = _make_endpoints(2, [(4096,)], NoCompression(), part_size_bytes=2 ** 14)
    run_group_emulated(endpoints, weights=[1.0, 1.0], peer_fractions=[0.5, 0.5])
    for endpoint in endpoints:
        endpoint.check_canaries()
    guard = endpoints[0]._guards["outbox0"]
    endpoints[0]._bytes[guard:guard + 8].zero_()
    with pytest.raises(RuntimeError, match="outbox0"):
        endpoints[0].check_canaries()
    endpoints[1].check_canaries()
    assert GUARD_BYTES >= 256


def test_stage_timers_record_device_time():
    from hivemind_b200.utils import profiling

    profiling.enable(nvtx=True, timing=True)
    try:
        profiling.timing_summary(reset=True)
        x = torch.randn(1 << 20, device="cuda")
        for _ in range(3):
            with profiling.device_range("test.stage"):
                x = x * 1.0001
        summary = profiling.timing_summary()
        assert summary["test.stage"]["count"] == 3 and summary["test.stage"]["total_ms"] > 0
    finally:
        profiling.enable(nvtx=False, timing=False)


def test_device_codecs_match_cpu_codecs():
    torch.manual_seed(3)
    x = torch.randn(128, 128, 64)
    xc = x.cuda()
    for codec, bound in [(Float16Compression(), 5e-8), (ScaledFloat16Compression(), 5e-8),
                         (Uniform8BitQuantization(), 8e-4), (Quantile8BitQuantization(), 8e-4),
                         (BlockwiseQuantization(), 8e-4)]:
        msg = codec.compress(xc, CompressionInfo.from_tensor(xc))
        restored = deserialize_torch_tensor(msg)
        assert restored.shape == x.shape
        assert (restored - x).pow(2).mean().item() < bound, type(codec).__name__
        cpu_msg = codec.compress(x, CompressionInfo.from_tensor(x))
        assert len(cpu_msg.buffer) == len(msg.buffer)
    # the quantile codec estimates its borders from a sample on the device and from quantiles of chunk quantiles on
    # the CPU (hivemind/compression/quantization.py:105-122); both must fill the 256 bins about equally and
    # reconstruct about equally well
    q = Quantile8BitQuantization()
    idx_gpu, book_gpu = q.quantize(xc)
    idx_cpu, book_cpu = q.quantize(x)
    for idx in (idx_gpu.cpu(), idx_cpu):
        counts = torch.bincount(idx.flatten().long(), minlength=256).float()
        assert counts.min() > 0.3 * counts.mean() and counts.max() < 2.5 * counts.mean()
    mse_gpu = (book_gpu.cpu()[idx_gpu.cpu().long()] - x).pow(2).mean().item()
    mse_cpu = (book_cpu[idx_cpu.long()] - x).pow(2).mean().item()
    assert mse_gpu < 1.5 * mse_cpu, (mse_gpu, mse_cpu)
    borders_gpu = torch.stack([x[idx_gpu.cpu() == b].max() for b in range(255)])
    exact = torch.quantile(x.flatten()[:: 4].double(), torch.arange(1, 256, dtype=torch.float64) / 256).float()
    assert (borders_gpu - exact).abs().max().item() < 0.25  # tails of N(0, 1) are sparse; the body is far tighter
    assert (borders_gpu[32:224] - exact[32:224]).abs().max().item() < 0.03
    u_gpu = deserialize_torch_tensor(Uniform8BitQuantization().compress(xc, CompressionInfo.from_tensor(xc)))
    u_cpu = deserialize_torch_tensor(Uniform8BitQuantization().compress(x, CompressionInfo.from_tensor(x)))
    assert (u_gpu - u_cpu).abs().max().item() < 0.05  # same bins up to rounding at bin edges

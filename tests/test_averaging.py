"""DecentralizedAverager over the RPC path on CPU: weighted averages, modes, codecs, state download, triggers.
Cases modelled on the reference's tests/test_averaging.py and tests/test_allreduce.py."""
import random
import time

import pytest
import torch

from hivemind_b200.averaging import AveragingStage, DecentralizedAverager
from hivemind_b200.averaging.load_balancing import load_balance_peers
from hivemind_b200.averaging.partition import compute_part_layout
from hivemind_b200.compression import Float16Compression, Uniform8BitQuantization
from hivemind_b200.dht import DHT


def launch_dht_instances(n, **kwargs):
    first = DHT(start=True, **kwargs)
    maddrs = first.get_visible_maddrs()
    return [first] + [DHT(initial_peers=maddrs, start=True, **kwargs) for _ in range(n - 1)]


def _shutdown(*items):
    for item in items:
        item.shutdown()


def test_load_balancing_properties():
    assert load_balance_peers(100, (None, None)) == (50, 50)
    assert load_balance_peers(100, (None, None, None, None, None)) == (20, 20, 20, 20, 20)
    assert load_balance_peers(100, (0, 0, 0, None, None)) == (0, 0, 0, 50, 50)
    shares = load_balance_peers(1000, (100, 100, 1, 1))
    assert sum(shares) == 1000 and shares[2] + shares[3] < shares[0] + shares[1]
    assert load_balance_peers(100, (1e3, 1.0), min_size=10)[1] == 0
    for _ in range(20):
        n = random.randint(2, 10)
        bw = [random.choice([None, 0.0, random.random() * 100 + 1]) for _ in range(n)]
        if all(b == 0.0 for b in bw):
            bw[0] = 1.0
        vec = random.randint(1, 10 ** 6)
        shares = load_balance_peers(vec, bw)
        assert sum(shares) == vec and all(s >= 0 for s in shares)
        assert all(s == 0 for s, b in zip(shares, bw) if b == 0.0)


def test_part_layout_respects_fractions_and_tensor_boundaries():
    numels = [1000, 0, 37, 5000]
    specs = compute_part_layout(numels, [4] * 4, [1.0] * 4, [0.25, 0.0, 0.75], part_size_bytes=1024)
    assert sum(s.length for s in specs) == sum(numels)
    per_peer = [sum(s.length for s in specs if s.owner == p) for p in range(3)]
    assert per_peer[1] == 0 and abs(per_peer[0] - 0.25 * sum(numels)) <= 1
    for s in specs:
        assert 0 < s.length <= 256 and s.start + s.length <= numels[s.tensor_index]
    owners = [s.owner for s in specs]
    assert owners == sorted(owners)


@pytest.mark.parametrize("n_clients,n_aux", [(0, 0), (1, 0), (1, 1)])
def test_weighted_allreduce_with_modes(n_clients, n_aux):
    n_peers = 4
    dhts = launch_dht_instances(n_peers)
    modes = ["client"] * n_clients + ["aux"] * n_aux + ["node"] * (n_peers - n_clients - n_aux)
    random.shuffle(modes)
    torch.manual_seed(0)
    tensors = [[torch.randn(123), torch.randn(3, 50), torch.zeros(0)] for _ in range(n_peers)]
    weights = [random.uniform(0.5, 2.0) for _ in range(n_peers)]
    averagers = [DecentralizedAverager([t.clone() for t in tensors[i]], dhts[i], start=True, prefix="mygroup",
                                       target_group_size=n_peers, min_matchmaking_time=4.0, request_timeout=1.0,
                                       client_mode=modes[i] == "client", auxiliary=modes[i] == "aux",
                                       part_size_bytes=256)
                 for i in range(n_peers)]
    try:
        futures = [a.step(wait=False, weight=w, gather=dict(idx=i), timeout=30)
                   for i, (a, w) in enumerate(zip(averagers, weights))]
        gathered = [f.result(60) for f in futures]
        senders = [i for i in range(n_peers) if modes[i] != "aux"]
        total_w = sum(weights[i] for i in senders)
        for k in range(3):
            ref = sum(tensors[i][k] * weights[i] for i in senders) / total_w
            for i in senders:
                with averagers[i].get_tensors() as ts:
                    assert torch.allclose(ts[k], ref, atol=1e-5), (i, k)
        for i in range(n_peers):
            assert len(gathered[i]) == n_peers
            assert gathered[i][averagers[i].peer_id] == dict(idx=i)
    finally:
        _shutdown(*averagers, *dhts)


def test_codec_error_bounds_between_two_peers():
    dhts = launch_dht_instances(2)
    torch.manual_seed(1)
    x0, x1 = torch.randn(4096), torch.randn(4096)
    results = {}
    try:
        for name, codec in (("fp16", Float16Compression()), ("uniform8", Uniform8BitQuantization())):
            avs = [DecentralizedAverager([x.clone()], dht, start=True, prefix=f"codec{name}", target_group_size=2,
                                         min_matchmaking_time=2.0, request_timeout=1.0, compression=codec)
                   for x, dht in ((x0, dhts[0]), (x1, dhts[1]))]
            futures = [a.step(wait=False, timeout=30) for a in avs]
            [f.result(60) for f in futures]
            with avs[0].get_tensors() as ts:
                results[name] = (ts[0] - (x0 + x1) / 2).pow(2).mean().item()
            _shutdown(*avs)
        assert 0 < results["fp16"] <= 1e-5
        assert 1e-5 < results["uniform8"] <= 1e-2
    finally:
        _shutdown(*dhts)


def test_too_few_peers_fails_and_trigger_stages():
    dhts = launch_dht_instances(2)
    avs = [DecentralizedAverager([torch.ones(8) * i], dhts[i], start=True, prefix="trig", target_group_size=2,
                                 min_matchmaking_time=1.0, request_timeout=0.5) for i in range(2)]
    try:
        with pytest.raises(Exception):
            avs[0].step(timeout=2.0, allow_retries=False)  # nobody else is looking
        controls = [a.step(wait=False, require_trigger=True, timeout=30) for a in avs]
        deadline = time.time() + 20
        while time.time() < deadline and not all(c.stage == AveragingStage.AWAITING_TRIGGER for c in controls):
            time.sleep(0.05)
        assert all(c.stage == AveragingStage.AWAITING_TRIGGER for c in controls)
        controls[0].weight = 3.0  # weights stay mutable until all-reduce begins
        for c in controls:
            c.allow_allreduce()
        [c.result(30) for c in controls]
        with avs[1].get_tensors() as ts:
            assert torch.allclose(ts[0], torch.full((8,), 0.25))  # (0*3 + 1*1) / 4
        assert all(c.stage == AveragingStage.FINISHED for c in controls)
        cancelled = avs[0].step(wait=False, timeout=30)
        time.sleep(0.2)
        cancelled.cancel()
        assert cancelled.cancelled()
    finally:
        _shutdown(*avs, *dhts)


def test_state_download_prefers_higher_priority():
    dhts = launch_dht_instances(3)
    avs = [DecentralizedAverager([torch.full((5,), float(i))], dhts[i], start=True, prefix="state", target_group_size=2,
                                 declare_state_period=1.0) for i in range(3)]
    try:
        avs[0].state_sharing_priority, avs[1].state_sharing_priority = 5, 10
        avs[2].allow_state_sharing = False
        time.sleep(1.0)
        metadata, tensors = avs[2].load_state_from_peers(timeout=10)
        assert "group_key" in metadata and torch.allclose(tensors[0], torch.full((5,), 1.0))
        avs[0].state_sharing_priority = 20
        time.sleep(1.0)
        _, tensors = avs[2].load_state_from_peers(timeout=10)
        assert torch.allclose(tensors[0], torch.full((5,), 0.0))
        avs[0].allow_state_sharing = avs[1].allow_state_sharing = False
        time.sleep(1.5)
        assert avs[2].load_state_from_peers(timeout=5) is None
    finally:
        _shutdown(*avs, *dhts)


def test_remote_work_items_are_interleaved_over_owners():
    """Work lists of the device butterfly: same items, but consecutive items read from different GPUs and every GPU
    starts its walk at the peer after itself."""
    from hivemind_b200.parallel.device_butterfly import _interleave_by_owner

    n_peers, me = 4, 1
    owners_of_parts = [0, 0, 0, 2, 2, 3, 3, 3, 3]  # parts of the other three peers (peer 1 owns none of these)
    items = [(part, chunk, 0, 0) for part in range(len(owners_of_parts)) for chunk in range(2)]
    owners = [owners_of_parts[part] for part, _, _, _ in items]
    merged = _interleave_by_owner(items, owners, first_owner=(me + 1) % n_peers, n_peers=n_peers)
    assert sorted(merged) == sorted(items)
    walk = [owners_of_parts[part] for part, _, _, _ in merged]
    assert walk[:6] == [2, 3, 0, 2, 3, 0]  # round-robin starting at peer 2
    assert walk[-2:] == [3, 3]  # the longest queue drains last
    for owner in set(owners_of_parts):  # order inside one owner's queue is kept
        assert [item for item in merged if owners_of_parts[item[0]] == owner] == \
               [item for item in items if owners_of_parts[item[0]] == owner]
    assert _interleave_by_owner([], [], first_owner=0, n_peers=4) == []


def test_device_path_decision_on_described_arenas():
    """The rule that decides between the device path and the RPC butterfly, on hand-made ``describe()`` blobs."""
    from hivemind_b200.parallel.device_butterfly import peers_can_share_memory

    layout = {"data": 0, "avg0": 1024}
    a = dict(machine="m1", proc=b"A" * 16, dev=0, ptr=1, handle=b"h" * 64, layout=layout, total=100, supported=True)
    b = dict(a, proc=b"B" * 16, dev=1)
    assert peers_can_share_memory(a, [a, b]) and peers_can_share_memory(b, [a, b])
    assert not peers_can_share_memory(a, [a])  # a group of one
    assert not peers_can_share_memory(a, [a, None])  # a member without a device arena
    assert not peers_can_share_memory(a, [a, dict(b, machine="m2")])
    assert not peers_can_share_memory(a, [a, dict(b, total=101)])
    assert not peers_can_share_memory(a, [a, dict(b, layout={"data": 0, "avg0": 2048})])
    # two processes need handles on BOTH sides, whichever member asks (equal pids or device indices prove nothing)
    no_handle = dict(b, handle=None)
    assert not peers_can_share_memory(a, [a, no_handle]) and not peers_can_share_memory(no_handle, [a, no_handle])
    # inside one process raw pointers are enough
    same_proc = dict(a, dev=1, handle=None)
    assert peers_can_share_memory(dict(a, handle=None), [dict(a, handle=None), same_proc])
    assert not peers_can_share_memory(a, [a, dict(b, supported=False)])


def test_device_parts_come_in_whole_waves_of_the_grid():
    """Part sizing of the device butterfly: a reducer's span is cut into at most GRID_CTAS x waves parts of at most
    MAX_PART_CHUNKS chunks, every member derives the same size from (total elements, group size) alone, and small
    tensors fall apart into single chunks (maximum parallelism)."""
    from hivemind_b200.parallel.device_butterfly import CHUNK, GRID_CTAS, MAX_PART_CHUNKS, device_part_chunks

    for total in (1, 255, CHUNK, 3 * CHUNK + 5, 2 ** 20, 2 ** 26, 2 ** 28 + 12345, 2 ** 30):
        for peers in (1, 2, 3, 4, 8, 16):
            chunks = device_part_chunks(total, peers)
            span = -(-(-(-total // CHUNK)) // peers)
            assert 1 <= chunks <= MAX_PART_CHUNKS
            parts = -(-span // chunks)
            waves = -(-parts // GRID_CTAS)
            assert parts <= GRID_CTAS * waves
            if span <= GRID_CTAS:
                assert chunks == 1
            else:  # the last wave is at least two thirds full: no CTA idles for most of a stage
                assert parts > GRID_CTAS * (waves - 1) + GRID_CTAS * 2 // 3 or chunks == MAX_PART_CHUNKS


def test_a_client_that_starts_searching_first_still_joins_the_group():
    """A client-mode peer cannot lead, so it has to be able to join peers that declared themselves AFTER its own
    search began (their turn to lead comes later than the moment the client first promised). With a full group the
    round starts at once; a client that had to sit out its own matchmaking window first would join seconds later,
    or miss a group that closes in the meantime."""
    dhts = launch_dht_instances(3)
    averagers = [DecentralizedAverager([torch.full((16,), float(i))], dhts[i], start=True, prefix="late_leaders",
                                       target_group_size=3, min_matchmaking_time=4.0, request_timeout=1.0,
                                       client_mode=(i == 0)) for i in range(3)]
    try:
        started = time.perf_counter()
        client_step = averagers[0].step(wait=False, timeout=20, allow_retries=False)
        time.sleep(0.1)  # the client has found the group key empty by now
        others = [averager.step(wait=False, timeout=20, allow_retries=False) for averager in averagers[1:]]
        for control in [client_step] + others:
            assert len(control.result(30)) == 3
        assert time.perf_counter() - started < 3.0, "the client waited out its own window before it asked anybody"
        for averager in averagers:
            with averager.get_tensors() as tensors:
                assert torch.allclose(tensors[0], torch.full((16,), 1.0))
    finally:
        _shutdown(*averagers, *dhts)

"""Group formation around DecentralizedAverager: key manager, group bits, multi-round grids, gathered data,
more peers than a group holds, state download. Behaviours pinned by the reference's tests/test_averaging.py."""
import asyncio
import threading
import time

import pytest
import torch

from hivemind_b200.averaging import DecentralizedAverager
from hivemind_b200.averaging.group_info import GroupInfo
from hivemind_b200.averaging.key_manager import GroupKeyManager, is_valid_group
from hivemind_b200.dht import DHT
from hivemind_b200.utils.timed_storage import get_dht_time


def launch_dht_instances(n, **kwargs):
    first = DHT(start=True, **kwargs)
    maddrs = first.get_visible_maddrs()
    return [first] + [DHT(initial_peers=maddrs, start=True, **kwargs) for _ in range(n - 1)]


def _shutdown(*items):
    for item in items:
        item.shutdown()


def _step_all(averagers, **kwargs):
    """Run ``step`` on every averager at once; returns the per-averager results (exceptions included)."""
    results = [None] * len(averagers)

    def run(i):
        try:
            results[i] = averagers[i].step(**kwargs)
        except Exception as e:
            results[i] = e

    threads = [threading.Thread(target=run, args=(i,)) for i in range(len(averagers))]
    [t.start() for t in threads]
    [t.join(120) for t in threads]
    return results


def test_key_manager_declares_retracts_and_reshuffles():
    dht = DHT(start=True)
    try:
        assert is_valid_group("prefix.0b0101") and is_valid_group("prefix.0b")
        assert not is_valid_group("pre.fix.0b01") and not is_valid_group("prefix.0b012") and not is_valid_group("prefix")
        manager = GroupKeyManager(dht, "km", initial_group_bits="0110", target_group_size=4)
        assert manager.current_key == "km.0b0110"
        peers = [DHT(start=True, initial_peers=dht.get_visible_maddrs()) for _ in range(2)]
        try:
            now = get_dht_time()

            async def scenario(_dht, _node):
                ids = [p.peer_id for p in peers]
                assert await manager.declare_averager("km.0b0110", ids[0], now + 60)
                assert await manager.declare_averager("km.0b0110", ids[1], now + 61)
                assert await manager.declare_averager("km.0b1111", ids[1], now + 61)
                found = dict(await manager.get_averagers("km.0b0110", only_active=True))
                assert set(found) == set(ids) and found[ids[0]] == pytest.approx(now + 60)
                # a retraction outlives the announcement it cancels
                assert await manager.declare_averager("km.0b0110", ids[0], now + 60, looking_for_group=False)
                active = [p for p, _ in await manager.get_averagers("km.0b0110", only_active=True)]
                everyone = [p for p, _ in await manager.get_averagers("km.0b0110", only_active=False)]
                assert active == [ids[1]] and set(everyone) == set(ids)
                assert await manager.get_averagers("km.0b0000", only_active=True) == []
                return True

            assert dht.run_coroutine(scenario)

            # members of one group spread over different buckets; the key keeps its length
            members = tuple([dht.peer_id] + [p.peer_id for p in peers])
            buckets = set()
            for peer_id in members:
                m = GroupKeyManager(dht, "km", initial_group_bits="0110", target_group_size=4)
                m.peer_id = peer_id
                asyncio.new_event_loop().run_until_complete(
                    m.update_key_on_group_assembled(GroupInfo(b"group-id", members, gathered=(b"",) * 3)))
                assert len(m.group_bits) == 4 and m.group_bits[:2] == "10"  # old bits shift left by two
                buckets.add(m.group_bits[2:])
            assert len(buckets) == 3
        finally:
            _shutdown(*peers)
    finally:
        dht.shutdown()


def test_group_bits_can_be_read_and_set():
    dht = DHT(start=True)
    averager = DecentralizedAverager([torch.randn(3)], dht, start=True, prefix="bits", target_group_size=2,
                                     initial_group_bits="00101")
    try:
        assert averager.get_group_bits() == "00101"
        averager.set_group_bits("11011")
        assert averager.get_group_bits() == "11011"
        with pytest.raises(Exception):
            averager.set_group_bits("12")
    finally:
        _shutdown(averager, dht)


def test_grid_of_peers_converges_to_the_global_mean_in_log_rounds():
    """8 peers in groups of 2 under 2-bit keys (pairs share a key): every round the members of a group move to
    different keys, the number of distinct values halves, and after 3 rounds every peer holds the mean of all 8
    (reference: test_allreduce_grid)."""
    dhts = launch_dht_instances(8)
    torch.manual_seed(0)
    values = [torch.randn(16) for _ in range(8)]
    averagers = [DecentralizedAverager([values[i].clone()], dhts[i], start=True, prefix="grid", target_group_size=2,
                                       initial_group_bits=bin(i // 2)[2:].rjust(2, "0"), min_matchmaking_time=1.5,
                                       request_timeout=0.5) for i in range(8)]
    try:
        reference = torch.stack(values).mean(0)
        spread = []
        for round_index in range(3):
            results = _step_all(averagers, timeout=30)
            assert all(isinstance(r, dict) and len(r) == 2 for r in results), results
            with_tensors = []
            for a in averagers:
                with a.get_tensors() as ts:
                    with_tensors.append(ts[0].clone())
            spread.append(max((t - reference).abs().max().item() for t in with_tensors))
            distinct = {tuple(round(v, 4) for v in t.tolist()) for t in with_tensors}
            assert len(distinct) == 8 // 2 ** (round_index + 1)
        assert spread[2] < 1e-5 and spread[0] > spread[2]
    finally:
        _shutdown(*averagers, *dhts)


def test_gathered_data_reaches_every_group_member():
    dhts = launch_dht_instances(4)
    averagers = [DecentralizedAverager([torch.ones(4) * i], dhts[i], start=True, prefix="gather",
                                       target_group_size=4, min_matchmaking_time=2.0, request_timeout=0.5)
                 for i in range(4)]
    try:
        results = [None] * 4

        def run(i):
            results[i] = averagers[i].step(gather=dict(index=i, tag=f"peer{i}", blob=b"\x00" * i), timeout=30)

        threads = [threading.Thread(target=run, args=(i,)) for i in range(4)]
        [t.start() for t in threads]
        [t.join(60) for t in threads]
        for i, gathered in enumerate(results):
            assert len(gathered) == 4
            assert gathered[averagers[i].peer_id] == dict(index=i, tag=f"peer{i}", blob=b"\x00" * i)
            assert sorted(item["index"] for item in gathered.values()) == [0, 1, 2, 3]
        with averagers[2].get_tensors() as ts:
            assert torch.allclose(ts[0], torch.full((4,), 1.5))
    finally:
        _shutdown(*averagers, *dhts)


def test_more_peers_than_a_group_holds_all_get_averaged_eventually():
    """12 peers look for groups of 4 under one key; leaders turn away the overflow and everybody ends up in some
    group within a few attempts (reference: test_overcrowded)."""
    dhts = launch_dht_instances(12)
    averagers = [DecentralizedAverager([torch.ones(2) * i], dhts[i], start=True, prefix="crowd", target_group_size=4,
                                       min_matchmaking_time=2.0, request_timeout=0.5, initial_group_bits="")
                 for i in range(12)]
    try:
        successes = 0
        for _ in range(3):
            results = _step_all(averagers, timeout=8, allow_retries=False)
            ok = [r for r in results if isinstance(r, dict)]
            assert all(2 <= len(r) <= 4 for r in ok)
            successes += len(ok)
        assert successes >= 12  # on average at least a third of the attempts ends in a group
    finally:
        _shutdown(*averagers, *dhts)


class _StatefulAverager(DecentralizedAverager):
    """Shares a metadata dict and its tensors, like an optimizer-state averager would."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.metadata = {}

    def get_current_state(self):
        with self.get_tensors() as tensors:
            return dict(self.metadata), [t.clone() for t in tensors], None


def test_state_download_returns_metadata_and_tensors_and_respects_sharing_switch():
    dhts = launch_dht_instances(2)
    donor = _StatefulAverager([torch.arange(6, dtype=torch.float32), torch.ones(2, 3)], dhts[0], start=True,
                              prefix="state", target_group_size=2)
    donor.metadata = dict(step=17, note="hello")
    joiner = _StatefulAverager([torch.zeros(6), torch.zeros(2, 3)], dhts[1], start=True, prefix="state",
                               target_group_size=2, allow_state_sharing=False)
    try:
        deadline, loaded = time.time() + 30, None
        while loaded is None and time.time() < deadline:
            loaded = joiner.load_state_from_peers(timeout=5)
        metadata, tensors = loaded
        assert metadata == dict(step=17, note="hello")
        assert torch.equal(tensors[0], torch.arange(6, dtype=torch.float32)) and torch.equal(tensors[1], torch.ones(2, 3))
        # the joiner does not share: the donor finds nobody to download from
        assert donor.load_state_from_peers(timeout=3) is None
        donor.allow_state_sharing = False
        assert joiner.load_state_from_peers(timeout=3) is None
    finally:
        _shutdown(donor, joiner, *dhts)

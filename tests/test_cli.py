"""Command-line entry points: a DHT node and an expert server started as subprocesses (reference: tests/test_cli_scripts.py,
tests/test_start_server.py)."""
import os
import re
import signal
import subprocess
import sys
import time

import torch

from hivemind_b200.dht import DHT
from hivemind_b200.hivemind_cli.run_server import parse_args
from hivemind_b200.moe import get_experts

ENV = dict(os.environ, PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))), PYTHONUNBUFFERED="1")


def _wait_for_line(proc, pattern, timeout=60):
    deadline = time.time() + timeout
    seen = []
    while time.time() < deadline:
        line = proc.stderr.readline()
        if not line:
            if proc.poll() is not None:
                break
            continue
        seen.append(line)
        match = re.search(pattern, line)
        if match:
            return match
    raise AssertionError("pattern not found in output:\n" + "".join(seen))


def test_run_dht_and_join():
    first = subprocess.Popen([sys.executable, "-m", "hivemind_b200.hivemind_cli.run_dht", "--refresh_period", "1",
                              "--host_maddrs", "/ip4/127.0.0.1/tcp/0"], stderr=subprocess.PIPE, text=True, env=ENV)
    try:
        maddr = _wait_for_line(first, r"(/ip4/127\.0\.0\.1/tcp/\d+/p2p/\S+)").group(1)
        _wait_for_line(first, r"1 DHT nodes \(including this one\)")
        second = subprocess.Popen([sys.executable, "-m", "hivemind_b200.hivemind_cli.run_dht", "--refresh_period", "1",
                                   "--host_maddrs", "/ip4/127.0.0.1/tcp/0", "--initial_peers", maddr],
                                  stderr=subprocess.PIPE, text=True, env=ENV)
        try:
            _wait_for_line(second, r"2 DHT nodes \(including this one\)")
            _wait_for_line(first, r"2 DHT nodes \(including this one\)")
        finally:
            second.send_signal(signal.SIGTERM)
            assert second.wait(30) == 0
    finally:
        first.send_signal(signal.SIGTERM)
        assert first.wait(30) == 0


def test_run_server_cli(tmp_path):
    identity = tmp_path / "server.id"
    config = tmp_path / "server.yml"
    config.write_text("expert_cls: nop\nhidden_dim: 16\nmax_batch_size: 64\ninitial_peers: \"[]\"\n")
    args = parse_args(["-c", str(config), "--num_experts", "2", "--optimizer", "none"])
    assert args["expert_cls"] == "nop" and args["hidden_dim"] == 16 and args["num_experts"] == 2 and args["initial_peers"] == []
    proc = subprocess.Popen([sys.executable, "-m", "hivemind_b200.hivemind_cli.run_server", "-c", str(config),
                             "--expert_uids", "cli.0", "cli.1", "--device", "cpu", "--optimizer", "none",
                             "--identity_path", str(identity), "--host_maddrs", "/ip4/127.0.0.1/tcp/0",
                             "--num_handlers", "1"], stderr=subprocess.PIPE, text=True, env=ENV, cwd=str(tmp_path))
    try:
        maddr = _wait_for_line(proc, r"Running DHT node on \['(/ip4/127\.0\.0\.1/tcp/\d+/p2p/\S+?)'").group(1)
        _wait_for_line(proc, r"Started")
        assert identity.exists()
        dht = DHT(initial_peers=[maddr], start=True)
        try:
            deadline = time.time() + 30
            experts = [None, None]
            while time.time() < deadline and any(e is None for e in experts):
                experts = get_experts(dht, ["cli.0", "cli.1"])
                time.sleep(0.5)
            assert all(e is not None for e in experts)
            x = torch.randn(3, 16)
            assert torch.allclose(experts[0](x), x)
        finally:
            dht.shutdown()
    finally:
        proc.send_signal(signal.SIGTERM)
        assert proc.wait(30) == 0

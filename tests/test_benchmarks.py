"""The CPU modes of the benchmark scripts run end to end on small settings and print the JSON lines they promise
(the reference keeps its benchmarks alive through a CI job, .github/workflows/run-benchmarks.yml)."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ENV = dict(os.environ, PYTHONPATH=ROOT, PYTHONUNBUFFERED="1")


def _run(script: str, *args: str, timeout: float = 300):
    done = subprocess.run([sys.executable, os.path.join(ROOT, "benchmarks", script), *args], capture_output=True,
                          text=True, env=ENV, timeout=timeout, cwd=ROOT)
    assert done.returncode == 0, (done.stdout[-1500:], done.stderr[-1500:])
    lines = [json.loads(line) for line in done.stdout.splitlines() if line.startswith("{")]
    assert lines, done.stdout[-1500:]
    return lines


def test_dht_benchmark_both_workloads():
    (plain,) = _run("benchmark_dht.py", "--num_peers", "6", "--num_threads", "2", "--total_num_rounds", "2",
                    "--failure_rate", "0")
    assert plain["benchmark"] == "dht" and plain["store_success_rate"] == 1.0 and plain["get_success_rate"] == 1.0
    assert plain["stores"] == plain["gets"] == 2 * 2 * 4 and plain["alive_peers"] == 6

    (experts,) = _run("benchmark_dht.py", "--num_peers", "8", "--num_processes", "2", "--num_experts", "48",
                      "--expert_batch_size", "16", "--expiration", "999")
    assert experts["benchmark"] == "dht_experts" and experts["peers"] == 8 and experts["processes"] == 3
    assert experts["store_success_rate"] == 1.0 and experts["get_success_rate"] == 1.0
    assert experts["stored_records"] == 3 * experts["unique_uids"], "a uid and its two grid prefixes"
    assert experts["node_survival_rate"] == 1.0 and experts["mean_get_seconds_per_uid"] > 0


@pytest.mark.parametrize("extra", [(), ("--peer-processes",)])
def test_rpc_payload_benchmark(extra):
    lines = _run("benchmark_averaging.py", "--mode", "rpc_payload", "--num_peers", "2", "--sizes-mb", "2",
                 "--codecs", "none", "float16", "--rounds", "1", *extra)
    assert [line["codec"] for line in lines] == ["none", "float16"]
    for line in lines:
        assert line["benchmark"] == "averaging_rpc_payload" and line["processes"] == (2 if extra else 1)
        assert line["payload_mb_per_s_per_peer"] > 0
        if not extra:
            assert line["max_abs_error_vs_mean"] < (1e-5 if line["codec"] == "none" else 5e-3)


def test_swarm_averaging_benchmark():
    (line,) = _run("benchmark_averaging.py", "--mode", "swarm", "--num_peers", "4", "--target_group_size", "2",
                   "--num_rounds", "1", "--min_matchmaking_time", "2", "--round_timeout", "20", "--hid_size", "32",
                   "--num_layers", "1")
    assert line["benchmark"] == "averaging_swarm" and line["total_steps"] == 4 and line["successful_steps"] >= 2


def test_tensor_compression_benchmark():
    lines = _run("benchmark_tensor_compression.py", "--size", "50000", "--num_iters", "2")
    assert len(lines) >= 6  # one line per wire codec
    assert all(any(isinstance(value, float) for value in line.values()) for line in lines)

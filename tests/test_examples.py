"""The ALBERT example end to end on CPU with the tiny model: two trainers and the monitor as child processes."""
import os
import re
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ENV = dict(os.environ, PYTHONPATH=ROOT, PYTHONUNBUFFERED="1")
COMMON = ["--run_id", "example_test", "--host_maddrs", "/ip4/127.0.0.1/tcp/0"]
TRAIN = ["--model", "tiny", "--device", "cpu", "--target_batch_size", "64", "--per_device_train_batch_size", "8",
         "--seq_length", "32", "--matchmaking_time", "1.0", "--save_steps", "0", "--average_state_every", "1",
         "--request_timeout", "1.0", "--min_refresh_period", "0.1", "--default_refresh_period", "0.2",
         "--max_refresh_period", "0.5", "--delay_grad_averaging", "false", "--delay_optimizer_step", "false"]


def test_albert_example_trainers_and_monitor(tmp_path):
    first_log = open(tmp_path / "first.log", "w")
    first = subprocess.Popen([sys.executable, os.path.join(ROOT, "examples/albert/run_trainer.py"), *COMMON, *TRAIN,
                              "--max_epochs", "6", "--output_dir", str(tmp_path / "a")], stderr=first_log, stdout=first_log,
                             env=ENV)
    procs = [first]
    try:
        maddr, deadline = None, time.time() + 60
        while maddr is None and time.time() < deadline:
            found = re.search(r"(/ip4/127\.0\.0\.1/tcp/\d+/p2p/\S+)", (tmp_path / "first.log").read_text())
            maddr = found.group(1) if found else None
            time.sleep(0.2)
        assert maddr is not None, (tmp_path / "first.log").read_text()[-2000:]
        second_log = open(tmp_path / "second.log", "w")
        procs.append(subprocess.Popen([sys.executable, os.path.join(ROOT, "examples/albert/run_trainer.py"), *COMMON, *TRAIN,
                                       "--initial_peers", maddr, "--max_epochs", "6", "--output_dir", str(tmp_path / "b")],
                                      stderr=second_log, stdout=second_log, env=ENV))
        monitor_log = open(tmp_path / "monitor.log", "w")
        procs.append(subprocess.Popen([sys.executable, os.path.join(ROOT, "examples/albert/run_training_monitor.py"),
                                       *COMMON, "--initial_peers", maddr, "--refresh_period", "0.5", "--max_reports", "2"],
                                      stderr=monitor_log, stdout=monitor_log, env=ENV))
        for proc in procs:
            assert proc.wait(timeout=240) == 0, "\n".join((tmp_path / n).read_text()[-1500:]
                                                         for n in ("first.log", "second.log", "monitor.log"))
        assert "step 6" in (tmp_path / "first.log").read_text() or "step 6" in (tmp_path / "second.log").read_text()
        assert re.search(r"step \d+: \d+ peers alive", (tmp_path / "monitor.log").read_text())
    finally:
        for proc in procs:
            if proc.poll() is None:
                proc.kill()


def test_powersgd_benchmark_runs_on_cpu_with_two_ranks():
    """benchmarks/benchmark_powersgd.py end to end on the tiny GPT-2 (gloo ranks, host timers): the PowerSGD
    averager finishes its steps and the script prints one JSON line with positive throughput."""
    import json

    for averager in ("powersgd",):
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
               "127.0.0.1", "--master-port", "29577", os.path.join(ROOT, "benchmarks/benchmark_powersgd.py"),
               "--model", "tiny", "--steps", "2", "--warmup", "3", "--rank-r", "4", "--batch", "2", "--seq-len", "32",
               "--averager", averager]
        done = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=ROOT)
        assert done.returncode == 0, done.stderr[-2000:]
        lines = [line for line in done.stdout.splitlines() if line.startswith("{")]
        assert len(lines) == 1, done.stdout[-2000:]
        row = json.loads(lines[0])
        assert row["n_gpus"] == 2 and row["value"] > 0 and row["steps"] == 2
        assert row["config"]["model"] == "gpt2-tiny"
        if averager == "powersgd":
            assert row["averaged_elements_per_round"] < row["parameters"]  # factors are smaller than the gradients

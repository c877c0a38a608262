"""The ALBERT example end to end on CPU with the tiny model: two trainers and the monitor as child processes."""
import os
import re
import subprocess
import sys
import time

import pytest

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


def test_tokenized_corpus_feeds_the_trainer(tmp_path):
    """examples/albert/tokenize_corpus.py on a small synthetic corpus (training its own SentencePiece model), then
    one trainer for two epochs on the resulting file; the batch source never masks padding or marker tokens."""
    import random

    import torch

    pytest.importorskip("sentencepiece")
    rng = random.Random(0)
    words = ["alpha", "beta", "gamma", "delta", "epsilon", "zeta", "eta", "theta", "iota", "kappa", "lambda", "mu"]
    with open(tmp_path / "corpus.txt", "w") as corpus:
        for title in range(25):
            corpus.write(f" = Document {title} = \n")
            for _ in range(rng.randint(2, 9)):
                corpus.write(" ".join(rng.choice(words) for _ in range(rng.randint(3, 14))).capitalize() + ". ")
            corpus.write("\n\n")
    tokens_path = tmp_path / "tokens.pt"
    done = subprocess.run([sys.executable, os.path.join(ROOT, "examples/albert/tokenize_corpus.py"), "--text",
                           str(tmp_path / "corpus.txt"), "--out", str(tokens_path), "--train_vocab_size", "64",
                           "--seq_length", "32"], capture_output=True, text=True, env=ENV, timeout=120)
    assert done.returncode == 0, done.stderr[-2000:]
    data = torch.load(tokens_path)
    ids, special = data["input_ids"], data["special_ids"]
    assert ids.dtype == torch.int64 and ids.shape[1] == 32 and ids.shape[0] >= 25
    assert special == {"<pad>": 0, "<unk>": 1, "[CLS]": 2, "[SEP]": 3, "[MASK]": 4}
    assert (ids[:, 0] == special["[CLS]"]).all() and ((ids == special["[SEP]"]).sum(1) == 1).all()
    assert not (ids == special["[MASK]"]).any() and ids.max() < data["vocab_size"] <= 64
    after_sep = (ids == special["[SEP]"]).cumsum(1).roll(1, dims=1)
    after_sep[:, 0] = 0
    assert (ids[after_sep.bool()] == special["<pad>"]).all(), "only padding follows [SEP]"

    sys.path.insert(0, os.path.join(ROOT, "examples", "albert"))
    try:
        from arguments import TrainingArguments
        from run_trainer import BatchSource

        from hivemind_b200.models.albert import AlbertConfig
        args = TrainingArguments(dataset_path=str(tokens_path), seq_length=32, per_device_train_batch_size=16)
        batch = BatchSource(AlbertConfig.tiny(), args, seed=1).next()
    finally:
        sys.path.pop(0)
    scored = batch["labels"] != -100
    assert scored.any() and (batch["labels"][scored] > special["[MASK]"]).all(), "markers and padding are never targets"
    assert (batch["input_ids"][scored] == special["[MASK]"]).all()
    assert (batch["input_ids"][:, 0] == special["[CLS]"]).all()

    # the same corpus as rows of two segments, for both of ALBERT's objectives
    pairs_path = tmp_path / "pairs.pt"
    done = subprocess.run([sys.executable, os.path.join(ROOT, "examples/albert/tokenize_corpus.py"), "--text",
                           str(tmp_path / "corpus.txt"), "--out", str(pairs_path), "--train_vocab_size", "64",
                           "--seq_length", "32", "--sentence_order"], capture_output=True, text=True, env=ENV, timeout=120)
    assert done.returncode == 0, done.stderr[-2000:]
    pairs = torch.load(pairs_path)
    rows, kinds, order = pairs["input_ids"], pairs["token_type_ids"], pairs["sentence_order_label"]
    assert rows.shape == kinds.shape and order.shape == (rows.shape[0],) and set(order.tolist()) == {0, 1}
    assert ((rows == special["[SEP]"]).sum(1) == 2).all() and (rows[:, 0] == special["[CLS]"]).all()
    first_sep = (rows == special["[SEP]"]).float().argmax(1)
    columns = torch.arange(32).unsqueeze(0)
    real = rows != special["<pad>"]
    assert (kinds[real & (columns <= first_sep.unsqueeze(1))] == 0).all(), "segment A and its [SEP] are type 0"
    assert (kinds[real & (columns > first_sep.unsqueeze(1))] == 1).all(), "segment B and its [SEP] are type 1"
    assert (kinds[~real] == 0).all()

    for name, dataset, extra in (("plain", tokens_path, []), ("pairs", pairs_path, ["--sentence_order", "true"])):
        log = open(tmp_path / f"trainer_{name}.log", "w")
        trainer = subprocess.run([sys.executable, os.path.join(ROOT, "examples/albert/run_trainer.py"), *COMMON, *TRAIN,
                                  "--run_id", f"tokenized_{name}", "--dataset_path", str(dataset), "--max_epochs", "2",
                                  "--output_dir", str(tmp_path / f"out_{name}"), *extra],
                                 stderr=log, stdout=log, env=ENV, timeout=240)
        text = (tmp_path / f"trainer_{name}.log").read_text()
        assert trainer.returncode == 0 and "step 2" in text, text[-2000:]

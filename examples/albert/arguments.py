"""Command-line arguments of the ALBERT example, grouped the way the reference groups them
(examples/albert/arguments.py:7-151): swarm membership, averager, optimizer, model/data and training loop."""
import argparse
from dataclasses import dataclass, field, fields
from typing import List, Optional


@dataclass
class BaseTrainingArguments:
    run_id: str = field(default="albert", metadata={"help": "unique name of this collaborative run (DHT key prefix)"})
    initial_peers: List[str] = field(default_factory=list, metadata={
        "help": "multiaddrs of peers already in the run, e.g. /ip4/203.0.113.1/tcp/31337/p2p/XXXX; empty = start a new run"})
    host_maddrs: List[str] = field(default_factory=lambda: ["/ip4/0.0.0.0/tcp/0"], metadata={"help": "addresses to listen on"})
    announce_maddrs: List[str] = field(default_factory=list, metadata={"help": "addresses to announce to other peers"})
    identity_path: Optional[str] = field(default=None, metadata={"help": "private key file for a stable peer id"})


@dataclass
class AveragerArguments:
    target_group_size: int = field(default=256, metadata={"help": "maximum number of peers in one all-reduce group"})
    min_matchmaking_time: Optional[float] = field(default=None, metadata={"help": "override matchmaking_time for the averagers"})
    request_timeout: float = field(default=3.0, metadata={"help": "seconds to wait for a groupmate's answer during matchmaking"})


@dataclass
class ProgressTrackerArguments:
    min_refresh_period: float = field(default=0.5, metadata={"help": "shortest interval between progress refreshes"})
    max_refresh_period: float = field(default=30, metadata={"help": "longest interval between progress refreshes"})
    default_refresh_period: float = field(default=3, metadata={"help": "refresh interval before any estimate exists"})
    expected_drift_peers: float = field(default=3, metadata={"help": "expected number of peers that may join or leave per step"})
    expected_drift_rate: float = field(default=0.2, metadata={"help": "expected fraction of peers that may join or leave per step"})
    metadata_expiration: float = field(default=120, metadata={"help": "lifetime of a peer's progress record in the DHT"})


@dataclass
class OptimizerArguments:
    target_batch_size: int = field(default=4096, metadata={"help": "samples per collaborative optimizer step, over all peers"})
    client_mode: bool = field(default=False, metadata={"help": "never accept incoming connections (a peer behind a firewall)"})
    batch_size_lead: int = field(default=0, metadata={"help": "start looking for a group this many samples early"})
    matchmaking_time: float = field(default=5.0, metadata={"help": "seconds spent looking for groupmates before a step"})
    averaging_timeout: float = field(default=60.0, metadata={"help": "give up an averaging round after this many seconds"})
    next_chunk_timeout: float = field(default=10.0, metadata={"help": "ban a groupmate that stalls a transfer this long"})
    delay_optimizer_step: bool = field(default=True, metadata={"help": "run the optimizer step in the background"})
    delay_grad_averaging: bool = field(default=True, metadata={"help": "average gradients in the background"})
    average_state_every: int = field(default=5, metadata={"help": "average parameters and statistics every N steps"})
    use_local_updates: bool = field(default=False, metadata={"help": "local SGD: step locally, average only parameters"})
    grad_compression: str = field(default="uniform8", metadata={"help": "none | float16 | meanstd16 | uniform8 | quantile8 | blockwise8 | size_adaptive"})
    state_compression: str = field(default="float16", metadata={"help": "codec of parameter averaging and state downloads"})
    power_sgd_rank: int = field(default=0, metadata={"help": "if > 0, average gradients with PowerSGD of this rank"})


@dataclass
class TrainingArguments:
    model: str = field(default="large", metadata={"help": "large (ALBERT-large shape) or tiny (for smoke tests)"})
    seq_length: int = field(default=512, metadata={"help": "tokens per sequence"})
    per_device_train_batch_size: int = field(default=32, metadata={"help": "sequences per forward/backward pass"})
    gradient_accumulation_steps: int = field(default=1, metadata={"help": "passes between calls of the collaborative optimizer"})
    learning_rate: float = field(default=0.00176)
    warmup_steps: int = field(default=5000)
    total_steps: int = field(default=125000, metadata={"help": "length of the linear schedule, in collaborative steps"})
    adam_epsilon: float = field(default=1e-6)
    weight_decay: float = field(default=0.01)
    clamp_value: float = field(default=10000.0, metadata={"help": "LAMB clamps the weight norm in its trust ratio to this"})
    max_local_steps: Optional[int] = field(default=None, metadata={"help": "stop after this many forward/backward passes"})
    max_epochs: Optional[int] = field(default=None, metadata={"help": "stop after this many collaborative steps"})
    dataset_path: Optional[str] = field(default=None, metadata={
        "help": "a torch file with int64 'input_ids' [n, seq]; default: synthetic token ids"})
    sentence_order: bool = field(default=False, metadata={
        "help": "train sentence-order prediction next to the masked LM (every peer of a run must agree); the dataset "
                "then needs two-segment rows (tokenize_corpus.py --sentence_order), synthetic data gets random ones"})
    output_dir: str = field(default="outputs", metadata={"help": "where local checkpoints are written"})
    save_steps: int = field(default=500, metadata={"help": "save a local checkpoint every N collaborative steps (0 = never)"})
    backup_every_steps: int = field(default=10, metadata={"help": "keep an in-memory copy of the weights every N collaborative steps (rolled back to on NaN)"})
    seed: int = field(default=0)
    device: Optional[str] = field(default=None, metadata={"help": "torch device; default: cuda if present"})
    statistics_expiration: float = field(default=600, metadata={"help": "lifetime of this peer's metrics record in the DHT"})


def add_dataclass_arguments(parser: argparse.ArgumentParser, *dataclass_types) -> None:
    for cls in dataclass_types:
        group = parser.add_argument_group(cls.__name__)
        for f in fields(cls):
            help_text = f.metadata.get("help", "")
            default = f.default_factory() if f.default_factory is not field().default_factory else f.default  # type: ignore
            if f.type in (bool, "bool"):
                group.add_argument(f"--{f.name}", type=lambda s: s.lower() in ("1", "true", "yes"), default=default,
                                   help=help_text, metavar="BOOL")
            elif "List" in str(f.type):
                group.add_argument(f"--{f.name}", nargs="*", default=default, help=help_text)
            else:
                base = {"int": int, "float": float, "str": str}.get(
                    str(f.type).replace("typing.Optional[", "").replace("Optional[", "").rstrip("]").replace("<class '", "").rstrip("'>"), str)
                group.add_argument(f"--{f.name}", type=base, default=default, help=help_text)


def parse_into(namespace: argparse.Namespace, cls):
    return cls(**{f.name: getattr(namespace, f.name) for f in fields(cls)})

"""Host experts from the command line until SIGINT or SIGTERM.

Flags follow the reference's ``hivemind-server`` (hivemind/hivemind_cli/run_server.py:19-121). Options can also come
from a YAML file (``-c config.yml``; ``config.yml`` in the working directory is read if present); command-line
values win over the file.
"""
import argparse
import os
from functools import partial
from pathlib import Path
from signal import SIGINT, SIGTERM, signal, strsignal
from threading import Event

import torch
import yaml

from hivemind_b200.moe import Server
from hivemind_b200.moe.server.layers import schedule_name_to_scheduler
from hivemind_b200.proto.runtime_pb2 import CompressionType
from hivemind_b200.utils.limits import increase_file_limit
from hivemind_b200.utils.logging import get_logger, use_hivemind_log_handler

use_hivemind_log_handler("in_root_logger")
logger = get_logger(__name__)
DEFAULT_CONFIG = "config.yml"


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(description="Run a hivemind_b200 expert server")
    parser.add_argument("-c", "--config", default=None, help="YAML file with option values")
    parser.add_argument("--num_experts", type=int, default=None, help="The number of experts to serve")
    parser.add_argument("--expert_pattern", type=str, default=None,
                        help='expert uids are sampled from this pattern, e.g. "myexpert.[0:256].[0:1024]" means uids '
                             "between myexpert.0.0 and myexpert.255.1023; use with --num_experts, or use --expert_uids")
    parser.add_argument("--expert_uids", type=str, nargs="*", default=None, help="the exact list of expert uids")
    parser.add_argument("--expert_cls", type=str, default="ffn",
                        help="expert type: 'ffn', 'transformer', 'det_dropout', 'nop' or a class from --custom_module_path")
    parser.add_argument("--hidden_dim", type=int, default=1024, help="main dimension of the expert class")
    parser.add_argument("--host_maddrs", type=str, nargs="+", default=["/ip4/0.0.0.0/tcp/0"],
                        help="Multiaddrs to listen on; default: all IPv4 interfaces, any TCP port")
    parser.add_argument("--announce_maddrs", type=str, nargs="+", default=None, help="Visible multiaddrs to announce")
    parser.add_argument("--no_relay", action="store_false", dest="use_relay", help="accepted for compatibility")
    parser.add_argument("--use_auto_relay", action="store_true", help="accepted for compatibility; no effect")
    parser.add_argument("--num_handlers", type=int, default=None, help="number of connection handlers")
    parser.add_argument("--min_batch_size", type=int, default=1, help="minimum batch size of expert operations")
    parser.add_argument("--max_batch_size", type=int, default=16384, help="maximum number of rows in one batch")
    parser.add_argument("--device", type=str, default=None, help="torch device of all experts (default: cuda if present)")
    parser.add_argument("--optimizer", type=str, default="adam", help="adam, sgd or none")
    parser.add_argument("--scheduler", type=str, choices=list(schedule_name_to_scheduler.keys()), default="none",
                        help="learning-rate schedule")
    parser.add_argument("--num_warmup_steps", type=int, help="warm-up steps of the schedule")
    parser.add_argument("--num_training_steps", type=int, help="total steps of the schedule")
    parser.add_argument("--update_period", type=float, default=30, help="seconds between DHT declarations")
    parser.add_argument("--expiration", type=float, default=None, help="lifetime of DHT declarations in seconds")
    parser.add_argument("--clip_grad_norm", type=float, help="maximum gradient norm of each expert")
    parser.add_argument("--initial_peers", type=str, nargs="*", default=[], help="multiaddrs of DHT peers to join")
    parser.add_argument("--increase_file_limit", action="store_true", help="raise the open-files limit")
    parser.add_argument("--compression", type=str, default="NONE", help="tensor compression on the wire")
    parser.add_argument("--checkpoint_dir", type=Path, help="directory for expert checkpoints")
    parser.add_argument("--stats_report_interval", type=int, help="seconds between throughput reports")
    parser.add_argument("--custom_module_path", type=str, help="python file with @register_expert_class modules")
    parser.add_argument("--identity_path", type=str, help="private key file for a deterministic peer id")
    return parser


def parse_args(argv=None) -> dict:
    parser = build_parser()
    known, _ = parser.parse_known_args(argv)
    config_path = known.config or (DEFAULT_CONFIG if os.path.exists(DEFAULT_CONFIG) else None)
    if config_path is not None:
        with open(config_path) as f:
            values = yaml.safe_load(f) or {}
        valid = {action.dest for action in parser._actions}
        defaults = {}
        for key, value in values.items():
            if key in ("no_dht",):  # obsolete keys of old configuration files
                continue
            if key == "initial_peers" and isinstance(value, str):
                value = yaml.safe_load(value) or []
            if key not in valid:
                raise ValueError(f"unknown option {key!r} in {config_path}")
            defaults[key] = value
        parser.set_defaults(**defaults)
    args = vars(parser.parse_args(argv))
    args.pop("config", None)
    return args


def main(argv=None) -> None:
    args = parse_args(argv)
    optimizer = args.pop("optimizer")
    if optimizer == "adam":
        optim_cls = torch.optim.Adam
    elif optimizer == "sgd":
        optim_cls = partial(torch.optim.SGD, lr=0.01)
    elif optimizer == "none":
        optim_cls = None
    else:
        raise ValueError("optimizer must be adam, sgd or none")
    if args.pop("increase_file_limit"):
        increase_file_limit()
    compression = getattr(CompressionType, args.pop("compression"))
    server = Server.create(**args, optim_cls=optim_cls, start=True, compression=compression)
    exit_event = Event()

    def on_signal(number: int, _frame) -> None:
        logger.info(f"Caught signal {number} ({strsignal(number)}), shutting down")
        exit_event.set()

    signal(SIGTERM, on_signal)
    signal(SIGINT, on_signal)
    try:
        exit_event.wait()
    finally:
        server.shutdown()
        server.join()


if __name__ == "__main__":
    main()

"""Command-line entry points: ``python -m hivemind_b200.hivemind_cli.run_dht`` and ``...run_server``."""

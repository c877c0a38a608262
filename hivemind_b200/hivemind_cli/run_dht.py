"""Run a standalone DHT node (a bootstrap / rendezvous peer) until SIGINT or SIGTERM.

Same flags as the reference's ``hivemind-dht`` (hivemind/hivemind_cli/run_dht.py:26-107); every ``refresh_period``
seconds the node logs the size of its routing table and storage and issues a lookup that refreshes stale peers.
libp2p-specific switches (relays, IPFS bootstrap) are accepted for compatibility and have no effect on this
transport.
"""
from argparse import ArgumentParser
from secrets import token_hex
from signal import SIGINT, SIGTERM, signal, strsignal
from threading import Event

from hivemind_b200.dht import DHT, DHTNode
from hivemind_b200.utils.logging import get_logger, use_hivemind_log_handler
from hivemind_b200.utils.networking import log_visible_maddrs

use_hivemind_log_handler("in_root_logger")
logger = get_logger(__name__)


async def report_status(dht: DHT, node: DHTNode) -> None:
    known = len(node.protocol.routing_table.uid_to_peer_id) + 1
    logger.info(f"{known} DHT nodes (including this one) are in the local routing table")
    logger.debug(f"Routing table contents: {node.protocol.routing_table}")
    logger.info(f"Local storage contains {len(node.protocol.storage)} keys")
    logger.debug(f"Local storage contents: {node.protocol.storage}")
    await node.get(f"heartbeat_{token_hex(16)}", latest=True)  # touching the swarm evicts peers that are gone


def build_parser() -> ArgumentParser:
    parser = ArgumentParser(description="Run a hivemind_b200 DHT node")
    parser.add_argument("--initial_peers", nargs="*", default=[],
                        help="Multiaddrs of peers that will welcome you into an existing DHT, "
                             "e.g. /ip4/203.0.113.1/tcp/31337/p2p/XXXX /ip4/203.0.113.2/tcp/7777/p2p/YYYY")
    parser.add_argument("--host_maddrs", nargs="*", default=["/ip4/0.0.0.0/tcp/0"],
                        help="Multiaddrs to listen on; default: all IPv4 interfaces, any TCP port")
    parser.add_argument("--announce_maddrs", nargs="*", help="Visible multiaddrs to announce to other peers")
    parser.add_argument("--use_ipfs", action="store_true", help="accepted for compatibility; no effect")
    parser.add_argument("--identity_path", help="Private key file: makes the peer id deterministic "
                                                "(the key is created if the file does not exist)")
    parser.add_argument("--no_relay", action="store_false", dest="use_relay", help="accepted for compatibility")
    parser.add_argument("--use_auto_relay", action="store_true", help="accepted for compatibility; no effect")
    parser.add_argument("--refresh_period", type=int, default=30, help="Seconds between status reports")
    return parser


def main(argv=None) -> None:
    args = build_parser().parse_args(argv)
    dht = DHT(start=True, initial_peers=args.initial_peers, host_maddrs=args.host_maddrs,
              announce_maddrs=args.announce_maddrs, use_ipfs=args.use_ipfs, identity_path=args.identity_path,
              use_relay=args.use_relay, use_auto_relay=args.use_auto_relay)
    log_visible_maddrs(dht.get_visible_maddrs(), only_p2p=args.use_ipfs)
    exit_event = Event()

    def on_signal(number: int, _frame) -> None:
        logger.info(f"Caught signal {number} ({strsignal(number)}), shutting down")
        exit_event.set()

    signal(SIGTERM, on_signal)
    signal(SIGINT, on_signal)
    try:
        while not exit_event.is_set():
            dht.run_coroutine(report_status, return_future=False)
            exit_event.wait(args.refresh_period)
    finally:
        dht.shutdown()


if __name__ == "__main__":
    main()

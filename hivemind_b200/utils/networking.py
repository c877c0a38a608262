"""Address helpers (reference: hivemind/utils/networking.py:12-59)."""
from __future__ import annotations

from ipaddress import ip_address
from typing import List, Sequence

from hivemind_b200.utils.logging import TextStyle, get_logger
from hivemind_b200.utils.multiaddr import Multiaddr

LOCALHOST = "127.0.0.1"
logger = get_logger(__name__)


def choose_ip_address(maddrs: Sequence[Multiaddr], prefer_global: bool = True,
                      protocol_priority: Sequence[str] = ("ip4", "ip6")) -> str:
    """Pick the address another peer would most likely reach: global before private, ip4 before ip6."""
    for need_global in ((True, False) if prefer_global else (False, True)):
        for protocol in protocol_priority:
            for addr in maddrs:
                if protocol in addr:
                    value = addr[protocol]
                    if ip_address(value).is_global == need_global:
                        return value
    raise ValueError(f"no IP address found among {maddrs}")


def log_visible_maddrs(visible_maddrs: List[Multiaddr], only_p2p: bool) -> None:
    if only_p2p:
        unique = {addr["p2p"] for addr in visible_maddrs}
        initial_peers = " ".join(f"/p2p/{addr}" for addr in unique)
    else:
        available_ips = [Multiaddr(addr) for addr in visible_maddrs if "ip4" in addr or "ip6" in addr]
        if available_ips:
            preferred = choose_ip_address(available_ips)
            selected = [addr for addr in visible_maddrs if preferred in str(addr)]
            if selected:
                visible_maddrs = selected
        initial_peers = " ".join(str(addr) for addr in visible_maddrs)
    logger.info(f"Running a DHT instance. To connect other peers to this one, use "
                f"{TextStyle.get('BOLD')}{TextStyle.get('BLUE')}--initial_peers {initial_peers}{TextStyle.get('RESET')}")
    logger.info(f"Full list of visible multiaddresses: {' '.join(str(addr) for addr in visible_maddrs)}")

"""``PeerID``, ``PeerInfo``, ``StreamInfo`` under the reference's module path
(hivemind/p2p/p2p_daemon_bindings/datastructures.py)."""
from hivemind_b200.p2p.datastructures import PeerID, PeerInfo, StreamInfo, sha256_digest  # noqa: F401

from hivemind_b200.p2p.control import P2PDaemonError, P2PHandlerError
from hivemind_b200.p2p.datastructures import PeerID, PeerInfo, StreamInfo
from hivemind_b200.p2p.p2p_daemon import P2P, P2PContext, RPCError
from hivemind_b200.p2p.servicer import ServicerBase, StubBase

"""Module paths of the reference's daemon bindings (hivemind/p2p/p2p_daemon_bindings/).

``utils`` holds the libp2p daemon's message framing (varint-prefixed ``p2pd_pb2`` messages) and the error types;
``control``, ``p2pclient`` and ``datastructures`` give the reference's names to this package's control client and
data types, whose implementations live in ``hivemind_b200.p2p.control`` and ``hivemind_b200.p2p.datastructures``
(the transport daemon of this package speaks its own framed protocol)."""

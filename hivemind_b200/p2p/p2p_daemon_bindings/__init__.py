"""Import paths of the reference's daemon bindings (hivemind/p2p/p2p_daemon_bindings/), kept so that code written
against them finds the same names here. The implementations live in ``hivemind_b200.p2p.control`` and
``hivemind_b200.p2p.datastructures``: the transport daemon of this package speaks its own framed protocol, not the
libp2p daemon's protobuf control protocol."""

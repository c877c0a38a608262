"""Self-describing network addresses: ``/ip4/127.0.0.1/tcp/4001/p2p/Qm...`` (text and binary forms).

The reference vendors py-multiaddr (hivemind/utils/multiaddr/*, 1.4k lines, depending on the absent wheels
``netaddr``, ``varint``, ``base58``, ``py-cid``, ``py-multihash``). This is an independent implementation of the
subset a swarm on IP networks uses: ip4, ip6, dns*, tcp, udp, quic, ws, tls, unix, p2p, p2p-circuit.
"""
from hivemind_b200.utils.multiaddr.multiaddr import Multiaddr, Protocol, protocol_with_code, protocol_with_name  # noqa
from hivemind_b200.utils.multiaddr import protocols  # noqa

"""Self-describing network addresses: ``/ip4/127.0.0.1/tcp/4001/p2p/Qm...`` in text and binary form.

The reference vendors py-multiaddr (hivemind/utils/multiaddr/*, depending on the absent wheels ``netaddr``,
``varint``, ``base58``, ``py-cid``, ``py-multihash``). This package is written from the format's specification with
the same module layout and names: ``Multiaddr`` (``multiaddr``), ``Protocol`` / ``ProtocolRegistry`` / ``REGISTRY`` /
``protocol_with_*`` (``protocols``), ``string_to_bytes`` / ``bytes_to_string`` / ``bytes_iter`` (``transforms``), value
codecs for ip4, ip6, ip6zone, ports, host names, unix paths, onion / onion3 and peer ids (``codecs``), and the error
classes (``exceptions``).
"""
from hivemind_b200.utils.multiaddr import exceptions, protocols, transforms  # noqa: F401
from hivemind_b200.utils.multiaddr.multiaddr import Multiaddr  # noqa: F401
from hivemind_b200.utils.multiaddr.protocols import (Protocol, protocol_with_any, protocol_with_code,  # noqa: F401
                                                     protocol_with_name, protocols_with_string)

__all__ = ("Multiaddr", "Protocol", "protocol_with_name", "protocol_with_code", "protocol_with_any",
           "protocols_with_string", "protocols", "transforms", "exceptions")

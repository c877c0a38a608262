"""The control client under the reference's module path (hivemind/p2p/p2p_daemon_bindings/control.py:89).
``ControlClient`` is this package's ``DaemonClient``: same role (one-shot commands, the persistent multiplexed
connection for unary calls, inbound stream listener), different wire protocol."""
from hivemind_b200.p2p.control import (DEFAULT_MAX_MSG_SIZE, MAX_UNARY_PAYLOAD_SIZE, DaemonClient, StreamHandler,  # noqa: F401
                                       UnaryHandler)

ControlClient = DaemonClient

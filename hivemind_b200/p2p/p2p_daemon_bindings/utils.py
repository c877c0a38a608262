"""Error types of the daemon bindings under the reference's module path
(hivemind/p2p/p2p_daemon_bindings/utils.py:16-33)."""
from hivemind_b200.p2p.control import DispatchFailure, P2PDaemonError, P2PHandlerError  # noqa: F401


class ControlFailure(P2PDaemonError):
    """The daemon answered a control request with an error."""

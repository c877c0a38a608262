"""``Client`` under the reference's module path (hivemind/p2p/p2p_daemon_bindings/p2pclient.py:21): there it is a
thin facade over ``ControlClient``; here the control client already has that interface."""
from hivemind_b200.p2p.control import DaemonClient

Client = DaemonClient

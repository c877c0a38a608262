"""Control protocol of the go-libp2p-daemon (schema of hivemind/proto/p2pd.proto, package ``p2pclient.p2pd.pb``).

This package's own transport daemon speaks a simpler framing (``hivemind_b200/p2p/control.py``); the messages are here
for tools that talk to a libp2p daemon and for the framing helpers in ``hivemind_b200.p2p.p2p_daemon_bindings.utils``.
"""
from hivemind_b200.proto._schema import build_file

_TYPE = ("type", 1, "Type", "required")

_m = build_file(
    "hivemind_b200/p2pd.proto", package="p2pclient.p2pd.pb", syntax="proto2",
    messages={
        "Request": dict(
            enums={"Type": [("IDENTIFY", 0), ("CONNECT", 1), ("STREAM_OPEN", 2), ("STREAM_HANDLER", 3),
                            ("REMOVE_STREAM_HANDLER", 10), ("DHT", 4), ("LIST_PEERS", 5), ("CONNMANAGER", 6),
                            ("DISCONNECT", 7), ("PUBSUB", 8), ("PERSISTENT_CONN_UPGRADE", 9)]},
            fields=[_TYPE, ("connect", 2, "ConnectRequest", "optional"), ("streamOpen", 3, "StreamOpenRequest", "optional"),
                    ("streamHandler", 4, "StreamHandlerRequest", "optional"),
                    ("removeStreamHandler", 9, "RemoveStreamHandlerRequest", "optional"),
                    ("dht", 5, "DHTRequest", "optional"), ("connManager", 6, "ConnManagerRequest", "optional"),
                    ("disconnect", 7, "DisconnectRequest", "optional"), ("pubsub", 8, "PSRequest", "optional")]),
        "Response": dict(
            enums={"Type": [("OK", 0), ("ERROR", 1)]},
            fields=[_TYPE, ("error", 2, "ErrorResponse", "optional"), ("streamInfo", 3, "StreamInfo", "optional"),
                    ("identify", 4, "IdentifyResponse", "optional"), ("dht", 5, "DHTResponse", "optional"),
                    ("peers", 6, "PeerInfo", "repeated"), ("pubsub", 7, "PSResponse", "optional")]),
        "PersistentConnectionRequest": dict(
            oneofs={"message": ["addUnaryHandler", "removeUnaryHandler", "callUnary", "unaryResponse", "cancel"]},
            fields=[("callId", 1, "bytes", "required"), ("addUnaryHandler", 2, "AddUnaryHandlerRequest", "optional"),
                    ("removeUnaryHandler", 6, "RemoveUnaryHandlerRequest", "optional"),
                    ("callUnary", 3, "CallUnaryRequest", "optional"), ("unaryResponse", 4, "CallUnaryResponse", "optional"),
                    ("cancel", 5, "Cancel", "optional")]),
        "PersistentConnectionResponse": dict(
            oneofs={"message": ["callUnaryResponse", "requestHandling", "daemonError", "cancel"]},
            fields=[("callId", 1, "bytes", "required"), ("callUnaryResponse", 2, "CallUnaryResponse", "optional"),
                    ("requestHandling", 3, "CallUnaryRequest", "optional"), ("daemonError", 4, "DaemonError", "optional"),
                    ("cancel", 5, "Cancel", "optional")]),
        "IdentifyResponse": [("id", 1, "bytes", "required"), ("addrs", 2, "bytes", "repeated")],
        "ConnectRequest": [("peer", 1, "bytes", "required"), ("addrs", 2, "bytes", "repeated"),
                           ("timeout", 3, "int64", "optional")],
        "StreamOpenRequest": [("peer", 1, "bytes", "required"), ("proto", 2, "string", "repeated"),
                              ("timeout", 3, "int64", "optional")],
        "StreamHandlerRequest": [("addr", 1, "bytes", "required"), ("proto", 2, "string", "repeated"),
                                 ("balanced", 3, "bool", "required")],
        "RemoveStreamHandlerRequest": [("addr", 1, "bytes", "required"), ("proto", 2, "string", "repeated")],
        "ErrorResponse": [("msg", 1, "string", "required")],
        "StreamInfo": [("peer", 1, "bytes", "required"), ("addr", 2, "bytes", "required"), ("proto", 3, "string", "required")],
        "DHTRequest": dict(
            enums={"Type": [("FIND_PEER", 0), ("FIND_PEERS_CONNECTED_TO_PEER", 1), ("FIND_PROVIDERS", 2),
                            ("GET_CLOSEST_PEERS", 3), ("GET_PUBLIC_KEY", 4), ("GET_VALUE", 5), ("SEARCH_VALUE", 6),
                            ("PUT_VALUE", 7), ("PROVIDE", 8)]},
            fields=[_TYPE, ("peer", 2, "bytes", "optional"), ("cid", 3, "bytes", "optional"), ("key", 4, "bytes", "optional"),
                    ("value", 5, "bytes", "optional"), ("count", 6, "int32", "optional"), ("timeout", 7, "int64", "optional")]),
        "DHTResponse": dict(
            enums={"Type": [("BEGIN", 0), ("VALUE", 1), ("END", 2)]},
            fields=[_TYPE, ("peer", 2, "PeerInfo", "optional"), ("value", 3, "bytes", "optional")]),
        "PeerInfo": [("id", 1, "bytes", "required"), ("addrs", 2, "bytes", "repeated")],
        "ConnManagerRequest": dict(
            enums={"Type": [("TAG_PEER", 0), ("UNTAG_PEER", 1), ("TRIM", 2)]},
            fields=[_TYPE, ("peer", 2, "bytes", "optional"), ("tag", 3, "string", "optional"), ("weight", 4, "int64", "optional")]),
        "DisconnectRequest": [("peer", 1, "bytes", "required")],
        "PSRequest": dict(
            enums={"Type": [("GET_TOPICS", 0), ("LIST_PEERS", 1), ("PUBLISH", 2), ("SUBSCRIBE", 3)]},
            fields=[_TYPE, ("topic", 2, "string", "optional"), ("data", 3, "bytes", "optional")]),
        "PSMessage": [("from", 1, "bytes", "optional"), ("data", 2, "bytes", "optional"), ("seqno", 3, "bytes", "optional"),
                      ("topicIDs", 4, "string", "repeated"), ("signature", 5, "bytes", "optional"), ("key", 6, "bytes", "optional")],
        "PSResponse": [("topics", 1, "string", "repeated"), ("peerIDs", 2, "bytes", "repeated")],
        "CallUnaryRequest": [("peer", 1, "bytes", "required"), ("proto", 2, "string", "required"), ("data", 3, "bytes", "required")],
        "CallUnaryResponse": dict(oneofs={"result": ["response", "error"]},
                                  fields=[("response", 1, "bytes", "optional"), ("error", 2, "bytes", "optional")]),
        "AddUnaryHandlerRequest": [("proto", 1, "string", "required"), ("balanced", 2, "bool", "required")],
        "RemoveUnaryHandlerRequest": [("proto", 1, "string", "required")],
        "DaemonError": [("message", 1, "string", "optional")],
        "Cancel": [],
        "RPCError": [("message", 1, "string", "optional")],
    },
)
globals().update(_m)
__all__ = tuple(_m)

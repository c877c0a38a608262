"""DHT ping / store / find messages (schema of hivemind/proto/dht.proto:7-65)."""
from hivemind_b200.proto import auth_pb2  # noqa: F401  (registers the auth dependency)
from hivemind_b200.proto._schema import build_file

_m = build_file(
    "hivemind_b200/dht.proto",
    deps=["hivemind_b200/auth.proto"],
    enums={"ResultType": [("NOT_FOUND", 0), ("FOUND_REGULAR", 1), ("FOUND_DICTIONARY", 2)]},
    messages={
        "NodeInfo": [("node_id", 1, "bytes", "")],
        "PingRequest": [("auth", 1, "RequestAuthInfo", ""), ("peer", 2, "NodeInfo", ""), ("validate", 3, "bool", "")],
        "PingResponse": [("auth", 1, "ResponseAuthInfo", ""), ("peer", 2, "NodeInfo", ""),
                         ("dht_time", 4, "double", ""), ("available", 5, "bool", "")],
        "StoreRequest": [("auth", 1, "RequestAuthInfo", ""), ("keys", 2, "bytes", "repeated"),
                         ("subkeys", 3, "bytes", "repeated"), ("values", 4, "bytes", "repeated"),
                         ("expiration_time", 5, "double", "repeated"), ("in_cache", 6, "bool", "repeated"),
                         ("peer", 7, "NodeInfo", "")],
        "StoreResponse": [("auth", 1, "ResponseAuthInfo", ""), ("store_ok", 2, "bool", "repeated"),
                          ("peer", 3, "NodeInfo", "")],
        "FindRequest": [("auth", 1, "RequestAuthInfo", ""), ("keys", 2, "bytes", "repeated"), ("peer", 3, "NodeInfo", "")],
        "FindResult": [("type", 1, "ResultType", ""), ("value", 2, "bytes", ""), ("expiration_time", 3, "double", ""),
                       ("nearest_node_ids", 4, "bytes", "repeated"), ("nearest_peer_ids", 5, "bytes", "repeated")],
        "FindResponse": [("auth", 1, "ResponseAuthInfo", ""), ("results", 2, "FindResult", "repeated"),
                         ("peer", 3, "NodeInfo", "")],
    },
)
NodeInfo, PingRequest, PingResponse = _m["NodeInfo"], _m["PingRequest"], _m["PingResponse"]
StoreRequest, StoreResponse, FindRequest = _m["StoreRequest"], _m["StoreResponse"], _m["FindRequest"]
FindResult, FindResponse, ResultType = _m["FindResult"], _m["FindResponse"], _m["ResultType"]
NOT_FOUND, FOUND_REGULAR, FOUND_DICTIONARY = 0, 1, 2

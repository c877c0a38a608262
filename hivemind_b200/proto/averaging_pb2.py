"""Matchmaking, all-reduce and state-download messages (schema of hivemind/proto/averaging.proto:5-56)."""
from hivemind_b200.proto import runtime_pb2  # noqa: F401  (registers the Tensor dependency)
from hivemind_b200.proto._schema import build_file

_CODES = ["NO_CODE", "REQUEST_JOIN", "ACCEPTED", "BEGIN_ALLREDUCE", "PART_FOR_AVERAGING", "AVERAGED_PART",
          "NOT_DECLARED", "NOT_A_LEADER", "BAD_EXPIRATION_TIME", "BAD_SCHEMA_HASH", "BAD_GROUP_ID",
          "DUPLICATE_PEER_ID", "GROUP_IS_FULL", "NOT_LOOKING_FOR_GROUP", "PROTOCOL_VIOLATION", "INTERNAL_ERROR",
          "CANCELLED", "GROUP_DISBANDED", "BAD_GROUP_KEY"]

_m = build_file(
    "hivemind_b200/averaging.proto",
    deps=["hivemind_b200/runtime.proto"],
    enums={"MessageCode": [(name, i) for i, name in enumerate(_CODES)]},
    messages={
        "JoinRequest": [("schema_hash", 2, "bytes", ""), ("expiration", 3, "double", ""), ("gather", 4, "bytes", ""),
                        ("client_mode", 5, "bool", ""), ("group_key", 6, "string", "")],
        "MessageFromLeader": [("code", 1, "MessageCode", ""), ("group_id", 2, "bytes", ""),
                              ("suggested_leader", 3, "bytes", ""), ("ordered_peer_ids", 4, "bytes", "repeated"),
                              ("gathered", 5, "bytes", "repeated")],
        "AveragingData": [("code", 1, "MessageCode", ""), ("group_id", 2, "bytes", ""), ("peer_id", 3, "bytes", ""),
                          ("tensor_part", 4, "Tensor", ""), ("weight", 5, "double", "")],
        "DownloadRequest": [],
        "DownloadData": [("metadata", 1, "bytes", ""), ("tensor_part", 2, "Tensor", "")],
    },
)
JoinRequest, MessageFromLeader, AveragingData = _m["JoinRequest"], _m["MessageFromLeader"], _m["AveragingData"]
DownloadRequest, DownloadData, MessageCode = _m["DownloadRequest"], _m["DownloadData"], _m["MessageCode"]
for _i, _name in enumerate(_CODES):
    globals()[_name] = _i

"""Tensor and expert RPC messages (schema of hivemind/proto/runtime.proto:1-39)."""
from hivemind_b200.proto._schema import build_file

_m = build_file(
    "hivemind_b200/runtime.proto",
    enums={"CompressionType": [("NONE", 0), ("MEANSTD_16BIT", 1), ("FLOAT16", 2), ("QUANTILE_8BIT", 3),
                               ("UNIFORM_8BIT", 4), ("BLOCKWISE_8BIT", 5)]},
    messages={
        "ExpertUID": [("uid", 1, "string", "")],
        "ExpertInfo": [("serialized_info", 1, "bytes", "")],
        "Tensor": [("buffer", 1, "bytes", ""), ("size", 2, "uint32", "repeated"), ("requires_grad", 3, "bool", ""),
                   ("dtype", 4, "string", ""), ("compression", 5, "CompressionType", ""), ("chunks", 6, "int32", "")],
        "ExpertRequest": [("uid", 1, "string", ""), ("tensors", 2, "Tensor", "repeated"), ("metadata", 3, "bytes", "")],
        "ExpertResponse": [("tensors", 2, "Tensor", "repeated"), ("metadata", 3, "bytes", "")],
    },
)
ExpertUID, ExpertInfo, Tensor = _m["ExpertUID"], _m["ExpertInfo"], _m["Tensor"]
ExpertRequest, ExpertResponse = _m["ExpertRequest"], _m["ExpertResponse"]
CompressionType = _m["CompressionType"]
NONE, MEANSTD_16BIT, FLOAT16, QUANTILE_8BIT, UNIFORM_8BIT, BLOCKWISE_8BIT = range(6)

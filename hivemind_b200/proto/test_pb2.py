"""Toy request/response messages for transport tests (schema of hivemind/proto/test.proto)."""
from hivemind_b200.proto._schema import build_file

_m = build_file(
    "hivemind_b200/test.proto",
    messages={"TestRequest": [("number", 1, "int32", "")], "TestResponse": [("number", 1, "int32", "")]},
)
TestRequest, TestResponse = _m["TestRequest"], _m["TestResponse"]

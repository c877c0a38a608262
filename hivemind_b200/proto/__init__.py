"""Protobuf schemas of the wire protocol, built at import time (no protoc needed)."""
from hivemind_b200.proto import auth_pb2, averaging_pb2, crypto_pb2, dht_pb2, runtime_pb2, test_pb2  # noqa: F401

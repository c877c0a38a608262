"""libp2p key envelope used to derive peer ids from identity keys (schema of hivemind/proto/crypto.proto)."""
from hivemind_b200.proto._schema import build_file

_m = build_file(
    "hivemind_b200/crypto.proto",
    package="crypto.pb",
    syntax="proto2",
    enums={"KeyType": [("RSA", 0), ("Ed25519", 1), ("Secp256k1", 2), ("ECDSA", 3)]},
    messages={
        "PublicKey": [("key_type", 1, "KeyType", "required"), ("data", 2, "bytes", "required")],
        "PrivateKey": [("key_type", 1, "KeyType", "required"), ("data", 2, "bytes", "required")],
    },
)
PublicKey, PrivateKey, KeyType = _m["PublicKey"], _m["PrivateKey"], _m["KeyType"]
RSA, Ed25519, Secp256k1, ECDSA = 0, 1, 2, 3

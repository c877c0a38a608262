"""Access tokens and signed request/response envelopes (schema of hivemind/proto/auth.proto:3-22)."""
from hivemind_b200.proto._schema import build_file

_m = build_file(
    "hivemind_b200/auth.proto",
    messages={
        "AccessToken": [("username", 1, "string", ""), ("public_key", 2, "bytes", ""),
                        ("expiration_time", 3, "string", ""), ("signature", 4, "bytes", "")],
        "RequestAuthInfo": [("client_access_token", 1, "AccessToken", ""), ("service_public_key", 2, "bytes", ""),
                            ("time", 3, "double", ""), ("nonce", 4, "bytes", ""), ("signature", 5, "bytes", "")],
        "ResponseAuthInfo": [("service_access_token", 1, "AccessToken", ""), ("nonce", 2, "bytes", ""),
                             ("signature", 3, "bytes", "")],
    },
)
AccessToken, RequestAuthInfo, ResponseAuthInfo = _m["AccessToken"], _m["RequestAuthInfo"], _m["ResponseAuthInfo"]

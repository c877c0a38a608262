"""Peer identity and stream metadata.

``PeerID`` follows the libp2p rule used by the reference (hivemind/p2p/p2p_daemon_bindings/datastructures.py:18-88):
the id is the multihash of the protobuf-wrapped public key — identity multihash for encodings of at most 42 bytes,
sha2-256 otherwise — and prints as base58.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass
from typing import Any, List, Optional, Sequence, Union

from cryptography.hazmat.primitives import serialization

from hivemind_b200.proto import crypto_pb2
from hivemind_b200.utils.base58 import b58decode, b58encode, varint_encode
from hivemind_b200.utils.multiaddr import Multiaddr

_MULTIHASH_IDENTITY, _MULTIHASH_SHA256 = 0x00, 0x12
_MAX_INLINE_KEY_LENGTH = 42


class PeerID:
    """A peer's identity: the multihash bytes; the base58 text form is derived the first time somebody asks for it
    (routing replies create thousands of these per second and almost never print them)."""

    __slots__ = ("_bytes", "_text")

    def __init__(self, peer_id_bytes: bytes) -> None:
        self._bytes = bytes(peer_id_bytes)
        self._text: Optional[str] = None

    @property
    def _b58_str(self) -> str:
        if self._text is None:
            self._text = b58encode(self._bytes)
        return self._text

    def to_bytes(self) -> bytes:
        return self._bytes

    def to_base58(self) -> str:
        return self._b58_str

    to_string = to_base58

    def __getstate__(self):
        return (self._bytes,)

    def __setstate__(self, state):
        (self._bytes,), self._text = state, None

    @property
    def xor_id(self) -> int:
        return int(hashlib.sha256(self._bytes).hexdigest(), 16)

    def pretty(self) -> str:
        return self._b58_str

    def __repr__(self) -> str:
        return f"<PeerID {self._b58_str}>"

    def __str__(self) -> str:
        return self._b58_str

    def __eq__(self, other: Any) -> bool:
        if isinstance(other, str):
            return self._b58_str == other
        if isinstance(other, bytes):
            return self._bytes == other
        if isinstance(other, PeerID):
            return self._bytes == other._bytes
        return False

    def __lt__(self, other: Any) -> bool:
        if not isinstance(other, PeerID):
            raise TypeError(f"'<' not supported between PeerID and {type(other)}")
        return self._b58_str < other._b58_str

    def __hash__(self) -> int:
        return hash(self._bytes)

    @classmethod
    def from_base58(cls, b58_encoded: str) -> "PeerID":
        peer_id = cls(b58decode(b58_encoded))
        peer_id._text = b58_encoded
        return peer_id

    @classmethod
    def from_identity(cls, data: bytes) -> "PeerID":
        """Derive the id from a serialized ``crypto.pb.PrivateKey`` holding a DER-encoded RSA key."""
        key_data = crypto_pb2.PrivateKey.FromString(data).data
        private_key = serialization.load_der_private_key(key_data, password=None)
        return cls.from_private_key(private_key)

    @classmethod
    def from_private_key(cls, private_key) -> "PeerID":
        public_der = private_key.public_key().public_bytes(encoding=serialization.Encoding.DER,
                                                           format=serialization.PublicFormat.SubjectPublicKeyInfo)
        encoded = crypto_pb2.PublicKey(key_type=crypto_pb2.RSA, data=public_der).SerializeToString()
        if len(encoded) <= _MAX_INLINE_KEY_LENGTH:
            digest, code = encoded, _MULTIHASH_IDENTITY
        else:
            digest, code = hashlib.sha256(encoded).digest(), _MULTIHASH_SHA256
        return cls(varint_encode(code) + varint_encode(len(digest)) + digest)


def sha256_digest(data: Union[str, bytes]) -> bytes:
    if isinstance(data, str):
        data = data.encode("utf8")
    return hashlib.sha256(data).digest()


@dataclass(frozen=True)
class StreamInfo:
    peer_id: PeerID
    addr: Multiaddr
    proto: str

    def __repr__(self) -> str:
        return f"<StreamInfo peer_id={self.peer_id} addr={self.addr} proto={self.proto}>"

    def to_protobuf(self):
        """The ``p2pd_pb2.StreamInfo`` form (peer id and address in their binary forms)."""
        from hivemind_b200.proto import p2pd_pb2

        return p2pd_pb2.StreamInfo(peer=self.peer_id.to_bytes(), addr=self.addr.to_bytes(), proto=self.proto)

    @classmethod
    def from_protobuf(cls, message) -> "StreamInfo":
        return cls(peer_id=PeerID(message.peer), addr=Multiaddr(message.addr), proto=message.proto)


class PeerInfo:
    def __init__(self, peer_id: PeerID, addrs: Sequence[Multiaddr]) -> None:
        self.peer_id = peer_id
        self.addrs: List[Multiaddr] = list(addrs)

    def __eq__(self, other: Any) -> bool:
        return isinstance(other, PeerInfo) and self.peer_id == other.peer_id and self.addrs == other.addrs

    def __repr__(self) -> str:
        return f"PeerInfo(peer_id={self.peer_id!r}, addrs={self.addrs!r})"

    @classmethod
    def from_protobuf(cls, message) -> "PeerInfo":
        """From a ``p2pd_pb2.PeerInfo`` (or any message with ``id`` and repeated binary ``addrs``)."""
        return cls(PeerID(message.id), [Multiaddr(raw) for raw in message.addrs])

    def to_protobuf(self):
        from hivemind_b200.proto import p2pd_pb2

        return p2pd_pb2.PeerInfo(id=self.peer_id.to_bytes(), addrs=[addr.to_bytes() for addr in self.addrs])

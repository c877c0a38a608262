"""RSA keys for signed DHT records and access tokens (reference: hivemind/utils/crypto.py:12-101).

RSA-2048, PSS padding with SHA-256, signatures base64-encoded; public keys serialise to the OpenSSH
``ssh-rsa ...`` text form so that they can be embedded in DHT keys.
"""
from __future__ import annotations

import base64
import threading
from abc import ABC, abstractmethod
from typing import Optional

from cryptography import exceptions
from cryptography.hazmat.primitives import hashes, serialization
from cryptography.hazmat.primitives.asymmetric import padding, rsa

_PADDING = padding.PSS(mgf=padding.MGF1(hashes.SHA256()), salt_length=padding.PSS.MAX_LENGTH)


class PrivateKey(ABC):
    @abstractmethod
    def sign(self, data: bytes) -> bytes:
        ...

    @abstractmethod
    def get_public_key(self) -> "PublicKey":
        ...


class PublicKey(ABC):
    @abstractmethod
    def verify(self, data: bytes, signature: bytes) -> bool:
        ...

    @abstractmethod
    def to_bytes(self) -> bytes:
        ...

    @classmethod
    @abstractmethod
    def from_bytes(cls, key: bytes) -> "PublicKey":
        ...


class RSAPrivateKey(PrivateKey):
    _process_wide_key: Optional["RSAPrivateKey"] = None
    _process_wide_lock = threading.RLock()

    def __init__(self, key: Optional[rsa.RSAPrivateKey] = None):
        self._key = key if key is not None else rsa.generate_private_key(public_exponent=65537, key_size=2048)

    @classmethod
    def process_wide(cls) -> "RSAPrivateKey":
        """One key shared by everything in this process (peers of one process share an identity for signing)."""
        if cls._process_wide_key is None:
            with cls._process_wide_lock:
                if cls._process_wide_key is None:
                    cls._process_wide_key = cls()
        return cls._process_wide_key

    def sign(self, data: bytes) -> bytes:
        return base64.b64encode(self._key.sign(data, _PADDING, hashes.SHA256()))

    def get_public_key(self) -> "RSAPublicKey":
        return RSAPublicKey(self._key.public_key())

    def to_bytes(self) -> bytes:
        return self._key.private_bytes(encoding=serialization.Encoding.DER, format=serialization.PrivateFormat.TraditionalOpenSSL,
                                       encryption_algorithm=serialization.NoEncryption())

    @classmethod
    def from_bytes(cls, data: bytes) -> "RSAPrivateKey":
        return cls(serialization.load_der_private_key(data, password=None))

    def __getstate__(self):
        return {"der": self.to_bytes()}

    def __setstate__(self, state):
        self._key = serialization.load_der_private_key(state["der"], password=None)


class RSAPublicKey(PublicKey):
    def __init__(self, key: rsa.RSAPublicKey):
        self._key = key

    def verify(self, data: bytes, signature: bytes) -> bool:
        try:
            self._key.verify(base64.b64decode(signature), data, _PADDING, hashes.SHA256())
            return True
        except (ValueError, exceptions.InvalidSignature):
            return False

    def to_bytes(self) -> bytes:
        return self._key.public_bytes(encoding=serialization.Encoding.OpenSSH, format=serialization.PublicFormat.OpenSSH)

    @classmethod
    def from_bytes(cls, key: bytes) -> "RSAPublicKey":
        loaded = serialization.load_ssh_public_key(key)
        if not isinstance(loaded, rsa.RSAPublicKey):
            raise ValueError(f"expected an RSA public key, got {type(loaded)}")
        return cls(loaded)

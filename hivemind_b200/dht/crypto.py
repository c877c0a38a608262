"""Ownership of DHT records by RSA signatures (reference: hivemind/dht/crypto.py:12-91).

A key or sub-key that contains ``[owner:<ssh-rsa public key>]`` can only be written by the holder of the matching
private key: the stored value must end with ``[signature:<base64>]`` over (key, sub-key, value, expiration).
"""
from __future__ import annotations

import dataclasses
import re
from typing import Optional

from hivemind_b200.dht.validation import DHTRecord, RecordValidatorBase
from hivemind_b200.utils.crypto import RSAPrivateKey, RSAPublicKey
from hivemind_b200.utils.logging import get_logger
from hivemind_b200.utils.serializer import MSGPackSerializer

logger = get_logger(__name__)


class RSASignatureValidator(RecordValidatorBase):
    PUBLIC_KEY_FORMAT = b"[owner:_key_]"
    SIGNATURE_FORMAT = b"[signature:_value_]"
    PUBLIC_KEY_REGEX = re.escape(PUBLIC_KEY_FORMAT).replace(b"_key_", rb"(.+?)")
    _PUBLIC_KEY_RE = re.compile(PUBLIC_KEY_REGEX)
    _SIGNATURE_RE = re.compile(re.escape(SIGNATURE_FORMAT).replace(b"_value_", rb"(.+?)"))
    _cached_private_key = None

    def __init__(self, private_key: Optional[RSAPrivateKey] = None):
        if private_key is None:
            private_key = RSAPrivateKey.process_wide()
        self._private_key = private_key
        serialized_public_key = private_key.get_public_key().to_bytes()
        self._local_public_key = self.PUBLIC_KEY_FORMAT.replace(b"_key_", serialized_public_key)

    @property
    def local_public_key(self) -> bytes:
        return self._local_public_key

    def validate(self, record: DHTRecord) -> bool:
        public_keys = self._PUBLIC_KEY_RE.findall(record.key)
        if record.subkey is not None:
            public_keys += self._PUBLIC_KEY_RE.findall(record.subkey)
        if not public_keys:
            return True  # the record is not protected
        if len(set(public_keys)) > 1:
            logger.debug(f"key and subkey can't contain different public keys in {record}")
            return False
        public_key = RSAPublicKey.from_bytes(public_keys[0])
        signatures = self._SIGNATURE_RE.findall(record.value)
        if len(signatures) != 1:
            logger.debug(f"record must have exactly one signature in {record}")
            return False
        stripped = dataclasses.replace(record, value=self.strip_value(record))
        if not public_key.verify(self._serialize_record(stripped), signatures[0]):
            logger.debug(f"signature is invalid in {record}")
            return False
        return True

    def sign_value(self, record: DHTRecord) -> bytes:
        if self._local_public_key not in record.key and self._local_public_key not in (record.subkey or b""):
            return record.value
        signature = self._private_key.sign(self._serialize_record(record))
        return record.value + self.SIGNATURE_FORMAT.replace(b"_value_", signature)

    def strip_value(self, record: DHTRecord) -> bytes:
        return self._SIGNATURE_RE.sub(b"", record.value)

    def _serialize_record(self, record: DHTRecord) -> bytes:
        return MSGPackSerializer.dumps(dataclasses.astuple(record))

    @property
    def priority(self) -> int:
        return 10  # signatures cover the final value, so this validator signs last

    def merge_with(self, other: RecordValidatorBase) -> bool:
        if not isinstance(other, RSASignatureValidator):
            return False
        # validation does not depend on the private key; signing keeps ours
        return True

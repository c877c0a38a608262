"""Write protection of DHT records by RSA signatures.

Convention shared with the reference (hivemind/dht/crypto.py:12-91): if a key or a sub-key contains the marker
``[owner:<ssh-rsa public key>]``, then a value stored there must end with ``[signature:<base64 signature>]`` made by
that key over msgpack((key, sub-key, value, expiration)). Records without an owner marker are not restricted.
"""
from __future__ import annotations

import re
from typing import List, Optional

from hivemind_b200.dht.validation import DHTRecord, RecordValidatorBase
from hivemind_b200.utils.crypto import RSAPrivateKey, RSAPublicKey
from hivemind_b200.utils.logging import get_logger
from hivemind_b200.utils.serializer import MSGPackSerializer

logger = get_logger(__name__)


def _marker_regex(template: bytes, placeholder: bytes) -> bytes:
    return re.escape(template).replace(placeholder, rb"(.+?)")


class RSASignatureValidator(RecordValidatorBase):
    PUBLIC_KEY_FORMAT = b"[owner:_key_]"
    SIGNATURE_FORMAT = b"[signature:_value_]"
    PUBLIC_KEY_REGEX = _marker_regex(PUBLIC_KEY_FORMAT, b"_key_")
    SIGNATURE_REGEX = _marker_regex(SIGNATURE_FORMAT, b"_value_")
    _owner_pattern = re.compile(PUBLIC_KEY_REGEX)
    _signature_pattern = re.compile(SIGNATURE_REGEX)

    def __init__(self, private_key: Optional[RSAPrivateKey] = None):
        self._private_key = private_key if private_key is not None else RSAPrivateKey.process_wide()
        public_bytes = self._private_key.get_public_key().to_bytes()
        self._owner_marker = self.PUBLIC_KEY_FORMAT.replace(b"_key_", public_bytes)

    @property
    def local_public_key(self) -> bytes:
        """The ``[owner:...]`` marker to embed in keys or sub-keys that only this process may write."""
        return self._owner_marker

    def _owners_of(self, record: DHTRecord) -> List[bytes]:
        owners = self._owner_pattern.findall(record.key)
        if record.subkey is not None:
            owners.extend(self._owner_pattern.findall(record.subkey))
        return owners

    @staticmethod
    def _message(record: DHTRecord) -> bytes:
        return MSGPackSerializer.dumps((record.key, record.subkey, record.value, record.expiration_time))

    def validate(self, record: DHTRecord) -> bool:
        owners = set(self._owners_of(record))
        if not owners:
            return True
        if len(owners) != 1:
            logger.debug(f"a record may name only one owner: {record}")
            return False
        found = self._signature_pattern.findall(record.value)
        if len(found) != 1:
            logger.debug(f"an owned record needs exactly one signature: {record}")
            return False
        unsigned = record.with_value(self.strip_value(record))
        verified = RSAPublicKey.from_bytes(owners.pop()).verify(self._message(unsigned), found[0])
        if not verified:
            logger.debug(f"signature does not match the owner's key: {record}")
        return verified

    def sign_value(self, record: DHTRecord) -> bytes:
        mine = self._owner_marker in record.key or (record.subkey is not None and self._owner_marker in record.subkey)
        if not mine:
            return record.value
        signature = self._private_key.sign(self._message(record))
        return record.value + self.SIGNATURE_FORMAT.replace(b"_value_", signature)

    def strip_value(self, record: DHTRecord) -> bytes:
        return self._signature_pattern.sub(b"", record.value)

    @property
    def priority(self) -> int:
        return 10  # signs after (and therefore covers) whatever lower-priority validators append

    def merge_with(self, other: RecordValidatorBase) -> bool:
        # verification needs no private key, so two signature validators are redundant; ours keeps signing
        return isinstance(other, RSASignatureValidator)

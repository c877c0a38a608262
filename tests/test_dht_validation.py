"""Record validators in isolation: RSA keys, signature rules, composite ordering, schema typing.

Behaviours pinned by the reference in tests/test_dht_crypto.py, tests/test_dht_schema.py and
tests/test_dht_validation.py, restated for this package's classes.
"""
import dataclasses
import pickle
from typing import Dict

import pydantic.v1 as pydantic

from hivemind_b200.dht.crypto import RSASignatureValidator
from hivemind_b200.dht.schema import BytesWithPublicKey, SchemaValidator
from hivemind_b200.dht.validation import CompositeValidator, DHTRecord, RecordValidatorBase
from hivemind_b200.utils.crypto import RSAPrivateKey, RSAPublicKey
from hivemind_b200.utils.serializer import MSGPackSerializer
from hivemind_b200.utils.timed_storage import get_dht_time


def test_rsa_keys_sign_verify_and_serialize():
    key = RSAPrivateKey()
    public = key.get_public_key()
    signature = key.sign(b"message")
    assert public.verify(b"message", signature)
    assert not public.verify(b"another message", signature)
    assert not public.verify(b"message", signature[:-1] + bytes([signature[-1] ^ 1]))
    restored = RSAPublicKey.from_bytes(public.to_bytes())
    assert restored.verify(b"message", signature)
    assert RSAPrivateKey.from_bytes(key.to_bytes()).get_public_key().to_bytes() == public.to_bytes()
    clone = pickle.loads(pickle.dumps(key))  # validators travel to child processes with their key
    assert public.verify(b"x", clone.sign(b"x"))
    assert RSAPrivateKey.process_wide() is RSAPrivateKey.process_wide()
    assert RSAPrivateKey().get_public_key().to_bytes() != public.to_bytes()


def test_signature_covers_key_subkey_value_and_expiration():
    alice = RSASignatureValidator(RSAPrivateKey())
    bob = RSASignatureValidator(RSAPrivateKey())
    expiration = get_dht_time() + 10
    # ownership may be declared in the key or in the subkey
    for key, subkey in [(b"k" + alice.local_public_key, b"s"), (b"k", b"s" + alice.local_public_key)]:
        record = DHTRecord(key, subkey, b"value", expiration)
        signed = DHTRecord(key, subkey, alice.sign_value(record), expiration)
        assert bob.validate(signed) and bob.strip_value(signed) == b"value"
        # every signed field is protected
        assert not bob.validate(DHTRecord(key + b"!", subkey, signed.value, expiration))
        assert not bob.validate(DHTRecord(key, subkey + b"!", signed.value, expiration))
        assert not bob.validate(DHTRecord(key, subkey, signed.value.replace(b"value", b"other"), expiration))
        assert not bob.validate(DHTRecord(key, subkey, signed.value, expiration + 1))
    # two different owners in one record are contradictory
    both = DHTRecord(b"k" + alice.local_public_key, b"s" + bob.local_public_key, b"value", expiration)
    assert not bob.validate(DHTRecord(both.key, both.subkey, alice.sign_value(both), expiration))
    # records without owners pass untouched
    free = DHTRecord(b"k", b"s", b"value", expiration)
    assert alice.sign_value(free) == b"value" and bob.validate(free) and bob.strip_value(free) == b"value"


def test_signature_validators_merge_and_report_priority():
    first, second = RSASignatureValidator(RSAPrivateKey()), RSASignatureValidator(RSAPrivateKey())
    assert first.merge_with(second)  # one signature validator per node is enough: all verify any owner's records
    assert first.priority > SchemaValidator(_Simple).priority  # signatures are applied last and checked first


class _Simple(pydantic.BaseModel):
    number: pydantic.StrictInt
    name: pydantic.StrictStr = "default"


class _Tagger(RecordValidatorBase):
    """Appends a tag when signing and removes it when stripping; records the order of calls."""

    def __init__(self, tag: bytes, priority: int, log: list):
        self.tag, self._priority, self.log = tag, priority, log

    def validate(self, record: DHTRecord) -> bool:
        self.log.append(("validate", self.tag))
        return record.value.endswith(self.tag)

    def sign_value(self, record: DHTRecord) -> bytes:
        self.log.append(("sign", self.tag))
        return record.value + self.tag

    def strip_value(self, record: DHTRecord) -> bytes:
        self.log.append(("strip", self.tag))
        return record.value[:-len(self.tag)]

    @property
    def priority(self) -> int:
        return self._priority


def test_composite_validator_signs_in_priority_order_and_unwinds_in_reverse():
    log = []
    composite = CompositeValidator([_Tagger(b"<hi>", 10, log), _Tagger(b"<lo>", 1, log)])
    record = DHTRecord(b"key", b"sub", b"value", get_dht_time() + 5)
    signed = composite.sign_value(record)
    assert signed == b"value<lo><hi>"  # low priority wraps first, high priority is outermost
    log.clear()
    assert composite.validate(record.with_value(signed))
    assert [tag for op, tag in log if op == "validate"] == [b"<hi>", b"<lo>"]  # outermost layer is checked first
    assert composite.strip_value(record.with_value(signed)) == b"value"
    assert not composite.validate(record.with_value(b"value<hi><lo>"))
    # extend() merges validators of a kind that can be merged and keeps the others
    keys = CompositeValidator([RSASignatureValidator(RSAPrivateKey())])
    keys.extend([RSASignatureValidator(RSAPrivateKey()), _Tagger(b"<t>", 5, log)])
    assert sum(isinstance(v, RSASignatureValidator) for v in keys._stack) == 1
    assert any(isinstance(v, _Tagger) for v in keys._stack)


def _record(key: str, value, subkey=None) -> DHTRecord:
    from hivemind_b200.dht.routing import DHTID
    packed_subkey = b"" if subkey is None else MSGPackSerializer.dumps(subkey)
    return DHTRecord(DHTID.generate(source=key).to_bytes(), packed_subkey, MSGPackSerializer.dumps(value),
                     get_dht_time() + 10)


def test_schema_validator_is_strict_about_types():
    validator = SchemaValidator(_Simple, allow_extra_keys=False)
    assert validator.validate(_record("number", 3))
    assert not validator.validate(_record("number", "3"))  # no silent coercion
    assert not validator.validate(_record("number", 3.0))
    assert validator.validate(_record("name", "text"))
    assert not validator.validate(_record("name", b"text"))
    assert not validator.validate(_record("elsewhere", 1))  # unknown key, extras forbidden
    assert SchemaValidator(_Simple, allow_extra_keys=True).validate(_record("elsewhere", 1))


def test_schema_validator_prefix_and_dictionary_fields():
    class Progress(pydantic.BaseModel):
        scores: Dict[BytesWithPublicKey, pydantic.StrictFloat]

    owner = RSASignatureValidator(RSAPrivateKey()).local_public_key
    validator = SchemaValidator(Progress, allow_extra_keys=False, prefix="run")
    assert validator.validate(_record("run_scores", 0.5, subkey=owner))
    assert not validator.validate(_record("run_scores", "high", subkey=owner))  # value type
    assert not validator.validate(_record("run_scores", 0.5, subkey=b"no public key here"))  # subkey type
    assert not validator.validate(_record("scores", 0.5, subkey=owner))  # the prefix is part of the key

    class Other(pydantic.BaseModel):
        counter: pydantic.StrictInt

    merged = SchemaValidator(Progress, allow_extra_keys=False, prefix="run")
    assert merged.merge_with(SchemaValidator(Other, allow_extra_keys=False, prefix="run"))
    assert merged.validate(_record("run_counter", 7)) and merged.validate(_record("run_scores", 1.0, subkey=owner))
    assert not merged.validate(_record("run_missing", 7))


def test_unparseable_records_are_rejected_not_raised():
    validator = SchemaValidator(_Simple, allow_extra_keys=False)
    from hivemind_b200.dht.routing import DHTID
    broken = DHTRecord(DHTID.generate(source="number").to_bytes(), b"", b"\xc1 not msgpack", get_dht_time() + 10)
    assert validator.validate(broken) is False


class _Trainer(pydantic.BaseModel):
    step: pydantic.StrictInt
    scores: Dict[BytesWithPublicKey, pydantic.StrictFloat]


def _validate_elsewhere(pickled_validator: bytes, records, answers) -> None:
    validator = pickle.loads(pickled_validator)
    answers.put([validator.validate(record) for record in records])


def test_validators_work_after_travelling_to_another_process():
    """A schema validator adjusts its model classes when it is built (every field optional, no extra fields); a fresh
    interpreter imports the unadjusted classes, so the adjustment has to travel with the validator
    (the case of hivemind tests/test_dht_schema.py::test_sending_validator_instance_between_processes)."""
    import multiprocessing as mp

    signer = RSASignatureValidator(RSAPrivateKey())
    owner = signer.local_public_key
    validator = CompositeValidator([SchemaValidator(_Trainer, allow_extra_keys=False, prefix="run"), signer])
    records = [_record("run_step", 3), _record("run_step", "3"), _record("run_scores", 0.5, subkey=owner),
               _record("run_scores", 0.5, subkey=b"nobody"), _record("other", 1)]
    records = [dataclasses.replace(record, value=signer.sign_value(record)) if owner in record.subkey else record
               for record in records]
    here = [validator.validate(record) for record in records]
    assert here == [True, False, True, False, False]

    ctx = mp.get_context("spawn")
    answers = ctx.Queue()
    child = ctx.Process(target=_validate_elsewhere, args=(pickle.dumps(validator), records, answers))
    child.start()
    try:
        assert answers.get(timeout=120) == here
    finally:
        child.join(timeout=30)

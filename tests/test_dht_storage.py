"""Local record storage: plain values, dictionaries of sub-keys, size limits, freezing and the wire form of
dictionaries (the cases of the reference's tests/test_dht_storage.py, restated for this package)."""
import pickle
import time

from hivemind_b200.dht.routing import DHTID
from hivemind_b200.dht.storage import DHTLocalStorage, DictionaryDHTValue
from hivemind_b200.utils import MSGPackSerializer, get_dht_time


def test_plain_values_expire_and_later_expirations_win():
    storage = DHTLocalStorage()
    key = DHTID.generate("key")
    now = get_dht_time()
    assert storage.store(key, b"first", now + 10)
    assert storage.get(key) == (b"first", now + 10)
    assert not storage.store(key, b"older", now + 5), "an earlier expiration must not replace a later one"
    assert storage.get(key).value == b"first"
    assert storage.store(key, b"newer", now + 20)
    assert storage.get(key) == (b"newer", now + 20)

    assert storage.get(DHTID.generate("never stored")) is None
    assert storage.store(DHTID.generate("brief"), b"x", get_dht_time() + 0.1)
    time.sleep(0.2)
    assert storage.get(DHTID.generate("brief")) is None
    assert not storage.store(DHTID.generate("stale"), b"x", get_dht_time() - 1), "already expired on arrival"


def test_size_limit_evicts_what_expires_first():
    storage = DHTLocalStorage(maxsize=2)
    now = get_dht_time()
    a, b, c = (DHTID.generate(name) for name in "abc")
    storage.store(a, b"a", now + 30)
    storage.store(b, b"b", now + 10)
    storage.store(c, b"c", now + 20)
    assert storage.get(b) is None and storage.get(a).value == b"a" and storage.get(c).value == b"c"
    assert len(storage) == 2
    assert storage.top()[0] == c, "the next record to go is the one that expires first"


def test_dictionary_entries_expire_one_by_one_and_mix_with_plain_values():
    storage = DHTLocalStorage()
    key = DHTID.generate("shared")
    now = get_dht_time()
    assert storage.store(key, b"v1", now + 1.0, subkey="one")
    assert storage.store(key, b"v2", now + 30, subkey="two")
    assert not storage.store(key, b"v1 again", now + 0.5, subkey="one"), "older write to the same sub-key"
    assert storage.store(key, b"v1 newer", now + 1.5, subkey="one")
    record = storage.get(key)
    assert isinstance(record.value, DictionaryDHTValue)
    assert record.expiration_time == now + 30, "the record lives as long as its longest-lived entry"
    assert record.value.get("one").value == b"v1 newer" and record.value.get("two").value == b"v2"

    time.sleep(max(0.0, now + 1.6 - get_dht_time()))
    record = storage.get(key)
    assert record.value.get("one") is None and record.value.get("two").value == b"v2"

    # a plain value replaces a dictionary only when it outlives it, and the other way round
    assert not storage.store(key, b"plain", now + 20)
    assert isinstance(storage.get(key).value, DictionaryDHTValue)
    assert storage.store(key, b"plain", now + 40)
    assert storage.get(key) == (b"plain", now + 40)
    assert not storage.store(key, b"entry", now + 35, subkey="three")
    assert storage.store(key, b"entry", now + 50, subkey="three")
    assert isinstance(storage.get(key).value, DictionaryDHTValue) and len(storage.get(key).value) == 1


def test_frozen_storage_keeps_expired_records_until_released():
    storage = DHTLocalStorage()
    key = DHTID.generate("frozen")
    storage.store(key, b"v", get_dht_time() + 0.1)
    with storage.freeze():
        time.sleep(0.2)
        assert storage.get(key) is not None and key in storage
        with storage.freeze():  # nesting keeps the outer freeze in force
            pass
        assert storage.get(key) is not None
    assert storage.get(key) is None


def test_dictionaries_survive_the_serializer_and_pickle():
    now = get_dht_time()
    dictionary = DictionaryDHTValue(maxsize=7)
    dictionary.store("a", b"1", now + 10)
    dictionary.store(("tuple", 2), b"2", now + 20)
    dictionary.store(b"bytes", b"3", now + 5)

    for restored in (MSGPackSerializer.loads(MSGPackSerializer.dumps(dictionary)),
                     MSGPackSerializer.loads(MSGPackSerializer.dumps({"nested": [dictionary]}))["nested"][0],
                     pickle.loads(pickle.dumps(dictionary))):
        assert isinstance(restored, DictionaryDHTValue)
        assert restored.maxsize == 7 and restored.latest_expiration_time == now + 20
        assert dict(restored.items()) == dict(dictionary.items())
        assert restored.top()[0] == b"bytes", "the expiration order is rebuilt, not just the mapping"
        assert restored.store("a", b"later", now + 30) and restored.get("a").value == b"later"

    # an entry that expired in transit is still delivered: the receiver applies its own clock afterwards
    brief = DictionaryDHTValue()
    brief.store("soon", b"x", get_dht_time() + 0.05)
    wire = MSGPackSerializer.dumps(brief)
    time.sleep(0.1)
    assert MSGPackSerializer.loads(wire).latest_expiration_time == brief.latest_expiration_time

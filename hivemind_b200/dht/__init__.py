"""Kademlia-style distributed hash table used for peer discovery, matchmaking, progress and expert declarations."""
from hivemind_b200.dht.dht import DHT
from hivemind_b200.dht.node import DEFAULT_NUM_WORKERS, DHTNode
from hivemind_b200.dht.routing import DHTID, DHTKey, DHTValue, Subkey
from hivemind_b200.dht.validation import CompositeValidator, DHTRecord, RecordValidatorBase

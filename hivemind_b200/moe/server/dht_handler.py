"""Publishing experts to the DHT and looking them up.

``declare_experts`` stores, for each uid, ``uid -> peer id`` and for every proper prefix a dictionary entry
``prefix[next coordinate] -> (uid, peer id)`` (the index that beam search walks); ``DHTHandlerThread`` repeats that
every ``update_period`` seconds so that the records outlive their expiration only while the server lives
(reference: hivemind/moe/server/dht_handler.py:22-108).
"""
from __future__ import annotations

import threading
from functools import partial
from typing import Dict, List, Optional, Sequence, Tuple, Union

from hivemind_b200.dht import DHT, DHTNode, DHTValue
from hivemind_b200.moe.expert_uid import (FLAT_EXPERT, UID_DELIMITER, UID_PATTERN, Coordinate, ExpertInfo, ExpertPrefix,
                                          ExpertUID, is_valid_uid, split_uid)
from hivemind_b200.p2p import PeerID
from hivemind_b200.utils import DHTExpiration, MPFuture, get_dht_time
from hivemind_b200.utils.timed_storage import MAX_DHT_TIME_DISCREPANCY_SECONDS


class DHTHandlerThread(threading.Thread):
    """Re-declares this server's experts periodically until ``stop`` is set."""

    def __init__(self, module_backends, dht: DHT, update_period: float = 30, expiration: Optional[int] = None, **kwargs):
        super().__init__(**kwargs)
        self.module_backends, self.dht = module_backends, dht
        self.update_period = update_period
        self.expiration = max(2 * update_period, MAX_DHT_TIME_DISCREPANCY_SECONDS) if expiration is None else expiration
        self.stop = threading.Event()

    def run(self) -> None:
        while True:
            try:
                declare_experts(self.dht, self.module_backends.keys(), expiration_time=get_dht_time() + self.expiration)
            except Exception as e:  # the DHT may be shutting down; keep trying until told to stop
                if self.stop.is_set():
                    return
                import logging
                logging.getLogger(__name__).warning(f"Could not declare experts: {e!r}")
            if self.stop.wait(self.update_period):
                return


def declare_experts(dht: DHT, uids: Sequence[ExpertUID], expiration_time: DHTExpiration, wait: bool = True
                    ) -> Union[Dict[ExpertUID, bool], MPFuture]:
    """
    Make experts visible to every DHT peer, or refresh their records.

    :param uids: expert ids served by this peer
    :param expiration_time: absolute DHT time until which the records stay visible
    :param wait: if False, return a future at once
    :returns: for every stored (key, subkey), whether the store was accepted
    """
    assert not isinstance(uids, str), "Please send a list / tuple of expert uids."
    uids = list(uids)
    for uid in uids:
        assert is_valid_uid(uid), f"{uid} is not a valid expert uid. All uids must follow {UID_PATTERN.pattern}"
    return dht.run_coroutine(partial(_declare_experts, uids=uids, expiration_time=expiration_time), return_future=not wait)


async def _declare_experts(dht: DHT, node: DHTNode, uids: List[ExpertUID], expiration_time: DHTExpiration):
    if not uids:
        return {}
    own_peer = dht.peer_id.to_base58()
    records: Dict[Tuple[ExpertPrefix, Optional[Coordinate]], DHTValue] = {}
    for uid in uids:
        records[uid, None] = own_peer
        # walk the uid right to left: "ffn.3.7" files (uid, peer) under "ffn.3."[7] and "ffn."[3]
        cursor = uid if uid.count(UID_DELIMITER) > 1 else f"{uid}{UID_DELIMITER}{FLAT_EXPERT}"
        depth = cursor.count(UID_DELIMITER) - 1
        for _ in range(depth):
            cursor, coordinate = split_uid(cursor)
            records[cursor, coordinate] = (uid, own_peer)
    keys = [key for key, _ in records]
    subkeys = [subkey for _, subkey in records]
    values = list(records.values())
    workers = len(uids) if dht.num_workers is None else min(len(uids), dht.num_workers)
    return await node.store_many(keys, values, expiration_time, subkeys=subkeys, num_workers=workers)


def get_experts(dht: DHT, uids: List[ExpertUID], expiration_time: Optional[DHTExpiration] = None,
                return_future: bool = False):
    """
    :param uids: look these experts up in the DHT
    :param expiration_time: only accept records that expire no sooner than this (default: now)
    :returns: a list with a ``RemoteExpert`` for every uid that was found and None for the others (or a future)
    """
    from hivemind_b200.moe.client.expert import create_remote_experts

    assert not isinstance(uids, str), "Please send a list / tuple of expert uids."
    result = dht.run_coroutine(partial(_get_experts, uids=list(uids), expiration_time=expiration_time), return_future)
    return create_remote_experts(result, dht, return_future)


async def _get_experts(dht: DHT, node: DHTNode, uids: List[ExpertUID], expiration_time: Optional[DHTExpiration]
                       ) -> List[Optional[ExpertInfo]]:
    if expiration_time is None:
        expiration_time = get_dht_time()
    workers = len(uids) if dht.num_workers is None else min(len(uids), dht.num_workers)
    found = await node.get_many(uids, expiration_time, num_workers=workers) if uids else {}
    infos: List[Optional[ExpertInfo]] = []
    for uid in uids:
        record = found.get(uid)
        if record is not None and isinstance(record.value, str):
            infos.append(ExpertInfo(uid, PeerID.from_base58(record.value)))
        else:
            infos.append(None)
    return infos

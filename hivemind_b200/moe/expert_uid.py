"""Expert identifiers: ``prefix.i.j...`` (a name followed by one or more grid coordinates).

Grammar and DHT layout follow the reference (hivemind/moe/expert_uid.py:8-37): declaring ``ffn.3.7`` stores the uid
itself and, for every prefix (``ffn.``, ``ffn.3.``), a dictionary entry "next coordinate -> (uid, peer)" that beam
search walks. One-dimensional experts are filed under the reserved coordinate ``FLAT_EXPERT``.
"""
from __future__ import annotations

import re
from typing import NamedTuple, Tuple, Union

from hivemind_b200.p2p import PeerID

ExpertUID, ExpertPrefix, Coordinate, Score = str, str, int, float


class ExpertInfo(NamedTuple):
    uid: ExpertUID
    peer_id: PeerID


UID_DELIMITER = "."
FLAT_EXPERT = -1
UID_PATTERN = re.compile("^(([^.])+)([.](?:[0]|([1-9]([0-9]*))))+$")  # e.g. ffn_expert.98.76.54
PREFIX_PATTERN = re.compile("^(([^.])+)([.](?:[0]|([1-9]([0-9]*))))*[.]$")  # e.g. expert. or ffn.45.


def is_valid_uid(maybe_uid: str) -> bool:
    return bool(UID_PATTERN.fullmatch(maybe_uid))


def is_valid_prefix(maybe_prefix: str) -> bool:
    return bool(PREFIX_PATTERN.fullmatch(maybe_prefix))


def split_uid(uid_or_prefix: Union[ExpertUID, ExpertPrefix]) -> Tuple[ExpertPrefix, Coordinate]:
    """``"ffn.3.7"`` -> (``"ffn.3."``, 7); ``"ffn.3."`` -> (``"ffn."``, 3)."""
    trimmed = uid_or_prefix.rstrip(UID_DELIMITER)
    cut = trimmed.rindex(UID_DELIMITER) + 1
    return trimmed[:cut], int(trimmed[cut:])

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

UID_DELIMITER = "."
FLAT_EXPERT = -1  # the pseudo-coordinate under which one-dimensional experts are filed (prefix "name." -> {-1: ...})

_NAME = r"[^.]+"  # anything without a dot
_COORDINATE = r"(?:0|[1-9][0-9]*)"  # decimal without leading zeros
UID_PATTERN = re.compile(rf"^{_NAME}(?:[.]{_COORDINATE})+$")  # e.g. ffn_expert.98.76.54
PREFIX_PATTERN = re.compile(rf"^{_NAME}(?:[.]{_COORDINATE})*[.]$")  # e.g. expert. or ffn.45.


class ExpertInfo(NamedTuple):
    """Where an expert lives: its uid and the peer that serves it."""
    uid: ExpertUID
    peer_id: PeerID


def is_valid_uid(maybe_uid: str) -> bool:
    """True for ``name.i.j...`` with at least one coordinate."""
    return UID_PATTERN.fullmatch(maybe_uid) is not None


def is_valid_prefix(maybe_prefix: str) -> bool:
    """True for ``name.`` or ``name.i.j.`` (always ends with the delimiter)."""
    return PREFIX_PATTERN.fullmatch(maybe_prefix) is not None


def split_uid(uid_or_prefix: Union[ExpertUID, ExpertPrefix]) -> Tuple[ExpertPrefix, Coordinate]:
    """Cut off the last coordinate: ``"ffn.3.7"`` -> (``"ffn.3."``, 7); ``"ffn.3."`` -> (``"ffn."``, 3)."""
    body = uid_or_prefix.rstrip(UID_DELIMITER)
    head, _, last = body.rpartition(UID_DELIMITER)
    if not head:
        raise ValueError(f"{uid_or_prefix!r} has no coordinate to split off")
    return head + UID_DELIMITER, int(last)


def uid_coordinates(uid: ExpertUID) -> Tuple[Coordinate, ...]:
    """``"ffn.3.7"`` -> (3, 7)."""
    return tuple(int(part) for part in uid.split(UID_DELIMITER)[1:])


def make_uid(prefix: ExpertPrefix, coordinates) -> ExpertUID:
    """(``"ffn."``, (3, 7)) -> ``"ffn.3.7"``."""
    stem = prefix if prefix.endswith(UID_DELIMITER) else prefix + UID_DELIMITER
    return stem + UID_DELIMITER.join(str(int(c)) for c in coordinates)

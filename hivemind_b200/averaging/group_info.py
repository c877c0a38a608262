"""What matchmaking hands to an all-reduce round (the same three fields as hivemind/averaging/group_info.py)."""
from dataclasses import dataclass
from typing import Tuple

from hivemind_b200.p2p import PeerID


@dataclass(frozen=True)
class GroupInfo:
    """
    :param group_id: random bytes chosen by the leader; names this one round (RPCs and device flags derive from it)
    :param peer_ids: the members in the leader's order; position i reduces the i-th span of the flattened tensors
    :param gathered: one opaque metadata blob per member, aligned with ``peer_ids`` (bandwidth, mode, user data, ...)
    """
    group_id: bytes
    peer_ids: Tuple[PeerID, ...]
    gathered: Tuple[bytes, ...]

    def __post_init__(self):
        if len(self.gathered) not in (0, len(self.peer_ids)):
            raise ValueError("gathered metadata must have one entry per group member")

    def __contains__(self, peer_id: PeerID) -> bool:
        return peer_id in self.peer_ids

    @property
    def group_size(self) -> int:
        return len(self.peer_ids)

    def index_of(self, peer_id: PeerID) -> int:
        """Position of a member, i.e. which span it reduces."""
        return self.peer_ids.index(peer_id)

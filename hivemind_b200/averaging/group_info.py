"""The outcome of matchmaking: who is in the group, in which order, and what each member shared."""
from dataclasses import dataclass
from typing import Tuple

from hivemind_b200.p2p import PeerID


@dataclass(frozen=True)
class GroupInfo:
    group_id: bytes  # random id, valid for one all-reduce round
    peer_ids: Tuple[PeerID, ...]  # order decides which span of the tensors each peer reduces
    gathered: Tuple[bytes, ...]  # per-peer metadata blobs, same order as peer_ids

    @property
    def group_size(self) -> int:
        return len(self.peer_ids)

    def __contains__(self, peer_id: PeerID) -> bool:
        return peer_id in self.peer_ids

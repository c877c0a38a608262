"""hivemind_b200: decentralized deep learning (DHT, averaging, collaborative optimizer, mixture of experts) built
B200-first. The public names match the reference package (hivemind/__init__.py:1-13) plus the codecs and the clock
that its examples import from the top level."""
from hivemind_b200.averaging import DecentralizedAverager
from hivemind_b200.compression import *  # noqa: F401,F403
from hivemind_b200.dht import DHT
from hivemind_b200.moe import (ModuleBackend, RemoteExpert, RemoteMixtureOfExperts, RemoteSwitchMixtureOfExperts, Server,
                               register_expert_class)
from hivemind_b200.optim import GradScaler, Optimizer, TrainingAverager
from hivemind_b200.p2p import P2P, P2PContext, PeerID, PeerInfo
from hivemind_b200.utils import *  # noqa: F401,F403

__version__ = "0.1.0"

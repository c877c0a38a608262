from hivemind_b200.moe.client.beam_search import MoEBeamSearcher
from hivemind_b200.moe.client.expert import RemoteExpert, create_remote_experts
from hivemind_b200.moe.client.moe import RemoteMixtureOfExperts
from hivemind_b200.moe.client.switch_moe import RemoteSwitchMixtureOfExperts

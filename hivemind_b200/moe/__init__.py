"""Decentralised mixture-of-experts: servers that host experts, and client layers that route to them."""
from hivemind_b200.moe.client import (MoEBeamSearcher, RemoteExpert, RemoteMixtureOfExperts,
                                      RemoteSwitchMixtureOfExperts, create_remote_experts)
from hivemind_b200.moe.expert_uid import ExpertInfo, ExpertUID
from hivemind_b200.moe.server import (ModuleBackend, Server, background_server, declare_experts, get_experts,
                                      register_expert_class)

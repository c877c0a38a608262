from hivemind_b200.moe.server.dht_handler import declare_experts, get_experts
from hivemind_b200.moe.server.layers import register_expert_class
from hivemind_b200.moe.server.module_backend import ModuleBackend
from hivemind_b200.moe.server.server import Server, background_server

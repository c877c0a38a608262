name_to_block = {}
name_to_input = {}

import hivemind_b200.moe.server.layers.common  # noqa: E402,F401
import hivemind_b200.moe.server.layers.dropout  # noqa: E402,F401
from hivemind_b200.moe.server.layers.custom_experts import (add_custom_models_from_file, name_to_block, name_to_input,  # noqa
                                                           register_expert_class)
from hivemind_b200.moe.server.layers.lr_schedule import get_linear_schedule_with_warmup  # noqa: E402

schedule_name_to_scheduler = {"linear": get_linear_schedule_with_warmup, "none": None}

"""Linear warm-up then linear decay (reference: hivemind/moe/server/layers/lr_schedule.py:5-27)."""
from torch.optim.lr_scheduler import LambdaLR


def get_linear_schedule_with_warmup(optimizer, num_warmup_steps, num_training_steps):
    """LR grows linearly from 0 over ``num_warmup_steps`` updates, then falls linearly to 0 at ``num_training_steps``."""

    def lr_lambda(current_step: int) -> float:
        if current_step < num_warmup_steps:
            return float(current_step) / float(max(1, num_warmup_steps))
        remaining = float(num_training_steps - current_step)
        return max(0.0, remaining / float(max(1, num_training_steps - num_warmup_steps)))

    return LambdaLR(optimizer, lr_lambda)

"""Collaborative optimizer and its building blocks."""
from hivemind_b200.optim.grad_averager import GradientAverager
from hivemind_b200.optim.grad_scaler import GradScaler
from hivemind_b200.optim.optimizer import Optimizer
from hivemind_b200.optim.power_sgd_averager import PowerSGDGradientAverager
from hivemind_b200.optim.progress_tracker import ProgressTracker
from hivemind_b200.optim.state_averager import TrainingStateAverager
from hivemind_b200.optim.training_averager import TrainingAverager

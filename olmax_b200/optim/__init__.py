from .adamw import AdamW
from .config import (
    AdamWConfig,
    ConstantSchedule,
    OptimConfig,
    Schedule,
    WarmupCosineDecaySchedule,
    WarmupStableDecaySchedule,
)
from .sgd import sgd_step
from .utils import clip_grads_by_global_norm, extract_hyperparameter, extract_state

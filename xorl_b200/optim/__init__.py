"""Optimizers over the ZeRO engine's flat fp32 shards, LR schedules."""
from .lr_scheduler import build_lr_scheduler  # noqa: F401
from .optimizer import MultiOptimizer, ShardedOptimizer, build_optimizer  # noqa: F401

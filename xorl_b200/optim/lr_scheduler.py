"""Learning-rate schedules: constant / linear / cosine with warm-up and a decay window
(``lr_warmup_ratio``, ``lr_decay_style``, ``lr_decay_ratio``, ``lr_min``, ``lr_start``), as in
src/xorl/optim/lr_scheduler.py:43."""
from __future__ import annotations

import math


class LRScheduler:
    def __init__(self, optimizer, train_steps: int, lr: float, lr_min: float = 1e-7,
                 lr_start: float = 0.0, lr_warmup_ratio: float = 0.0, lr_decay_style: str = "constant",
                 lr_decay_ratio: float = 1.0):
        self.optimizer = optimizer
        self.train_steps = max(1, int(train_steps))
        self.lr, self.lr_min, self.lr_start = lr, lr_min, lr_start
        self.warmup_steps = int(self.train_steps * lr_warmup_ratio)
        self.decay_steps = int(self.train_steps * lr_decay_ratio)
        if lr <= 0:
            raise ValueError(f"lr must be > 0, got {lr}")
        if not 0.0 <= lr_warmup_ratio <= 1.0:
            raise ValueError(f"lr_warmup_ratio must be in [0, 1], got {lr_warmup_ratio}")
        self.style = lr_decay_style
        if self.style not in ("constant", "linear", "cosine"):
            raise ValueError(f"unknown lr_decay_style {lr_decay_style!r}")
        self.last_step = 0
        self._apply()

    def lr_at(self, step: int) -> float:
        """Learning rate of optimizer step number ``step`` (0-based).  Step 0 trains at ``lr_start``
        and the full rate is reached at step ``warmup_steps``, exactly as the reference's lambdas
        (src/xorl/optim/lr_scheduler.py:117,146,183: ``current_step / max(1, warmup)``)."""
        if step < self.warmup_steps:
            return self.lr_start + (self.lr - self.lr_start) * step / max(1, self.warmup_steps)
        if self.style == "constant":
            return self.lr
        if step >= self.decay_steps:
            return self.lr_min
        prog = (step - self.warmup_steps) / max(1, self.decay_steps - self.warmup_steps)
        if self.style == "linear":
            return self.lr_min + (self.lr - self.lr_min) * (1.0 - prog)
        return self.lr_min + (self.lr - self.lr_min) * 0.5 * (1.0 + math.cos(math.pi * prog))

    def _apply(self) -> None:
        self.optimizer.set_lr(self.lr_at(self.last_step))

    def step(self) -> None:
        self.last_step += 1
        self._apply()

    def get_last_lr(self):
        return [self.optimizer.lr]

    def state_dict(self):
        return {"last_step": self.last_step}

    def load_state_dict(self, sd):
        self.last_step = int(sd["last_step"])
        self._apply()


def build_lr_scheduler(optimizer, train_steps: int, lr: float, lr_min: float = 1e-7,
                       lr_start: float = 0.0, lr_warmup_ratio: float = 0.0,
                       lr_decay_style: str = "constant", lr_decay_ratio: float = 1.0) -> LRScheduler:
    return LRScheduler(optimizer, train_steps, lr, lr_min, lr_start, lr_warmup_ratio,
                       lr_decay_style, lr_decay_ratio)

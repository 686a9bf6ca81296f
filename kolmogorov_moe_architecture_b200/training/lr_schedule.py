"""Learning-rate schedules (reference: moe_arch/training/lr_schedule.py:11-185)."""
from __future__ import annotations

import math
from typing import List, Optional


class CosineScheduleWithWarmup:
    """Linear warm-up from ``warmup_init_lr`` to ``max_lr`` over ``warmup_steps``, cosine
    decay to ``min_lr`` at ``max_steps``, constant afterwards.  ``step()`` writes the
    same LR into every param group (group LR ratios are not preserved; this is the
    reference's behaviour, lr_schedule.py:98-103).  ``preserve_ratios=True`` scales
    each group's initial LR by lr/max_lr instead."""

    def __init__(self, optimizer, warmup_steps: int, max_steps: int, max_lr: float, min_lr: float,
                 warmup_init_lr: float = 0.0, preserve_ratios: bool = False):
        self.optimizer = optimizer
        self.warmup_steps, self.max_steps = warmup_steps, max_steps
        self.max_lr, self.min_lr, self.warmup_init_lr = max_lr, min_lr, warmup_init_lr
        self.current_step = 0
        self.preserve_ratios = preserve_ratios
        # ``initial_lr`` travels with the optimizer's state dict, so a scheduler built on a restored
        # optimizer (whose ``lr`` is already scaled) still sees each group's base rate
        self._base_lrs = [g.setdefault("initial_lr", g["lr"]) for g in optimizer.param_groups]

    def get_lr(self, step: Optional[int] = None) -> float:
        s = self.current_step if step is None else step
        if s < self.warmup_steps:
            return self.warmup_init_lr + (self.max_lr - self.warmup_init_lr) * (s / self.warmup_steps)
        if s < self.max_steps:
            prog = (s - self.warmup_steps) / (self.max_steps - self.warmup_steps)
            return self.min_lr + 0.5 * (self.max_lr - self.min_lr) * (1 + math.cos(math.pi * prog))
        return self.min_lr

    def step(self) -> float:
        self.current_step += 1
        return self.apply()

    def apply(self) -> float:
        """Write the rate of ``current_step`` into the param groups without advancing (used after a
        resume, so the first step after it runs at the rate the uninterrupted run would use)."""
        lr = self.get_lr()
        self._last_lr = []
        for g, base in zip(self.optimizer.param_groups, self._base_lrs):
            g["lr"] = base * lr / self.max_lr if self.preserve_ratios else lr
            self._last_lr.append(g["lr"])
        return lr

    def get_last_lr(self) -> List[float]:
        if not hasattr(self, "_last_lr"):
            return [self.get_lr(1)] * len(self.optimizer.param_groups)
        return self._last_lr

    def state_dict(self) -> dict:
        return {"current_step": self.current_step, "warmup_steps": self.warmup_steps,
                "max_steps": self.max_steps, "max_lr": self.max_lr, "min_lr": self.min_lr,
                "warmup_init_lr": self.warmup_init_lr}

    def load_state_dict(self, state_dict: dict) -> None:
        for k in ("current_step", "warmup_steps", "max_steps", "max_lr", "min_lr", "warmup_init_lr"):
            setattr(self, k, state_dict[k])


def get_lr_scheduler(optimizer, total_tokens: int, batch_size: int, seq_len: int,
                     warmup_steps: int = 2000, max_lr: float = 3e-4, min_lr_ratio: float = 0.1):
    max_steps = total_tokens // (batch_size * seq_len)
    return CosineScheduleWithWarmup(optimizer, warmup_steps, max_steps, max_lr, max_lr * min_lr_ratio, 0.0)


def cosine_lambda(warmup_steps: int, total_steps: int, min_ratio: float = 0.1):
    """Multiplier for ``torch.optim.lr_scheduler.LambdaLR`` as used by the distributed
    entrypoint (reference: train_distributed.py:400-418)."""
    def f(step: int) -> float:
        if step < warmup_steps:
            return step / max(1, warmup_steps)
        prog = (step - warmup_steps) / max(1, total_steps - warmup_steps)
        return max(min_ratio, 0.5 * (1.0 + math.cos(math.pi * min(prog, 1.0))))
    return f

"""Metric sinks: JSONL file, optional Weights & Biases, optional TensorBoard.

Metric names follow the reference (loss, lm_loss, aux_loss, mt_loss_t{i}, lr, grad_norm,
tokens_seen, tokens_per_sec, router/avg_entropy, router/max_usage, router/collapsed_layers;
reference: trainer.py:243-253, train.py:1097-1185).
"""
from __future__ import annotations

import json
import os
import time
from typing import Any, Dict, Optional


class MetricLogger:
    def __init__(self, jsonl_path: Optional[str] = None, use_wandb: bool = False, project: str = "moe-architecture",
                 run_name: Optional[str] = None, config: Optional[dict] = None, tensorboard_dir: Optional[str] = None,
                 rank: int = 0, entity: Optional[str] = None):
        self.rank = rank
        self.f = None
        self.wandb = None
        self.tb = None
        if rank != 0:
            return
        if jsonl_path:
            os.makedirs(os.path.dirname(os.path.abspath(jsonl_path)), exist_ok=True)
            self.f = open(jsonl_path, "a")
        if use_wandb:
            try:
                import wandb
                wandb.init(project=project, name=run_name, config=config, **({'entity': entity} if entity else {}))
                self.wandb = wandb
            except Exception as e:
                print(f"Warning: Could not initialize W&B: {e}")
        if tensorboard_dir:
            try:
                from torch.utils.tensorboard import SummaryWriter
                self.tb = SummaryWriter(tensorboard_dir)
            except Exception as e:
                print(f"Warning: TensorBoard unavailable: {e}")

    def log(self, metrics: Dict[str, Any], step: Optional[int] = None) -> None:
        if self.rank != 0:
            return
        clean = {k: (float(v) if hasattr(v, "item") else v) for k, v in metrics.items()}
        if self.f is not None:
            self.f.write(json.dumps({"time": time.time(), "step": step, **clean}) + "\n")
            self.f.flush()
        if self.wandb is not None:
            self.wandb.log(clean, step=step)
        if self.tb is not None:
            for k, v in clean.items():
                if isinstance(v, (int, float)):
                    self.tb.add_scalar(k, v, step)

    def close(self):
        if self.f is not None:
            self.f.close()
        if self.wandb is not None:
            self.wandb.finish()
        if self.tb is not None:
            self.tb.close()

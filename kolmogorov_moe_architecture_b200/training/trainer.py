"""``Trainer``: the library training loop (reference: moe_arch/training/trainer.py:24-388).

Same constructor arguments, metric names, evaluation and checkpoint format (format A:
``checkpoint_step_{N}.pt`` / ``checkpoint_final.pt`` / ``checkpoint_interrupted.pt``).  The step
itself goes through :class:`TrainEngine`; losses are accumulated on the device and read
back only at ``log_interval`` (the reference reads three scalars back every micro-step,
trainer.py:188-191).
"""
from __future__ import annotations

import math
import time
from pathlib import Path
from typing import Any, Dict, Optional

import torch

from ..utils.logging import MetricLogger
from .checkpoint import load_model_state, save_format_a
from .engine import TrainEngine


class Trainer:
    def __init__(self, model, optimizer, lr_scheduler, train_loader, val_loader, config: Dict[str, Any],
                 device: str = "cuda", use_amp: bool = True, gradient_accumulation_steps: int = 1,
                 gradient_clip_norm: float = 1.0, checkpoint_dir: str = "./checkpoints", log_interval: int = 10,
                 eval_interval: int = 1000, save_interval: int = 1000, use_wandb: bool = False,
                 jsonl_path: Optional[str] = None, dp=None, verbose: bool = True):
        self.device = torch.device(device)
        self.model = model.to(self.device) if dp is None else model
        self.optimizer, self.lr_scheduler = optimizer, lr_scheduler
        self.train_loader, self.val_loader, self.config = train_loader, val_loader, config
        self.use_amp = use_amp
        self.gradient_accumulation_steps, self.gradient_clip_norm = gradient_accumulation_steps, gradient_clip_norm
        self.checkpoint_dir = Path(checkpoint_dir)
        self.checkpoint_dir.mkdir(parents=True, exist_ok=True)
        self.log_interval, self.eval_interval, self.save_interval = log_interval, eval_interval, save_interval
        self.scaler = None
        self.global_step = self.epoch = self.tokens_seen = 0
        self.verbose = verbose
        self.logger = MetricLogger(jsonl_path=jsonl_path, use_wandb=use_wandb, project="moe-architecture",
                                   run_name=config.get("run_name", "moe-5b") if isinstance(config, dict) else None,
                                   config=config if isinstance(config, dict) else None)
        self.use_wandb = self.logger.wandb is not None
        params_fp32 = next(model.parameters()).dtype == torch.float32
        amp_dtype = torch.bfloat16 if (use_amp and params_fp32 and self.device.type == "cuda") else None
        # accumulation is keyed on the micro-step counter, as in the reference (trainer.py:200)
        self.engine = TrainEngine(self.model, optimizer, None, gradient_clip_norm, 1, amp_dtype, dp, self.device)

    def _batches(self):
        it = iter(self.train_loader)
        while True:
            try:
                yield next(it)
            except StopIteration:
                self.epoch += 1
                it = iter(self.train_loader)

    def train(self, max_steps: Optional[int] = None):
        self.model.train()
        ga = self.gradient_accumulation_steps
        acc = {"loss": None, "lm": None, "aux": None}
        start = time.time()
        lr = self.lr_scheduler.get_lr() if hasattr(self.lr_scheduler, "get_lr") else None
        batches = self._batches()
        while max_steps is None or self.global_step < max_steps:
            batch = next(batches)
            ids = batch["input_ids"].to(self.device, non_blocking=True)
            labels = batch["labels"].to(self.device, non_blocking=True)
            if getattr(self.engine, "dp", None) is not None:
                # gradients are reduced over the ranks only with the micro-batch that completes the step
                self.engine.dp.set_sync((self.global_step + 1) % ga == 0)
            out = self.engine._forward_backward_scaled(ids, labels, batch.get("attention_mask"), ga)
            for k, v in (("loss", out["loss"]), ("lm", out["lm_loss"]), ("aux", out["aux_loss"])):
                v = v.detach().float() if torch.is_tensor(v) else torch.tensor(float(v), device=self.device)
                acc[k] = v if acc[k] is None else acc[k] + v
            self.tokens_seen += ids.numel()
            if (self.global_step + 1) % ga == 0:
                gnorm = self.engine.apply_update()
                lr = self.lr_scheduler.step() if self.lr_scheduler is not None else lr
                if self.global_step % self.log_interval == 0:
                    el = time.time() - start
                    log = {"step": self.global_step, "epoch": self.epoch, "loss": float(acc["loss"]) / ga,
                           "lm_loss": float(acc["lm"]) / ga, "aux_loss": float(acc["aux"]) / ga, "lr": lr,
                           "grad_norm": float(gnorm) if gnorm is not None else None,
                           "tokens_seen": self.tokens_seen, "tokens_per_sec": self.tokens_seen / el if el > 0 else 0}
                    for k, v in (out.get("multitoken_loss_dict") or {}).items():
                        log[f"mt_{k}"] = float(v)
                    self.logger.log(log, step=self.global_step)
                    if self.verbose:
                        print(f"step {self.global_step} | loss {log['loss']:.4f} | lm {log['lm_loss']:.4f} | "
                              f"aux {log['aux_loss']:.6f} | {log['tokens_per_sec']:,.0f} tok/s")
                acc = {"loss": None, "lm": None, "aux": None}
                if self.global_step % self.eval_interval == 0 and self.global_step > 0 and self.val_loader is not None:
                    ev = self.evaluate()
                    self.logger.log(ev, step=self.global_step)
                    self.model.train()
                if self.global_step % self.save_interval == 0 and self.global_step > 0:
                    self.save_checkpoint(f"checkpoint_step_{self.global_step}.pt")
            self.global_step += 1
        self.save_checkpoint("checkpoint_final.pt")

    @torch.no_grad()
    def evaluate(self, num_batches: int = 100) -> Dict[str, float]:
        self.model.eval()
        tot = tot_lm = None
        n_tok = 0
        it = iter(self.val_loader)
        for _ in range(num_batches):
            try:
                b = next(it)
            except StopIteration:
                break
            ids, labels = b["input_ids"].to(self.device), b["labels"].to(self.device)
            out = self.model(ids, labels=labels, return_logits=False)
            w = ids.numel()
            tot = out["loss"].float() * w if tot is None else tot + out["loss"].float() * w
            tot_lm = out["lm_loss"].float() * w if tot_lm is None else tot_lm + out["lm_loss"].float() * w
            n_tok += w
        if n_tok == 0:
            return {"eval_loss": float("nan"), "eval_lm_loss": float("nan"), "eval_ppl": float("nan")}
        loss, lm = float(tot) / n_tok, float(tot_lm) / n_tok
        return {"eval_loss": loss, "eval_lm_loss": lm, "eval_ppl": math.exp(min(lm, 50.0))}

    def save_checkpoint(self, filename: str):
        save_format_a(str(self.checkpoint_dir / filename), self.model, self.optimizer, self.lr_scheduler,
                      self.global_step, self.epoch, self.tokens_seen, self.config, self.scaler)

    def load_checkpoint(self, checkpoint_path: str):
        _, ck = load_model_state(self.model, checkpoint_path, map_location=self.device)
        self.optimizer.load_state_dict(ck["optimizer_state_dict"])
        if self.lr_scheduler is not None and ck.get("lr_scheduler_state_dict") is not None:
            self.lr_scheduler.load_state_dict(ck["lr_scheduler_state_dict"])
        self.global_step, self.epoch, self.tokens_seen = ck["global_step"], ck["epoch"], ck["tokens_seen"]

"""HuggingFace ``Trainer`` integration (reference: train_production.py:43-214).

``MoEModelWrapper`` gives the model the call signature and ``{'loss', 'logits'}`` result the HF
loop expects (its state-dict keys carry the ``model.`` prefix of reference checkpoints, format D);
``MoETrainer`` plugs in the hybrid Muon/AdamW optimizer and the cosine schedule;
``TrueLossLoggingCallback`` adds ``true_loss = loss / gradient_accumulation_steps`` to the logs.
Logits are only materialised when no labels are given (evaluation/generation); with labels
the loss comes from the fused LM-head + cross-entropy path.
"""
from __future__ import annotations

import torch

from .lr_schedule import CosineScheduleWithWarmup
from .muon_optimizer import get_muon_optimizer


class MoEModelWrapper(torch.nn.Module):
    def __init__(self, model, use_fp8: bool = False, return_logits_with_loss: bool = False):
        super().__init__()
        self.model = model
        self.config = model.config
        self.return_logits_with_loss = return_logits_with_loss

    def forward(self, input_ids, labels=None, attention_mask=None, **kwargs):
        need_logits = labels is None or self.return_logits_with_loss
        out = self.model(input_ids, attention_mask=attention_mask, labels=labels, return_logits=need_logits)
        res = {"loss": out["loss"]}
        if need_logits:
            res["logits"] = out["logits"]
        return res


def make_hf_classes():
    """Build the Trainer subclasses lazily so importing this package does not import transformers."""
    from transformers import Trainer, TrainerCallback

    class TrueLossLoggingCallback(TrainerCallback):
        def __init__(self, gradient_accumulation_steps: int):
            self.gradient_accumulation_steps = gradient_accumulation_steps

        def on_log(self, args, state, control, logs=None, **kwargs):
            if logs is not None and "loss" in logs:
                logs["accumulated_loss"] = logs["loss"]
                logs["true_loss"] = logs["loss"] / self.gradient_accumulation_steps

    class MoETrainer(Trainer):
        def __init__(self, muon_config: dict, lr_config: dict, log_interval: int = 10, *args, **kwargs):
            self.muon_config, self.lr_config, self.log_interval = muon_config, lr_config, log_interval
            self._seq_lengths, self._step_count = [], 0
            super().__init__(*args, **kwargs)

        def create_optimizer(self):
            if self.optimizer is None:
                if self.muon_config.get("type", "muon").lower() == "adamw":
                    self.optimizer = torch.optim.AdamW(self.model.parameters(), lr=self.args.learning_rate,
                                                       betas=(0.9, 0.95),
                                                       weight_decay=self.muon_config.get("weight_decay", 0.01))
                else:
                    self.optimizer = get_muon_optimizer(self.model, lr=self.args.learning_rate,
                                                        momentum=self.muon_config.get("momentum", 0.95),
                                                        weight_decay=self.muon_config.get("weight_decay", 0.01))
            return self.optimizer

        def create_scheduler(self, num_training_steps: int, optimizer=None):
            if self.lr_scheduler is None:
                self.lr_scheduler = CosineScheduleWithWarmup(
                    self.optimizer, self.args.warmup_steps, num_training_steps, self.args.learning_rate,
                    self.args.learning_rate * self.lr_config.get("min_lr_ratio", 0.1), 0.0)
            return self.lr_scheduler

        def compute_loss(self, model, inputs, return_outputs=False, num_items_in_batch=None):
            mi = {"input_ids": inputs["input_ids"], "labels": inputs.get("labels", inputs["input_ids"])}
            if "attention_mask" in inputs:
                mi["attention_mask"] = inputs["attention_mask"]
            self._step_count += 1
            if mi["input_ids"].shape[1] == 0:
                return torch.tensor(0.0, device=mi["input_ids"].device, requires_grad=True)
            out = model(**mi)
            return (out["loss"], out) if return_outputs else out["loss"]

    return MoETrainer, TrueLossLoggingCallback

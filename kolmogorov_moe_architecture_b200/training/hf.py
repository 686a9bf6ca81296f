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


class OnTheFlyDataCollator:
    """Collator for raw-text examples: tokenises ``example["text"]`` per batch (truncated and padded to
    ``max_length``) and sets ``labels = input_ids``, padding positions masked with -100 so they are not scored
    (reference: train_production.py:76-104, which scores the padding as well)."""

    def __init__(self, tokenizer, max_length: int):
        self.tokenizer, self.max_length = tokenizer, max_length

    def __call__(self, examples):
        batch = self.tokenizer([e["text"] for e in examples], truncation=True, max_length=self.max_length,
                               padding="max_length", return_tensors="pt")
        batch = dict(batch)
        labels = batch["input_ids"].clone()
        if "attention_mask" in batch:
            labels = labels.masked_fill(batch["attention_mask"] == 0, -100)
        batch["labels"] = labels
        return batch


def load_and_prepare_dataset(config: dict, tokenizer, split: str = "train"):
    """The ``data:`` section's data set for the HF loop: raw text rows for on-the-fly tokenisation
    (``data.tokenize_on_fly``) or rows tokenised up front to at most ``model.max_seq_len`` tokens, empty documents
    dropped, limited to ``data.max_examples``; a streaming data set is collected into memory first.  Without the
    ``datasets`` package or network access: a synthetic data set of random token rows, announced on stdout."""
    data = config.get("data") or {}
    max_len = int((config.get("model") or {}).get("max_seq_len", 2048))
    max_examples = data.get("max_examples")
    streaming = bool(data.get("use_streaming", False))
    on_fly = bool(data.get("tokenize_on_fly", False))
    try:
        import os
        if os.environ.get("HF_HUB_OFFLINE") == "1" or os.environ.get("KMOE_OFFLINE") == "1":
            raise RuntimeError("offline")
        from datasets import Dataset, load_dataset
        ds = load_dataset(data["dataset_name"], name=data.get("dataset_config"), split=split, streaming=streaming)
    except Exception as e:
        print(f"[data] {data.get('dataset_name')} unavailable ({type(e).__name__}); synthetic rows instead")
        return SyntheticRows(int((config.get("model") or {}).get("vocab_size", 50257)), max_len, int(max_examples or 1024))
    if streaming:
        rows = []
        for ex in ds:
            if ex.get("text", "").strip():
                rows.append(ex)
            if max_examples and len(rows) >= max_examples:
                break
        ds = Dataset.from_list(rows)
    else:
        if max_examples:
            ds = ds.select(range(min(int(max_examples), len(ds))))
        ds = ds.filter(lambda ex: ex.get("text", "").strip() != "")
    if on_fly:
        return ds
    tok = ds.map(lambda ex: tokenizer(ex["text"], truncation=True, max_length=max_len, padding=False), batched=True,
                 remove_columns=ds.column_names)
    return tok.filter(lambda ex: len(ex["input_ids"]) > 0)


class SyntheticRows(torch.utils.data.Dataset):
    """Random token rows with ``labels = input_ids`` (what the loaders fall back to without a data set)."""

    def __init__(self, vocab_size: int, seq_len: int, n: int, seed: int = 1234):
        g = torch.Generator().manual_seed(seed)
        self.rows = torch.randint(1, vocab_size, (n, seq_len), generator=g)

    def __len__(self):
        return self.rows.shape[0]

    def __getitem__(self, i):
        return {"input_ids": self.rows[i], "labels": self.rows[i].clone()}

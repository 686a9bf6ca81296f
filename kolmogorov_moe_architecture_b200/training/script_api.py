"""Helper functions and classes that the reference's training scripts define at module level and that other code
imports from them (``from train_distributed import wrap_model_with_fsdp, create_optimizer`` and the like).

The entry points of this framework are thin front ends of :mod:`.runner`; this module gives the same names the
same meaning on top of this framework's parts, and each entry script re-exports the ones its reference counterpart
defines.  References: train.py:52-237, train_distributed.py:60-744, train_custom.py:66-886.

Where a reference helper returns a wrapped model (FSDP), the helper here returns the model itself with the
parallel plan attached as ``model._kmoe_plan``: parameters are sharded or replicated by the plan, the optimizer
state lives in it, and ``create_optimizer`` / ``train_step`` / ``save_checkpoint`` look for it.
"""
from __future__ import annotations

import hashlib
import math
import os
from dataclasses import dataclass, field, fields
from typing import Any, Dict, Iterable, Iterator, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.data import DataLoader, IterableDataset

from ..utils.config_io import load_yaml, model_config_tolerant


# ----------------------------------------------------------------------------------------- configuration, ranks
def load_config(path: str = None, config_path: str = None) -> Dict[str, Any]:
    """The YAML file as a dict (``config_path``: the keyword some of the reference's scripts use)."""
    return load_yaml(config_path if path is None else path)


def setup_distributed() -> Tuple[int, int, int]:
    """(rank, world_size, local_rank).  Starts the default process group from the ``torchrun`` environment when
    there is one (NCCL on GPUs, gloo otherwise) and selects the local GPU; a plain single-process run gets
    (0, 1, 0) and no group."""
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    cuda = torch.cuda.is_available()
    if "RANK" in os.environ and "WORLD_SIZE" in os.environ and not dist.is_initialized():
        dist.init_process_group(backend="nccl" if cuda else "gloo")
    if cuda:
        torch.cuda.set_device(local_rank)
    if dist.is_initialized():
        return dist.get_rank(), dist.get_world_size(), local_rank
    return 0, 1, local_rank


def cleanup_distributed() -> None:
    if dist.is_initialized():
        dist.destroy_process_group()


def is_main_process() -> bool:
    return not dist.is_initialized() or dist.get_rank() == 0


def print_rank0(*args, **kwargs) -> None:
    if is_main_process():
        print(*args, **kwargs)


# --------------------------------------------------------------------------------------------------------- data
def load_tokenizer(config: Dict[str, Any]):
    """The tokenizer ``data.tokenizer_name`` names, with a pad token; the byte-level stand-in of
    ``data.TokenizerWrapper`` where it cannot be loaded."""
    from ..data.tokenizer import TokenizerWrapper
    name = (config.get("data") or {}).get("tokenizer_name", "gpt2")
    return TokenizerWrapper(name, vocab_size=None, verbose=is_main_process())


class PackedSequenceDataset(IterableDataset):
    """Documents of a text data set tokenised, joined with end-of-sequence tokens and cut into rows of
    ``max_seq_len``; rank r of ``world_size`` takes every ``world_size``-th row.  Without network access (or with
    ``KMOE_OFFLINE=1``) the rows are uniform random ids from ``seed``.  Yields ``input_ids`` and ``labels`` (equal:
    the model shifts), plus ``doc_ids`` when ``with_doc_ids``."""

    def __init__(self, dataset_name: str = "HuggingFaceFW/fineweb", dataset_config: Optional[str] = "sample-10BT",
                 tokenizer=None, max_seq_len: int = 2048, max_examples: Optional[int] = None, seed: int = 42,
                 rank: int = 0, world_size: int = 1, with_doc_ids: bool = False, vocab_size: Optional[int] = None):
        super().__init__()
        self.dataset_name, self.dataset_config, self.tokenizer = dataset_name, dataset_config, tokenizer
        self.max_seq_len, self.max_examples, self.seed = max_seq_len, max_examples, seed
        self.rank, self.world_size, self.with_doc_ids = rank, world_size, with_doc_ids
        self.vocab_size = vocab_size or getattr(tokenizer, "vocab_size", None) or 50257

    def _documents(self) -> Optional[Iterator[List[int]]]:
        from ..data.dolma_dataset import _open_first_available
        ds = _open_first_available("train", True, names=[(self.dataset_name, self.dataset_config)])
        if ds is None or self.tokenizer is None:
            return None

        def gen():
            for i, ex in enumerate(ds):
                if self.max_examples and i >= self.max_examples:
                    return
                text = ex.get("text", "")
                if text:
                    enc = self.tokenizer.encode(text, truncation=False)
                    yield enc["input_ids"] if isinstance(enc, dict) else enc
        return gen()

    def __iter__(self):
        from ..data.dolma_dataset import PackedDocumentDataset, SyntheticTokenDataset
        docs = self._documents()
        if docs is None:
            rows = iter(SyntheticTokenDataset(self.vocab_size, self.max_seq_len, seed=self.seed, rank=self.rank, low=1))
            stride = 1                                   # the synthetic stream is already per rank
        else:
            eos = getattr(self.tokenizer, "eos_token_id", 0) or 0
            rows = iter(PackedDocumentDataset(docs, self.max_seq_len, eos, 1, mask_cross_doc=False))
            stride = self.world_size
        for i, row in enumerate(rows):
            if stride > 1 and i % stride != self.rank:
                continue
            out = {"input_ids": row["input_ids"], "labels": row.get("labels", row["input_ids"]).clone()}
            if self.with_doc_ids and "doc_ids" in row:
                out["doc_ids"] = row["doc_ids"]
            yield out


def create_dataloader(config: Dict[str, Any], tokenizer, max_seq_len: Optional[int] = None,
                      batch_size: Optional[int] = None, rank: int = 0, world_size: int = 1) -> DataLoader:
    """Packed rows of the data set the ``data:`` section names, ``batch_size`` rows per batch."""
    data = config.get("data") or {}
    model = config.get("model") or {}
    train = config.get("training") or {}
    ds = PackedSequenceDataset(dataset_name=data.get("dataset_name", "HuggingFaceFW/fineweb"),
                               dataset_config=data.get("dataset_config", "sample-10BT"), tokenizer=tokenizer,
                               max_seq_len=max_seq_len or model.get("max_seq_len", 2048),
                               max_examples=data.get("max_examples"), rank=rank, world_size=world_size,
                               vocab_size=model.get("vocab_size"))
    return DataLoader(ds, batch_size=batch_size or train.get("batch_size", 1), num_workers=0,
                      pin_memory=torch.cuda.is_available())


# ------------------------------------------------------------------------------------------- model and parallel
def create_model(config: Dict[str, Any], rank: int = 0, world_size: int = 1):
    """(model, model configuration) from the ``model:`` section, read with the defaults of the reference's
    distributed launcher.  With ``moe_implementation: expert_parallel`` the expert count is rounded down to a
    multiple of the world size, as the reference does."""
    from ..models.transformer import MoETransformer
    cfg = model_config_tolerant(config)
    if cfg.moe_implementation == "expert_parallel" and world_size > 1 and cfg.n_experts % world_size:
        adjusted = max(cfg.n_experts // world_size, 1) * world_size
        print_rank0(f"n_experts {cfg.n_experts} -> {adjusted}: a multiple of the {world_size} ranks")
        cfg.n_experts = adjusted
    return MoETransformer(cfg, verbose=rank == 0), cfg


def _device_of(rank: int) -> torch.device:
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")


def wrap_model_with_fsdp(model: nn.Module, rank: int = 0, use_bf16: bool = True, cpu_offload: bool = False,
                         activation_checkpointing: bool = True, lr: float = 3e-4, weight_decay: float = 0.01,
                         betas=(0.9, 0.95)) -> nn.Module:
    """The reference's FULL_SHARD regime: every ``TransformerBlock`` (and the root: embedding, final norm, heads)
    becomes a unit of the parameter-sharded plan (``parallel.fsdp``), in bf16 on GPUs, optionally with the shards
    in pinned host memory, blocks recomputed in the backward pass when ``activation_checkpointing``.  Returns the
    model; the plan is ``model._kmoe_plan`` and holds the AdamW state."""
    from ..parallel.fsdp import FullyShardedDataParallel
    dev = _device_of(rank)
    model.to(dev)
    if use_bf16 and dev.type == "cuda":
        model.to(torch.bfloat16)
    if hasattr(model, "gradient_checkpointing"):
        model.gradient_checkpointing = bool(activation_checkpointing)
    model._kmoe_plan = FullyShardedDataParallel(model, lr=lr, betas=betas, weight_decay=weight_decay,
                                                cpu_offload=cpu_offload)
    return model


def setup_fsdp(model: nn.Module, config, local_rank: int = 0) -> nn.Module:
    """``wrap_model_with_fsdp`` driven by a ``TrainConfig`` (train_custom.py's name for it)."""
    return wrap_model_with_fsdp(model, local_rank, use_bf16=getattr(config, "dtype", "bfloat16") == "bfloat16",
                                cpu_offload=bool(getattr(config, "cpu_offload", False)),
                                activation_checkpointing=bool(getattr(config, "gradient_checkpointing", False)),
                                lr=float(getattr(config, "learning_rate", 3e-4)),
                                weight_decay=float(getattr(config, "weight_decay", 0.01)))


def create_optimizer(model: nn.Module, config: Dict[str, Any], use_8bit: bool = False):
    """AdamW at ``training.max_lr`` with betas (0.9, 0.95): weight decay ``optimizer.weight_decay`` on matrices,
    none on biases, norms and embeddings.  ``use_8bit`` takes bitsandbytes' 8-bit AdamW where it can be imported.
    A model under a parallel plan gets the plan's optimizer handle (the plan owns the sharded AdamW state), set to
    the same learning rate and decay."""
    opt = config.get("optimizer") or {}
    train = config.get("training") or {}
    lr, wd = float(train.get("max_lr", 3e-3)), float(opt.get("weight_decay", 0.01))
    plan = getattr(model, "_kmoe_plan", None)
    if plan is not None:
        handle = plan.optimizer
        for g in handle.param_groups:
            g["lr"] = lr
            if "weight_decay" in g:
                g["weight_decay"] = wd
        return handle
    decay, plain = [], []
    for name, p in model.named_parameters():
        if p.requires_grad:
            (plain if ("bias" in name or "norm" in name or "embedding" in name) else decay).append(p)
    groups = [{"params": decay, "weight_decay": wd}, {"params": plain, "weight_decay": 0.0}]
    if use_8bit:
        try:
            import bitsandbytes as bnb
            return bnb.optim.AdamW8bit(groups, lr=lr, betas=(0.9, 0.95), eps=1e-8)
        except ImportError:
            print_rank0("bitsandbytes is not installed: plain AdamW")
    return torch.optim.AdamW(groups, lr=lr, betas=(0.9, 0.95), eps=1e-8)


class WarmupCosine:
    """Linear warm-up to the base learning rates, then cosine decay to ``min_lr_ratio`` of them at ``total_steps``.
    Works on anything with ``param_groups`` (a torch optimizer or a plan's optimizer handle)."""

    def __init__(self, optimizer, warmup_steps: int, total_steps: int, min_lr_ratio: float = 0.1):
        self.optimizer, self.warmup, self.total, self.floor = optimizer, int(warmup_steps), int(total_steps), min_lr_ratio
        self.base = [float(g["lr"]) for g in optimizer.param_groups]
        self.last_step = 0
        self._apply()

    def factor(self, step: int) -> float:
        if step < self.warmup:
            return step / max(self.warmup, 1)
        progress = min(1.0, (step - self.warmup) / max(self.total - self.warmup, 1))
        return self.floor + (1.0 - self.floor) * 0.5 * (1.0 + math.cos(math.pi * progress))

    def _apply(self) -> None:
        f = self.factor(self.last_step)
        for g, b in zip(self.optimizer.param_groups, self.base):
            g["lr"] = b * f

    def step(self) -> None:
        self.last_step += 1
        self._apply()

    def get_last_lr(self) -> List[float]:
        return [float(g["lr"]) for g in self.optimizer.param_groups]

    get_lr = get_last_lr

    def state_dict(self) -> Dict[str, Any]:
        return {"last_step": self.last_step, "base": self.base}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.last_step, self.base = int(sd["last_step"]), list(sd["base"])
        self._apply()


def create_scheduler(optimizer, config: Dict[str, Any], total_steps: int) -> WarmupCosine:
    train = config.get("training") or {}
    return WarmupCosine(optimizer, train.get("warmup_steps", 500), total_steps, train.get("min_lr_ratio", 0.1))


class CosineWarmupScheduler(WarmupCosine):
    """train_custom.py's scheduler: absolute ``max_lr`` / ``min_lr`` instead of a ratio."""

    def __init__(self, optimizer, warmup_steps: int, max_steps: int = None, max_lr: Optional[float] = None,
                 min_lr: Optional[float] = None, total_steps: int = None):
        total_steps = max_steps if total_steps is None else total_steps
        if max_lr is not None:
            for g in optimizer.param_groups:
                g["lr"] = max_lr
        top = max(float(g["lr"]) for g in optimizer.param_groups)
        super().__init__(optimizer, warmup_steps, total_steps, (min_lr / top) if (min_lr is not None and top > 0) else 0.1)


# ------------------------------------------------------------------------------------------------- diagnostics
def check_parameter_gradients(model: nn.Module, step: int = 0, rank: int = 0) -> Dict[str, Any]:
    """Census of the gradients after a backward pass: per parameter group how many tensors have no gradient, a
    zero one, or a non-finite one, and the norms - the reference's ``--debug`` check."""
    from ..utils.fault import gradient_census, gradient_flow_report
    return {"step": step, "rank": rank, "census": gradient_census(model), "flow": gradient_flow_report(model)}


@torch.no_grad()
def collect_router_stats(model: nn.Module, batch: Optional[Dict[str, torch.Tensor]] = None) -> Dict[str, Dict[str, float]]:
    """Per MoE layer: share of the assignments of the busiest and idlest expert, normalised entropy of the usage,
    dead experts - from the counters the routers filled in the forward pass that just ran (``batch`` is accepted
    for the reference's signature; no second forward is needed)."""
    out: Dict[str, Dict[str, float]] = {}
    for name, mod in model.named_modules():
        counts = getattr(mod, "last_expert_counts", None)
        if counts is None:
            counts = getattr(mod, "_last_expert_counts", None)
        if counts is None or not torch.is_tensor(counts) or counts.numel() < 2:
            continue
        u = counts.float() / counts.float().sum().clamp(min=1)
        ent = float(-(u * torch.log(u + 1e-10)).sum() / math.log(u.numel()))
        out[name] = {"max_usage": float(u.max()), "min_usage": float(u.min()), "entropy": ent,
                     "dead_experts": int((u == 0).sum()), "n_experts": int(u.numel())}
    return out


def print_debug_stats(param_stats: Dict[str, Any], router_stats: Dict[str, Dict[str, float]], step: int,
                      rank: int = 0) -> None:
    if rank != 0:
        return
    from ..utils.fault import format_flow_report
    print(f"--- debug, step {step} ---")
    for group, s in (param_stats.get("census") or {}).items():
        print(f"  grad[{group}]: {s}")
    if param_stats.get("flow"):
        print(format_flow_report(param_stats["flow"]))
    for name, s in router_stats.items():
        print(f"  router {name}: entropy {s['entropy']:.3f} max {s['max_usage']:.3f} dead {s['dead_experts']}")


def check_router_collapse_fast(model: nn.Module, device=None, entropy_threshold: float = 0.7):
    """Router collapse probe on random hidden states, routers only (no forward pass of the model):
    (per-layer statistics, collapsed layers, one-line summary)."""
    from ..utils.fault import check_router_collapse
    return check_router_collapse(model, entropy_threshold=entropy_threshold)


# ------------------------------------------------------------------------------------------------ training step
def train_step(model: nn.Module, batch: Dict[str, torch.Tensor], optimizer, scheduler, grad_clip: float = 1.0,
               accumulation_steps: int = 1, step: int = 0, debug: bool = False, rank: int = 0) -> Dict[str, float]:
    """Forward, backward and - on every ``accumulation_steps``-th call - clip, optimizer step, scheduler step and
    gradient reset.  The batch goes to the model unshifted: the loss shifts labels itself, so shifting here as
    well (as the reference's launcher does, train_distributed.py:712-713 on top of losses.py:81-82) would train
    every head one position further ahead than it is named for."""
    dev = next((p.device for p in model.parameters() if p.device.type != "meta"), torch.device("cpu"))
    ids = batch["input_ids"].to(dev, non_blocking=True)
    labels = batch.get("labels", ids).to(dev, non_blocking=True)
    out = model(ids, labels=labels, return_logits=False) if _takes_return_logits(model) else model(ids, labels=labels)
    (out["loss"] / accumulation_steps).backward()
    aux = out.get("aux_loss", 0.0)
    metrics = {"loss": float(out["loss"].detach()), "lm_loss": float(out.get("lm_loss", out["loss"]).detach()),
               "aux_loss": float(aux.detach()) if torch.is_tensor(aux) else float(aux)}
    boundary = (step + 1) % accumulation_steps == 0
    if debug and boundary:
        print_debug_stats(check_parameter_gradients(model, step, rank), collect_router_stats(model, batch), step, rank)
    if boundary:
        plan = getattr(model, "_kmoe_plan", None)
        if plan is not None:
            metrics["grad_norm"] = float(plan.reduce_clip_and_step(optimizer, grad_clip if grad_clip > 0 else None))
        else:
            if grad_clip > 0:
                metrics["grad_norm"] = float(torch.nn.utils.clip_grad_norm_(model.parameters(), grad_clip))
            optimizer.step()
            optimizer.zero_grad(set_to_none=True)
        if scheduler is not None:
            scheduler.step()
    return metrics


def _takes_return_logits(model: nn.Module) -> bool:
    import inspect
    try:
        return "return_logits" in inspect.signature(model.forward).parameters
    except (TypeError, ValueError):
        return False


def compute_token_weights(seq_len: int, decay: float, device=None) -> torch.Tensor:
    """Loss weights by position: 1 everywhere for ``decay == 0``, else rising linearly by ``decay`` over the
    sequence, normalised to mean 1."""
    if decay == 0:
        return torch.ones(seq_len, device=device)
    w = 1.0 + decay * torch.arange(seq_len, device=device, dtype=torch.float32) / seq_len
    return w / w.mean()


def compute_loss(model: nn.Module, batch: Dict[str, torch.Tensor],
                 token_weights: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, Dict[str, float]]:
    """(loss, metrics).  Without weights: the model's own loss.  With ``token_weights`` (seq_len,): the
    position-weighted next-token cross-entropy of the first head, divided by the number of scored targets, plus
    the model's auxiliary loss."""
    ids, labels = batch["input_ids"], batch.get("labels", batch["input_ids"])
    out = model(ids, labels=labels, attention_mask=batch.get("attention_mask"))
    loss = out["loss"]
    if token_weights is not None and out.get("logits") is not None:
        logits, tgt = out["logits"][:, :-1], labels[:, 1:]
        ce = F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), tgt.reshape(-1), ignore_index=-100,
                             reduction="none").view(tgt.shape)
        w = token_weights[: ce.shape[1]].to(ce.device).unsqueeze(0)
        loss = (ce * w).sum() / (tgt != -100).sum().clamp(min=1)
        aux = out.get("aux_loss", 0.0)
        if torch.is_tensor(aux):
            loss = loss + aux
    metrics = {"loss": float(loss.detach()), "ppl": float(torch.exp(loss.detach().float().clamp(max=50)))}
    for k in ("lm_loss", "aux_loss"):
        if torch.is_tensor(out.get(k)):
            metrics[k] = float(out[k].detach())
    return loss, metrics


@torch.no_grad()
def evaluate(model: nn.Module, dataloader: Iterable, device=None, max_batches: int = 100) -> Dict[str, float]:
    """Mean language-model loss and perplexity over up to ``max_batches`` batches, in evaluation mode."""
    was_training = model.training
    model.eval()
    tot, n = 0.0, 0
    for i, b in enumerate(dataloader):
        if i >= max_batches:
            break
        ids = b["input_ids"].to(device) if device is not None else b["input_ids"]
        labels = b.get("labels", ids)
        labels = labels.to(device) if device is not None else labels
        out = model(ids, labels=labels)
        tot += float(out.get("lm_loss", out["loss"]))
        n += 1
    model.train(was_training)
    loss = tot / max(n, 1)
    return {"loss": loss, "ppl": math.exp(min(loss, 50.0)), "batches": n}


# ------------------------------------------------------------------------------------------------- bookkeeping
class TimingStats:
    """Running totals of the time spent per phase (``data``, ``forward``, ``backward``, ``optimizer``, ...)."""

    def __init__(self):
        self.reset()

    def reset(self) -> None:
        self.totals: Dict[str, float] = {}
        self.counts: Dict[str, int] = {}

    def update(self, phase: str = None, seconds: float = None, **phases: float) -> None:
        if phase is not None:
            phases[phase] = seconds
        for k, v in phases.items():
            self.totals[k] = self.totals.get(k, 0.0) + float(v)
            self.counts[k] = self.counts.get(k, 0) + 1

    def summary(self) -> str:
        whole = sum(self.totals.values()) or 1.0
        return " | ".join(f"{k} {1e3 * v / max(self.counts[k], 1):.1f} ms ({100 * v / whole:.0f} %)"
                          for k, v in self.totals.items())


class CUDAPrefetcher:
    """Iterates a loader one batch ahead: the next batch's host-to-device copy runs on a side stream while the
    current one is in use.  On a machine without a GPU it is the loader itself."""

    def __init__(self, dataloader: Iterable, device=None):
        self.loader = dataloader
        self.device = torch.device(device) if device is not None else _device_of(0)
        self.stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None

    def _move(self, batch):
        return {k: (v.to(self.device, non_blocking=True) if torch.is_tensor(v) else v) for k, v in batch.items()}

    def __iter__(self):
        it = iter(self.loader)
        if self.stream is None:
            yield from (self._move(b) for b in it)
            return
        nxt = None
        for b in it:
            with torch.cuda.stream(self.stream):
                moved = self._move(b)
            if nxt is not None:
                yield nxt
            torch.cuda.current_stream(self.device).wait_stream(self.stream)
            nxt = moved
        if nxt is not None:
            yield nxt


def get_model_state_dict(model: nn.Module) -> Dict[str, torch.Tensor]:
    """The state dict of the model itself: compile / data-parallel wrappers are looked through, and a model under
    the parameter-sharded plan is gathered in full (call on every rank)."""
    from .checkpoint import unwrap_model
    inner = unwrap_model(model)
    plan = getattr(inner, "_kmoe_plan", None)
    if plan is not None and hasattr(plan, "full_state_dict"):
        return plan.full_state_dict()
    return inner.state_dict()


def get_cache_path(tokenizer_name: str, seq_len: int, max_examples: Optional[int], pack_sequences: bool,
                   cache_dir: str = ".cache/tokenized") -> str:
    """Where a tokenised data set with these settings is cached: the settings are in the file name."""
    key = f"{tokenizer_name}|{seq_len}|{max_examples}|{int(bool(pack_sequences))}"
    tag = hashlib.md5(key.encode()).hexdigest()[:10]
    safe = tokenizer_name.replace("/", "_")
    return os.path.join(cache_dir, f"{safe}_s{seq_len}_n{max_examples or 'all'}_{'packed' if pack_sequences else 'padded'}_{tag}.pt")


@dataclass
class TrainConfig:
    """train_custom.py's flat training configuration: model, optimisation, data and logging settings in one
    object, filled from a YAML file's sections by ``from_yaml``.  Unknown keys are kept in ``extra``."""
    config_path: Optional[str] = None
    # optimisation
    learning_rate: float = 3e-4
    min_lr: float = 3e-5
    weight_decay: float = 0.01
    warmup_steps: int = 500
    max_steps: int = 10000
    batch_size: int = 4
    gradient_accumulation_steps: int = 1
    max_grad_norm: float = 1.0
    optimizer: str = "adamw"
    token_weight_decay: float = 0.0
    use_token_weights: bool = False
    # system
    dtype: str = "bfloat16"
    gradient_checkpointing: bool = False
    cpu_offload: bool = False
    use_fsdp: bool = True
    compile: bool = False
    seed: int = 42
    # data
    dataset_name: str = "HuggingFaceFW/fineweb"
    dataset_config: Optional[str] = "sample-10BT"
    tokenizer_name: str = "gpt2"
    max_seq_len: int = 2048
    max_examples: Optional[int] = None
    pack_sequences: bool = True
    use_document_attention_mask: bool = False
    num_workers: int = 0
    # logging / checkpoints
    checkpoint_dir: str = "checkpoints"
    save_interval: int = 1000
    log_interval: int = 10
    eval_interval: int = 500
    use_wandb: bool = False
    profile: bool = False
    model: Dict[str, Any] = field(default_factory=dict)
    extra: Dict[str, Any] = field(default_factory=dict)

    @classmethod
    def from_yaml(cls, path: str) -> "TrainConfig":
        raw = load_yaml(path)
        known = {f.name for f in fields(cls)}
        out = cls(config_path=path, model=dict(raw.get("model") or {}))
        rename = {"max_lr": "learning_rate", "gradient_clip_norm": "max_grad_norm", "total_steps": "max_steps"}
        for section in ("training", "optimizer", "data", "mixed_precision", "wandb"):
            for k, v in (raw.get(section) or {}).items():
                k = rename.get(k, k)
                if k == "type" and section == "optimizer":
                    out.optimizer = v
                elif k == "bf16" and section == "mixed_precision":
                    out.dtype = "bfloat16" if v else "float32"
                elif k == "enabled" and section == "wandb":
                    out.use_wandb = bool(v)
                elif k in known and k not in ("model", "extra"):
                    setattr(out, k, v)
                else:
                    out.extra[f"{section}.{k}"] = v
        train = raw.get("training") or {}
        if "min_lr_ratio" in train and "min_lr" not in train:
            out.min_lr = float(out.learning_rate) * float(train["min_lr_ratio"])
        if "max_seq_len" in out.model:
            out.max_seq_len = int(out.model["max_seq_len"])
        return out


# ------------------------------------------------------------------------------------------------- checkpoints
def save_checkpoint(model: nn.Module, optimizer, scheduler, step: int, config=None, metrics: Optional[Dict] = None,
                    is_fsdp: bool = False, checkpoint_dir: Optional[str] = None, keep: int = 3) -> Optional[str]:
    """Directory layout of train_custom.py: ``checkpoint-{step}/{model.pt, optimizer.pt, training_state.pt}``, the
    newest ``keep`` directories kept.  Under the parameter-sharded plan every rank takes part in gathering the full
    state dict (the reference returns early on the other ranks, which would hang the gather) and rank 0 writes."""
    from .checkpoint import save_format_c
    root = checkpoint_dir or getattr(config, "checkpoint_dir", None) or "checkpoints"
    state = {"step": int(step), "metrics": metrics or {},
             "scheduler": scheduler.state_dict() if scheduler is not None and hasattr(scheduler, "state_dict") else None}
    plan = getattr(model, "_kmoe_plan", None)
    if plan is not None and hasattr(plan, "full_state_dict"):
        full = plan.full_state_dict()                       # collective: every rank calls it
        if not is_main_process():
            return None
        d = os.path.join(root, f"checkpoint-{int(step)}")
        os.makedirs(d, exist_ok=True)
        torch.save(full, os.path.join(d, "model.pt"))
        torch.save(optimizer.state_dict() if optimizer is not None else {}, os.path.join(d, "optimizer.pt"))
        torch.save(state, os.path.join(d, "training_state.pt"))
        from .checkpoint import prune_checkpoints
        prune_checkpoints(root, keep)
        return d
    return save_format_c(root, int(step), model, optimizer, state, keep=keep, is_main=is_main_process())


def load_checkpoint(model: nn.Module, optimizer, scheduler, checkpoint_path: str, is_fsdp: bool = False) -> int:
    """Restore what ``save_checkpoint`` wrote; returns the step."""
    from .checkpoint import load_format_c
    plan = getattr(model, "_kmoe_plan", None)
    if plan is not None and hasattr(plan, "load_full_state_dict"):
        plan.load_full_state_dict(torch.load(os.path.join(checkpoint_path, "model.pt"), map_location="cpu"))
        state = torch.load(os.path.join(checkpoint_path, "training_state.pt"), map_location="cpu", weights_only=False)
    else:
        state = load_format_c(checkpoint_path, model, optimizer)
    if scheduler is not None and state.get("scheduler") is not None and hasattr(scheduler, "load_state_dict"):
        scheduler.load_state_dict(state["scheduler"])
    return int(state.get("step", 0))


class StandardDataset(IterableDataset):
    """One document per row, truncated or padded to ``max_seq_len`` (train_custom.py's unpacked alternative);
    padding positions carry the label -100.  Synthetic rows without network access."""

    def __init__(self, tokenizer=None, max_seq_len: int = 2048, dataset_name: str = "HuggingFaceFW/fineweb",
                 dataset_config: Optional[str] = "sample-10BT", max_examples: Optional[int] = None, rank: int = 0,
                 world_size: int = 1, seed: int = 42, vocab_size: Optional[int] = None):
        super().__init__()
        self.inner = PackedSequenceDataset(dataset_name, dataset_config, tokenizer, max_seq_len, max_examples, seed,
                                           rank, world_size, vocab_size=vocab_size)

    def __iter__(self):
        docs = self.inner._documents()
        if docs is None:
            yield from self.inner
            return
        S, pad = self.inner.max_seq_len, getattr(self.inner.tokenizer, "pad_token_id", 0) or 0
        for i, toks in enumerate(docs):
            if i % self.inner.world_size != self.inner.rank:
                continue
            ids = torch.full((S,), pad, dtype=torch.long)
            n = min(len(toks), S)
            ids[:n] = torch.tensor(toks[:n])
            labels = ids.clone()
            labels[n:] = -100
            yield {"input_ids": ids, "labels": labels}


# ------------------------------------------------------------------- single-GPU script (train.py) conveniences
def new_training_state() -> Dict[str, Any]:
    """The mutable record train.py keeps for its signal handler: model, optimizer, counters, where to save."""
    return {"model": None, "optimizer": None, "step": 0, "epoch": 0, "data_idx": 0, "losses": [], "total_tokens": 0,
            "config_path": None, "checkpoint_dir": None, "should_stop": False, "checkpoint_saved": False, "args": None}


_training_state = new_training_state()


def save_state_checkpoint(state: Dict[str, Any], path: str, reason: str = "scheduled") -> bool:
    """One ``.pt`` file in the layout of the reference's single-GPU script (step, epoch, data_idx, the last 1000
    losses, total_tokens, config_path, model_state_dict, optimizer_state_dict - a list of two for the hybrid
    optimizer).  False when the record holds no model."""
    from .checkpoint import save_format_b
    if state.get("model") is None:
        print("[checkpoint] nothing to save: no model")
        return False
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    save_format_b(path, state["model"], state.get("optimizer"), state["step"], state["epoch"], state["data_idx"],
                  state["losses"], state["total_tokens"], state.get("config_path"))
    last = f"{state['losses'][-1]:.4f}" if state["losses"] else "n/a"
    print(f"[checkpoint] saved ({reason}): {path}  step {state['step']} epoch {state['epoch']} loss {last}")
    state["checkpoint_saved"] = True
    return True


def signal_handler(signum, frame, state: Optional[Dict[str, Any]] = None) -> None:
    """SIGINT / SIGTERM: mark the run as stopping, save ``checkpoint-{step}-interrupted.pt`` once, exit 0."""
    import signal as _signal
    import sys
    st = _training_state if state is None else state
    name = _signal.Signals(signum).name
    print(f"\n[signal] {name}: saving a checkpoint and leaving")
    st["should_stop"] = True
    if not st["checkpoint_saved"] and st["model"] is not None and st.get("checkpoint_dir"):
        save_state_checkpoint(st, os.path.join(st["checkpoint_dir"], f"checkpoint-{st['step']}-interrupted.pt"),
                              reason=f"interrupted by {name}")
    sys.exit(0)


def get_dataloader(tokenizer, seq_len: int, batch_size: int, max_examples: Optional[int] = None,
                   pack_sequences: bool = True, tokenizer_name: str = "gpt2", cache: bool = True):
    """Batches of a tokenised text data set as one (n_batches, batch_size, seq_len) tensor, cached on disk under
    ``get_cache_path`` (the reference's single-GPU script indexes such a tensor, train.py:869-871).  Packed rows by
    default; without network access the rows are the synthetic stream."""
    path = get_cache_path(tokenizer_name, seq_len, max_examples, pack_sequences)
    if cache and os.path.exists(path):
        return torch.load(path, map_location="cpu")
    cls = PackedSequenceDataset if pack_sequences else StandardDataset
    ds = cls(tokenizer=tokenizer, max_seq_len=seq_len, max_examples=max_examples)
    n_rows = max((max_examples or 4096) // 4, batch_size) // batch_size * batch_size
    rows = []
    for row in ds:
        rows.append(row["input_ids"])
        if len(rows) >= n_rows:
            break
    rows = rows[: len(rows) // batch_size * batch_size]
    data = torch.stack(rows).view(-1, batch_size, seq_len)
    if cache:
        os.makedirs(os.path.dirname(path), exist_ok=True)
        torch.save(data, path)
    return data

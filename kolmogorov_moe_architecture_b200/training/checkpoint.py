"""Checkpoint I/O in the reference's formats, plus sharded saves.

Formats (all hold the model under the key schema of the reference, so files interchange):

* ``A`` - ``Trainer``: one ``.pt`` dict ``{model_state_dict, optimizer_state_dict,
  lr_scheduler_state_dict, global_step, epoch, tokens_seen, config[, scaler_state_dict]}``
  (reference: moe_arch/training/trainer.py:340-388).
* ``B`` - ``train.py``: ``{step, epoch, data_idx, losses[-1000:], total_tokens, config_path,
  model_state_dict, optimizer_state_dict}``; the hybrid optimizer's state is a list of two
  dicts; file ``checkpoint-{N}[-interrupted|-final].pt`` (reference: train.py:186-208).
* ``C`` - ``train_custom.py``: directory ``checkpoint-{step}/{model.pt, optimizer.pt,
  training_state.pt}``, newest three kept (reference: train_custom.py:770-847).
* ``D`` - HF ``Trainer`` directories whose model keys carry a ``model.`` prefix
  (reference: train_production.py:107-120).
* ``E`` - distillation: ``{layers: {idx: state_dict}, config}``.

``load_model_state`` accepts any of them (and a bare state dict, a ``model`` key, or keys
prefixed by ``_orig_mod.`` / ``module.`` / ``model.``).  ``save_sharded`` writes one
optimizer-state file per rank next to a single model file, all ranks taking part, so no
rank skips a collective (the reference's format-C writer returns early on non-main ranks
before a collective gather, train_custom.py:780-781).
"""
from __future__ import annotations

import os
import re
import shutil
from typing import Any, Dict, Optional

import torch

_PREFIXES = ("_orig_mod.", "module.", "model.")


def unwrap_model(model):
    for attr in ("_orig_mod", "module"):
        while hasattr(model, attr):
            model = getattr(model, attr)
    return model


def strip_prefixes(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out = {}
    for k, v in sd.items():
        changed = True
        while changed:
            changed = False
            for p in _PREFIXES:
                if k.startswith(p) and not k.startswith("model.layers") is False:
                    pass
            for p in ("_orig_mod.", "module."):
                if k.startswith(p):
                    k, changed = k[len(p):], True
        out[k] = v
    if out and all(k.startswith("model.") for k in out):
        out = {k[len("model."):]: v for k, v in out.items()}
    return out


def extract_model_state(obj: Any) -> Dict[str, torch.Tensor]:
    if isinstance(obj, dict):
        for key in ("model_state_dict", "model", "state_dict"):
            if key in obj and isinstance(obj[key], dict):
                return strip_prefixes(obj[key])
        if obj and all(torch.is_tensor(v) for v in obj.values()):
            return strip_prefixes(obj)
    raise ValueError("no model state dict found in checkpoint")


def load_checkpoint_file(path: str, map_location="cpu") -> Any:
    if os.path.isdir(path):
        for name in ("model.pt", "pytorch_model.bin"):
            f = os.path.join(path, name)
            if os.path.exists(f):
                return torch.load(f, map_location=map_location, weights_only=False)
        raise FileNotFoundError(f"no model file in {path}")
    return torch.load(path, map_location=map_location, weights_only=False)


def load_model_state(model, path_or_obj, strict: bool = True, map_location="cpu"):
    obj = load_checkpoint_file(path_or_obj, map_location) if isinstance(path_or_obj, str) else path_or_obj
    sd = extract_model_state(obj)
    return unwrap_model(model).load_state_dict(sd, strict=strict), obj


# ---------------------------------------------------------------- format A
def save_format_a(path, model, optimizer, lr_scheduler, global_step, epoch, tokens_seen, config, scaler=None):
    ck = {"model_state_dict": unwrap_model(model).state_dict(), "optimizer_state_dict": optimizer.state_dict(),
          "lr_scheduler_state_dict": lr_scheduler.state_dict() if lr_scheduler is not None else None,
          "global_step": global_step, "epoch": epoch, "tokens_seen": tokens_seen, "config": config}
    if scaler is not None:
        ck["scaler_state_dict"] = scaler.state_dict()
    _atomic_save(ck, path)


# ---------------------------------------------------------------- format B
def save_format_b(path, model, optimizer, step, epoch, data_idx, losses, total_tokens, config_path, extra=None):
    ck = {"step": step, "epoch": epoch, "data_idx": data_idx, "losses": list(losses)[-1000:],
          "total_tokens": total_tokens, "config_path": config_path,
          "model_state_dict": unwrap_model(model).state_dict(), "optimizer_state_dict": optimizer.state_dict()}
    if extra:
        ck.update(extra)
    _atomic_save(ck, path)


def format_b_name(step: int, suffix: Optional[str] = None) -> str:
    return f"checkpoint-{step}{'-' + suffix if suffix else ''}.pt"


# ---------------------------------------------------------------- format C
def save_format_c(root, step, model, optimizer, training_state: Dict, keep: int = 3, is_main: bool = True):
    d = os.path.join(root, f"checkpoint-{step}")
    if is_main:
        os.makedirs(d, exist_ok=True)
        _atomic_save(unwrap_model(model).state_dict(), os.path.join(d, "model.pt"))
        _atomic_save(optimizer.state_dict(), os.path.join(d, "optimizer.pt"))
        _atomic_save(training_state, os.path.join(d, "training_state.pt"))
        prune_checkpoints(root, keep)
    return d


def prune_checkpoints(root: str, keep: int = 3) -> None:
    ds = []
    for name in os.listdir(root):
        m = re.fullmatch(r"checkpoint-(\d+)", name)
        if m and os.path.isdir(os.path.join(root, name)):
            ds.append((int(m.group(1)), name))
    for _, name in sorted(ds)[:-keep] if keep > 0 else []:
        shutil.rmtree(os.path.join(root, name), ignore_errors=True)


def load_format_c(d: str, model, optimizer=None, map_location="cpu") -> Dict:
    unwrap_model(model).load_state_dict(torch.load(os.path.join(d, "model.pt"), map_location=map_location,
                                                   weights_only=False))
    if optimizer is not None and os.path.exists(os.path.join(d, "optimizer.pt")):
        optimizer.load_state_dict(torch.load(os.path.join(d, "optimizer.pt"), map_location=map_location,
                                             weights_only=False))
    ts = os.path.join(d, "training_state.pt")
    return torch.load(ts, map_location=map_location, weights_only=False) if os.path.exists(ts) else {}


# ---------------------------------------------------------- sharded (ZeRO) save
def save_sharded(root: str, step: int, model, dp, training_state: Dict, rank: int, keep: int = 3) -> str:
    """Rank 0 writes ``model.pt`` (parameters are replicated) and ``training_state.pt``; every rank
    writes ``optimizer-rank{r}.pt`` with the state of the tensors it owns."""
    import torch.distributed as dist
    d = os.path.join(root, f"checkpoint-{step}")
    os.makedirs(d, exist_ok=True)
    if rank == 0:
        _atomic_save(unwrap_model(model).state_dict(), os.path.join(d, "model.pt"))
        _atomic_save(training_state, os.path.join(d, "training_state.pt"))
    _atomic_save(dp.optimizer_state_dict(), os.path.join(d, f"optimizer-rank{rank}.pt"))
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
    if rank == 0:
        prune_checkpoints(root, keep)
    return d


def load_sharded(d: str, model, dp, rank: int, map_location="cpu") -> Dict:
    unwrap_model(model).load_state_dict(torch.load(os.path.join(d, "model.pt"), map_location=map_location,
                                                   weights_only=False))
    f = os.path.join(d, f"optimizer-rank{rank}.pt")
    if os.path.exists(f):
        dp.load_optimizer_state_dict(torch.load(f, map_location=map_location, weights_only=False))
    ts = os.path.join(d, "training_state.pt")
    return torch.load(ts, map_location=map_location, weights_only=False) if os.path.exists(ts) else {}


def save_param_sharded(root: str, step: int, plan, training_state: Dict, rank: int, keep: int = 3) -> str:
    """Checkpoint of the parameter-sharded plan: every rank helps gather the full parameters (rank 0
    writes them as an ordinary ``model.pt``) and writes its own shards with their AdamW moments."""
    import torch.distributed as dist
    d = os.path.join(root, f"checkpoint-{step}")
    os.makedirs(d, exist_ok=True)
    full = plan.full_state_dict(to_cpu=True)
    if rank == 0:
        _atomic_save(full, os.path.join(d, "model.pt"))
        _atomic_save(training_state, os.path.join(d, "training_state.pt"))
    _atomic_save(plan.shard_state_dict(), os.path.join(d, f"shards-rank{rank}.pt"))
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
    if rank == 0:
        prune_checkpoints(root, keep)
    return d


def load_param_sharded(d: str, plan, rank: int) -> Dict:
    """Restores shards and moments when the file of this rank matches the current layout, otherwise the
    parameters alone from ``model.pt`` (any world size)."""
    f = os.path.join(d, f"shards-rank{rank}.pt")
    done = False
    if os.path.exists(f):
        sd = torch.load(f, map_location="cpu", weights_only=False)
        if sd.get("world") == plan.world and sd.get("rank") == plan.rank:
            plan.load_shard_state_dict(sd)
            done = True
    if not done:
        plan.load_full_state_dict(torch.load(os.path.join(d, "model.pt"), map_location="cpu", weights_only=False))
    ts = os.path.join(d, "training_state.pt")
    return torch.load(ts, map_location="cpu", weights_only=False) if os.path.exists(ts) else {}


def _atomic_save(obj, path: str) -> None:
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    tmp = path + ".tmp"
    torch.save(obj, tmp)
    os.replace(tmp, path)

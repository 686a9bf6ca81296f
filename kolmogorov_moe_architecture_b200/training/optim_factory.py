"""Optimizer construction shared by the entrypoints and the benchmark."""
from __future__ import annotations

import torch

from .muon_optimizer import HybridOptimizer, Muon, split_muon_params


def make_adamw(params, lr: float, betas=(0.9, 0.95), weight_decay: float = 0.01):
    params = list(params)
    on_cuda = bool(params) and all(p.is_cuda for p in params)
    return torch.optim.AdamW(params, lr=lr, betas=betas, weight_decay=weight_decay, fused=on_cuda)


def build_optimizer(model, kind: str = "muon", lr: float = 1e-3, adamw_lr: float = 3e-4,
                    momentum: float = 0.95, weight_decay: float = 0.01, newton_iters: int = 5):
    """``muon``: Muon (Newton-Schulz, ``newton_iters`` steps) on the 2-D hidden weight matrices and
    AdamW on everything else (embeddings, heads, norms, biases, stacked expert tensors, conv and
    SSM vectors) - the dimension-and-name partition of the reference's ``get_muon_optimizer``
    outside sharded mode (muon_optimizer.py:526-537).  ``adamw``: AdamW on all parameters."""
    if kind == "adamw":
        return make_adamw(model.parameters(), adamw_lr, weight_decay=weight_decay)
    muon_p, adamw_p = split_muon_params(model, fsdp_mode=False)
    muon = Muon(muon_p, lr=lr, momentum=momentum, weight_decay=weight_decay,
                newton_iters=newton_iters) if muon_p else None
    adamw = make_adamw(adamw_p, adamw_lr, weight_decay=weight_decay) if adamw_p else None
    return HybridOptimizer(muon, adamw)

"""Mixture-of-Depths token router (reference: moe_arch/model/mod.py:18-171)."""
from __future__ import annotations

from typing import Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .linear import Linear


class MoDRouter(nn.Module):
    """Scalar router ``Linear(d, 1)`` choosing ``k = int(S * capacity)`` tokens per
    sequence; the kept indices are returned ascending and the output weights are a
    softmax over the kept logits.  A small MLP is trained with BCE to predict the
    selection from detached inputs (the causal-sampling predictor); that BCE, times
    ``mod_load_balance_loss_weight``, is the layer's auxiliary loss.
    """

    def __init__(self, config):
        super().__init__()
        self.d_model = config.d_model
        self.capacity_factor = config.mod_capacity_factor
        self.router = Linear(config.d_model, 1, bias=False)
        h = config.mod_router_hidden_dim
        self.aux_router = nn.Sequential(
            Linear(config.d_model, h, bias=False), nn.SiLU(), Linear(h, 1, bias=False))
        self.aux_loss_weight = config.mod_load_balance_loss_weight
        self.aux_loss = 0.0

    def num_selected(self, seq_len: int) -> int:
        return max(1, min(seq_len, int(seq_len * self.capacity_factor)))

    def _predictor_loss(self, hidden_states, topk_idx, like):
        aux_logits = self.aux_router(hidden_states.detach()).squeeze(-1)
        return self.aux_loss_weight * ops.mod_bce(aux_logits, topk_idx)

    def route_and_gather(self, hidden_states: torch.Tensor):
        """``forward`` followed by the gather of the kept rows, as one op (one node of the autograd graph on the
        GPU path): (kept rows (B, k, d), ascending indices, weights)."""
        B, S, _ = hidden_states.shape
        k = self.num_selected(S)
        picked, sorted_idx, weights, logits = ops.mod_score_gather(hidden_states, self.router.weight, k)
        self.aux_loss = self._predictor_loss(hidden_states, sorted_idx, logits) if self.training else 0.0
        return picked, sorted_idx, weights

    def forward(self, hidden_states: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
        B, S, _ = hidden_states.shape
        if S == 0:
            e_i = torch.zeros(B, 0, dtype=torch.long, device=hidden_states.device)
            e_f = hidden_states.new_zeros(B, 0)
            return e_i, e_f, e_f, e_i
        logits = self.router(hidden_states).squeeze(-1)
        k = self.num_selected(S)
        sorted_idx, weights, topk_idx = ops.mod_route(logits, k)
        self.aux_loss = self._predictor_loss(hidden_states, topk_idx, logits) if self.training else 0.0
        return sorted_idx, weights, logits, topk_idx


class MoDLayer(nn.Module):
    """Any layer under mixture-of-depths routing: the router keeps ``k`` positions per sequence, only those go
    through ``layer_module`` and come back weighted by the router; the other positions pass unchanged
    (``out = x`` there, ``out = x + w * layer(x_kept)`` at kept positions - the rule ``TransformerBlock`` applies to
    its FFN half).  In the reference this wrapper is stale (it unpacks three of the router's four results and
    overwrites the kept rows instead of adding to them, moe_arch/model/mod.py:174-234); this one follows the block's
    rule and exposes the router's auxiliary loss as ``aux_loss``.  At evaluation the layer runs on every position,
    as in the block."""

    def __init__(self, config, layer_module: nn.Module):
        super().__init__()
        self.config = config
        self.layer = layer_module
        self.router = MoDRouter(config)
        self.aux_loss = 0.0

    def forward(self, hidden_states: torch.Tensor, **layer_kwargs) -> torch.Tensor:
        if not self.training:
            self.aux_loss = 0.0
            return hidden_states + self.layer(hidden_states, **layer_kwargs)
        picked, idx, weights = self.router.route_and_gather(hidden_states)
        self.aux_loss = self.router.aux_loss
        processed = self.layer(picked, **layer_kwargs)
        return ops.mod_combine(hidden_states, processed, weights, idx)

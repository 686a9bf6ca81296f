"""``FusedSparseMoE`` and ``OptimizedGroupedExperts`` (API of the reference's
``moe_arch/model/fused_moe.py``).  In the reference "fused" is an aspiration - the router is
PyTorch and the experts a Python loop with a host sync per expert (fused_moe.py:249-253,300-319);
here both classes run the one grouped tcgen05 kernel path, keeping their parameter names
(``router_weight`` (d, E), ``w1/w2/w3``)."""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from .. import ops


def _init(w):
    nn.init.uniform_(w, -1.0 / math.sqrt(w.shape[1]), 1.0 / math.sqrt(w.shape[1]))


class OptimizedGroupedExperts(nn.Module):
    def __init__(self, n_experts: int, d_model: int, d_ff: int):
        super().__init__()
        self.n_experts, self.d_model, self.d_ff = n_experts, d_model, d_ff
        self.w1 = nn.Parameter(torch.empty(n_experts, d_model, d_ff))
        self.w2 = nn.Parameter(torch.empty(n_experts, d_model, d_ff))
        self.w3 = nn.Parameter(torch.empty(n_experts, d_ff, d_model))
        for w in (self.w1, self.w2, self.w3):
            _init(w)

    def forward(self, x, expert_indices, expert_weights):
        return ops.grouped_swiglu(x, self.w1, self.w2, self.w3, expert_indices, expert_weights)


class FusedSparseMoE(nn.Module):
    def __init__(self, d_model: int, d_ff: int, n_experts: int, top_k: int = 2):
        super().__init__()
        self.d_model, self.d_ff, self.n_experts, self.top_k = d_model, d_ff, n_experts, top_k
        self.router_weight = nn.Parameter(torch.empty(d_model, n_experts))
        self.w1 = nn.Parameter(torch.empty(n_experts, d_model, d_ff))
        self.w2 = nn.Parameter(torch.empty(n_experts, d_model, d_ff))
        self.w3 = nn.Parameter(torch.empty(n_experts, d_ff, d_model))
        nn.init.normal_(self.router_weight, std=0.02)
        for w in (self.w1, self.w2, self.w3):
            _init(w)
        self.aux_loss = 0.0

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        flat = x.reshape(-1, self.d_model)
        logits = flat @ self.router_weight
        w, idx = ops.topk_softmax_route(logits, self.top_k)
        if self.training:
            self.aux_loss = ops.moe_aux_loss(logits, idx, self.n_experts, 0.01, 0.001)
        return ops.grouped_swiglu(flat, self.w1, self.w2, self.w3, idx, w).view(shape)

"""Experts of unequal width that grow and shrink during distillation (counterpart of the
reference's ``Experiments/sparse_distillation/dynamic_experts.py``)."""
from __future__ import annotations

from typing import Dict, List

import torch
import torch.nn as nn
import torch.nn.functional as F


class DynamicExpertLayer(nn.Module):
    """SwiGLU experts with per-expert hidden width ``d_ffs[e]``; token-choice forward."""

    def __init__(self, d_model: int, d_ffs: List[int]):
        super().__init__()
        self.d_model, self.d_ffs = d_model, list(d_ffs)
        self.w1 = nn.ParameterList([nn.Parameter(torch.randn(d_model, f) * d_model ** -0.5) for f in d_ffs])
        self.w2 = nn.ParameterList([nn.Parameter(torch.randn(d_model, f) * d_model ** -0.5) for f in d_ffs])
        self.w3 = nn.ParameterList([nn.Parameter(torch.randn(f, d_model) * f ** -0.5) for f in d_ffs])

    @property
    def n_experts(self) -> int:
        return len(self.d_ffs)

    def expert(self, e: int, x: torch.Tensor) -> torch.Tensor:
        return (F.silu(x @ self.w1[e]) * (x @ self.w2[e])) @ self.w3[e]

    def forward(self, x: torch.Tensor, idx: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
        out = torch.zeros_like(x)
        for e in range(self.n_experts):
            tok, slot = (idx == e).nonzero(as_tuple=True)
            if tok.numel():
                out.index_add_(0, tok, self.expert(e, x[tok]) * weights[tok, slot].unsqueeze(1).to(x.dtype))
        return out


def interpolate_expert_weights(w1, w2, w3, new_f: int):
    """Resize one expert's hidden width.  Growing interpolates the hidden axis linearly; shrinking
    keeps the ``new_f`` hidden units with the largest L2 importance ||w1_j|| ||w2_j|| ||w3_j||."""
    f = w1.shape[1]
    if new_f == f:
        return w1, w2, w3
    if new_f < f:
        imp = w1.norm(dim=0) * w2.norm(dim=0) * w3.norm(dim=1)
        keep = torch.topk(imp, new_f).indices.sort().values
        return w1[:, keep], w2[:, keep], w3[keep]
    up = lambda t: F.interpolate(t.unsqueeze(0), size=new_f, mode="linear", align_corners=True).squeeze(0)
    scale = (f / new_f) ** 0.5
    return up(w1), up(w2), up(w3.t()).t() * scale * scale


class DynamicExpertTracker:
    """Exponential moving average of the per-expert reconstruction loss and token share."""

    def __init__(self, n_experts: int, momentum: float = 0.99):
        self.loss = torch.zeros(n_experts)
        self.share = torch.zeros(n_experts)
        self.momentum, self.steps = momentum, 0

    def update(self, per_expert_loss: torch.Tensor, counts: torch.Tensor):
        m = self.momentum if self.steps else 0.0
        self.loss = m * self.loss + (1 - m) * per_expert_loss.detach().float().cpu()
        self.share = m * self.share + (1 - m) * (counts.float() / counts.sum().clamp(min=1)).cpu()
        self.steps += 1

    def plan(self, d_ffs: List[int], top_k_grow=2, top_k_shrink=2, growth=1.25, shrink=0.8, lo=256, hi=8192) -> Dict[int, int]:
        order = torch.argsort(self.loss * self.share, descending=True).tolist()
        plan = {}
        for e in order[:top_k_grow]:
            plan[e] = min(hi, int(d_ffs[e] * growth) // 8 * 8)
        for e in order[::-1][:top_k_shrink]:
            if e not in plan:
                plan[e] = max(lo, int(d_ffs[e] * shrink) // 8 * 8)
        return {e: f for e, f in plan.items() if f != d_ffs[e]}


@torch.no_grad()
def reallocate_expert_layer(layer: DynamicExpertLayer, plan: Dict[int, int]) -> DynamicExpertLayer:
    for e, f in plan.items():
        a, b, c = interpolate_expert_weights(layer.w1[e].data, layer.w2[e].data, layer.w3[e].data, f)
        layer.w1[e], layer.w2[e], layer.w3[e] = nn.Parameter(a.contiguous()), nn.Parameter(b.contiguous()), nn.Parameter(c.contiguous())
        layer.d_ffs[e] = f
    return layer

"""Experts of unequal width that grow and shrink during distillation (counterpart of the
reference's ``Experiments/sparse_distillation/dynamic_experts.py``)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class DynamicExpertConfig:
    """When and by how much expert widths change (reference: dynamic_experts.py:33-51)."""
    reallocate_every_n_steps: int = 500
    growth_factor: float = 1.25
    shrink_factor: float = 0.8
    min_d_ff: int = 256
    max_d_ff: int = 8192
    top_k_grow: int = 2                 # the experts with the highest loss grow
    top_k_shrink: int = 2               # the ones with the lowest loss shrink
    maintain_param_budget: bool = True  # rescale all widths so that the total stays what it was
    round_to: int = 8                   # widths stay multiples of this (vector loads, tensor-core tiles)


@dataclass
class ExpertStats:
    """Running reconstruction loss of one expert since the last reallocation."""
    expert_idx: int
    d_ff: int
    total_loss: float = 0.0
    token_count: int = 0

    @property
    def avg_loss(self) -> float:
        return self.total_loss / max(self.token_count, 1)


class DynamicExpertLayer(nn.Module):
    """SwiGLU experts with per-expert hidden width ``d_ffs[e]``; token-choice forward."""

    def __init__(self, d_model: int = None, d_ffs: List[int] = None, d_ff_per_expert: List[int] = None,
                 activation: str = "swiglu", n_experts: int = None):
        """``DynamicExpertLayer(d_model, [f_0, f_1, ...])``, or in the reference's order
        ``DynamicExpertLayer(n_experts, d_model, d_ff_per_expert)`` (dynamic_experts.py:61)."""
        super().__init__()
        if d_ff_per_expert is not None and not isinstance(d_ffs, (list, tuple)):
            # reference order: the first positional is the expert count, the second the model width
            first, second = d_model, d_ffs
            if n_experts is None and second is not None:
                n_experts, d_model = first, second
            d_ffs = d_ff_per_expert
        assert activation == "swiglu", "dynamic experts are SwiGLU experts"
        assert n_experts is None or n_experts == len(d_ffs), "one width per expert"
        self.d_model, self.d_ffs = d_model, list(d_ffs)
        self.w1 = nn.ParameterList([nn.Parameter(torch.randn(d_model, f) * d_model ** -0.5) for f in d_ffs])
        self.w2 = nn.ParameterList([nn.Parameter(torch.randn(d_model, f) * d_model ** -0.5) for f in d_ffs])
        self.w3 = nn.ParameterList([nn.Parameter(torch.randn(f, d_model) * f ** -0.5) for f in d_ffs])

    @property
    def n_experts(self) -> int:
        return len(self.d_ffs)

    def expert(self, e: int, x: torch.Tensor) -> torch.Tensor:
        return (F.silu(x @ self.w1[e]) * (x @ self.w2[e])) @ self.w3[e]

    def forward_expert(self, x: torch.Tensor, expert_idx: int) -> torch.Tensor:
        return self.expert(expert_idx, x)

    @property
    def d_ff_per_expert(self) -> List[int]:
        return self.d_ffs

    def get_expert_params(self, expert_idx: int) -> int:
        return 3 * self.d_model * self.d_ffs[expert_idx]

    def get_total_params(self) -> int:
        return sum(self.get_expert_params(e) for e in range(self.n_experts))

    def get_avg_active_params(self, top_k: int = 2, usage: Optional[torch.Tensor] = None) -> float:
        """Expected expert parameters touched per token: ``top_k`` times the mean expert size, weighted by
        the experts' token shares when ``usage`` is given (wide experts that are rarely picked cost little)."""
        sizes = torch.tensor([float(self.get_expert_params(e)) for e in range(self.n_experts)])
        if usage is None:
            return float(top_k * sizes.mean())
        u = usage.float().cpu()
        return float(top_k * (sizes * u / u.sum().clamp(min=1e-12)).sum())

    def forward(self, x: torch.Tensor, idx: torch.Tensor = None, weights: torch.Tensor = None, *,
                expert_weights: torch.Tensor = None, token_indices: torch.Tensor = None):
        """Token choice: ``forward(x (T, d), idx (T, k), weights (T, k))`` -> (T, d).
        Expert choice (the reference's form, dynamic_experts.py:108-146): ``forward(x (B, S, d), expert_weights
        (B, E, C), token_indices (B, E, C))`` -> (output (B, S, d), {expert: its (B, C, d) outputs})."""
        if expert_weights is not None or (x.dim() == 3 and idx is not None and idx.is_floating_point()):
            ew = expert_weights if expert_weights is not None else idx
            ti = token_indices if token_indices is not None else weights
            out = torch.zeros_like(x)
            per_expert = {}
            for e in range(self.n_experts):
                gi = ti[:, e, :].unsqueeze(-1).expand(-1, -1, x.shape[-1])
                y = self.expert(e, torch.gather(x, 1, gi))
                per_expert[e] = y
                out = out.scatter_add(1, gi, y * ew[:, e, :].unsqueeze(-1).to(y.dtype))
            return out, per_expert
        out = torch.zeros_like(x)
        for e in range(self.n_experts):
            tok, slot = (idx == e).nonzero(as_tuple=True)
            if tok.numel():
                out.index_add_(0, tok, self.expert(e, x[tok]) * weights[tok, slot].unsqueeze(1).to(x.dtype))
        return out


def interpolate_expert_weights(old_w1, old_w2, old_w3, new_d_ff: int, importance: str = "sum",
                               rescale: str = "sqrt"):
    """Resize one expert's hidden width (reference: dynamic_experts.py:166-238; the defaults are its rules).

    Growing interpolates the hidden axis linearly and rescales the down projection.  The hidden units of a trained
    expert are not ordered, so neighbours are close to independent and the output - a sum over the units - grows
    like the square root of their number: ``rescale="sqrt"`` multiplies w3 by ``sqrt(old / new)`` (on random
    weights the output norm then stays within 10-35 % of the original).  ``rescale="exact"`` multiplies by
    ``old / new``, which is right only for weights that vary smoothly along the hidden axis.

    Shrinking keeps the ``new_d_ff`` most important hidden units in their original order.  The importance of unit j
    is ``||w1_j|| + ||w2_j|| + ||w3_j||`` (``importance="sum"``) or the product of the three norms
    (``"product"``: the size of the unit's contribution to the output)."""
    w1, w2, w3, new_f = old_w1, old_w2, old_w3, new_d_ff
    f = w1.shape[1]
    if new_f == f:
        return w1, w2, w3
    if new_f < f:
        n1, n2, n3 = w1.norm(dim=0), w2.norm(dim=0), w3.norm(dim=1)
        imp = n1 * n2 * n3 if importance == "product" else n1 + n2 + n3
        keep = torch.topk(imp, new_f).indices.sort().values
        return w1[:, keep], w2[:, keep], w3[keep]
    up = lambda t: F.interpolate(t.unsqueeze(0), size=new_f, mode="linear", align_corners=True).squeeze(0)
    scale = f / new_f if rescale == "exact" else (f / new_f) ** 0.5
    return up(w1), up(w2), up(w3.t()).t() * scale


class DynamicExpertTracker:
    """Per-expert loss bookkeeping for width reallocation.  Two views are kept: an exponential moving
    average of loss and token share (``update`` / ``plan``: grow where loss x share is largest), and plain
    sums since the last reallocation (``update_stats`` / ``compute_reallocation``, the reference's scheme:
    dynamic_experts.py:241-345 - rank by mean loss, grow the worst, shrink the best, optionally rescale all
    widths so the layer's parameter count stays put)."""

    def __init__(self, n_experts: int, initial_d_ff: Optional[int] = None, d_model: Optional[int] = None,
                 config: Optional[DynamicExpertConfig] = None, momentum: float = 0.99):
        # positional order of the reference: (n_experts, initial_d_ff, d_model, config)
        self.n_experts, self.d_model = n_experts, d_model
        self.config = config or DynamicExpertConfig()
        self.loss = torch.zeros(n_experts)
        self.share = torch.zeros(n_experts)
        self.momentum, self.steps = momentum, 0
        self.expert_stats: Dict[int, ExpertStats] = {e: ExpertStats(e, initial_d_ff or 0) for e in range(n_experts)}
        self.step_count = 0
        self.reallocation_history: List[Dict] = []

    # ---- moving averages
    def update(self, per_expert_loss: torch.Tensor, counts: torch.Tensor):
        m = self.momentum if self.steps else 0.0
        self.loss = m * self.loss + (1 - m) * per_expert_loss.detach().float().cpu()
        self.share = m * self.share + (1 - m) * (counts.float() / counts.sum().clamp(min=1)).cpu()
        self.steps += 1
        self.step_count += 1
        for e in range(self.n_experts):
            n = int(counts[e])
            self.expert_stats[e].total_loss += float(per_expert_loss[e]) * n
            self.expert_stats[e].token_count += n

    def plan(self, d_ffs: List[int], top_k_grow=2, top_k_shrink=2, growth=1.25, shrink=0.8, lo=256, hi=8192) -> Dict[int, int]:
        order = torch.argsort(self.loss * self.share, descending=True).tolist()
        plan = {}
        for e in order[:top_k_grow]:
            plan[e] = min(hi, int(d_ffs[e] * growth) // 8 * 8)
        for e in order[::-1][:top_k_shrink]:
            if e not in plan:
                plan[e] = max(lo, int(d_ffs[e] * shrink) // 8 * 8)
        return {e: f for e, f in plan.items() if f != d_ffs[e]}

    # ---- sums since the last reallocation
    def update_stats(self, expert_outputs: Dict[int, torch.Tensor], targets: Dict[int, torch.Tensor]) -> None:
        """``expert_outputs[e]`` / ``targets[e]``: (n_e, d_model) rows routed to expert e and what they should be."""
        for e, out in expert_outputs.items():
            if e in targets and out.numel():
                self.expert_stats[e].total_loss += float(F.mse_loss(out.detach().float(), targets[e].float(), reduction="sum"))
                self.expert_stats[e].token_count += out.shape[0]
        self.step_count += 1

    def set_widths(self, d_ffs: List[int]) -> None:
        for e, f in enumerate(d_ffs):
            self.expert_stats[e].d_ff = int(f)

    def should_reallocate(self) -> bool:
        return self.step_count > 0 and self.step_count % self.config.reallocate_every_n_steps == 0

    def compute_reallocation(self) -> Dict[int, int]:
        """New width for every expert (unchanged ones included): the ``top_k_grow`` experts with the highest mean
        loss grow, the ``top_k_shrink`` with the lowest shrink.  With ``maintain_param_budget`` all widths are then
        scaled by ``before / after`` - parameters are linear in the width, so the layer's size really stays what
        it was (the reference scales by the square root of that ratio, dynamic_experts.py:327-340, which leaves
        the budget off by the other square root).  Widths are rounded down to multiples of ``round_to``."""
        c = self.config
        rnd = lambda f: max(c.round_to, int(f) // c.round_to * c.round_to)
        ranked = sorted(self.expert_stats.values(), key=lambda s: s.avg_loss, reverse=True)
        new = {s.expert_idx: s.d_ff for s in ranked}
        grow = ranked[: c.top_k_grow]
        for s in grow:
            new[s.expert_idx] = min(rnd(s.d_ff * c.growth_factor), c.max_d_ff)
        for s in ranked[::-1][: c.top_k_shrink]:
            if s not in grow:
                new[s.expert_idx] = max(rnd(s.d_ff * c.shrink_factor), c.min_d_ff)
        if c.maintain_param_budget:
            before, after = sum(s.d_ff for s in ranked), sum(new.values())
            if after != before and after > 0:
                k = before / after                      # parameters are linear in the width
                new = {e: min(max(rnd(f * k), c.min_d_ff), c.max_d_ff) for e, f in new.items()}
        self.reallocation_history.append({"step": self.step_count, "d_ff": dict(new),
                                          "avg_loss": {s.expert_idx: s.avg_loss for s in ranked}})
        return new

    def reset_stats(self) -> None:
        for s in self.expert_stats.values():
            s.total_loss, s.token_count = 0.0, 0

    def get_report(self) -> str:
        d = self.d_model or 1
        ranked = sorted(self.expert_stats.values(), key=lambda s: s.avg_loss, reverse=True)
        total = sum(3 * d * s.d_ff for s in ranked) or 1
        lines = ["expert statistics (highest loss first):"]
        for s in ranked:
            p = 3 * d * s.d_ff
            lines.append(f"  expert {s.expert_idx:2d}: d_ff {s.d_ff:5d}  avg loss {s.avg_loss:.6f}  tokens {s.token_count}"
                         f"  params {p:,} ({100 * p / total:.1f} %)")
        w = [s.d_ff for s in ranked]
        lines.append(f"  total params {total:,}; d_ff min {min(w)} max {max(w)} mean {sum(w) / len(w):.0f}")
        return "\n".join(lines)


def print_active_params_report(layers: Dict[int, DynamicExpertLayer], top_k: int = 2,
                               usage: Optional[Dict[int, torch.Tensor]] = None) -> Dict[int, Dict[str, float]]:
    """Total and expected-active expert parameters per layer (reference: dynamic_experts.py:421-446)."""
    out = {}
    for i, layer in sorted(layers.items()):
        act = layer.get_avg_active_params(top_k, usage.get(i) if usage else None)
        out[i] = {"total": layer.get_total_params(), "active": act, "widths": list(layer.d_ffs)}
        print(f"  layer {i}: total {out[i]['total']:,}  active/token {act:,.0f}  widths {min(layer.d_ffs)}..{max(layer.d_ffs)}")
    return out


@torch.no_grad()
def reallocate_expert_layer(layer: DynamicExpertLayer, plan=None, device=None, new_d_ff=None) -> DynamicExpertLayer:
    """Resize the experts of ``layer`` in place.  ``plan``: {expert: new width}; a list of one width per expert
    (the reference's ``new_d_ff``, dynamic_experts.py:375-418) is taken as a plan for every expert.  ``device``
    moves the layer there afterwards."""
    plan = new_d_ff if plan is None else plan
    if isinstance(plan, (list, tuple)):
        plan = {e: int(f) for e, f in enumerate(plan) if int(f) != layer.d_ffs[e]}
    for e, f in plan.items():
        a, b, c = interpolate_expert_weights(layer.w1[e].data, layer.w2[e].data, layer.w3[e].data, f)
        layer.w1[e], layer.w2[e], layer.w3[e] = nn.Parameter(a.contiguous()), nn.Parameter(b.contiguous()), nn.Parameter(c.contiguous())
        layer.d_ffs[e] = f
    return layer.to(device) if device is not None else layer

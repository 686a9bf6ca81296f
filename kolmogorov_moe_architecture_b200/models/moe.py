"""Mixture-of-Experts FFN: routers, stacked experts and ``MoELayer``
(reference: moe_arch/model/moe.py:161-950).

State-dict names and layouts match the reference: ``router.router.{0,2}.weight``
and ``grouped_experts.{w1,w2,w3}`` with w1, w2 of shape (E, d, f) and w3 (E, f, d).
What differs is execution: the token-choice path never pads to the largest
expert, never synchronises with the host, and runs as one grouped kernel
(``ops.grouped_swiglu``) instead of scatter + 3 bmm + gather + index_add.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .linear import Linear


def _init_stacked(w: torch.Tensor) -> None:
    """Per-expert kaiming-uniform(a=sqrt(5)) with fan_in = in_features (dim 1):
    U(-1/sqrt(fan_in), 1/sqrt(fan_in)) (reference: moe.py:194-211)."""
    bound = 1.0 / math.sqrt(w.shape[1])
    nn.init.uniform_(w, -bound, bound)


class Router(nn.Module):
    """Token-choice router: MLP d->128->E, softmax over experts, top-k, renormalise."""

    def __init__(self, config):
        super().__init__()
        self.d_model, self.n_experts, self.top_k = config.d_model, config.n_experts, config.moe_top_k
        self.balanced_routing = getattr(config, "moe_balanced_routing", False)
        # (load-balance weight, z-loss weight) of the auxiliary loss computed with the routing pass
        self.aux_weights = (getattr(config, "moe_load_balance_loss_weight", 0.0),
                            getattr(config, "moe_router_z_loss_weight", 0.0))
        self.last_aux, self.last_counts = None, None
        self.router = nn.Sequential(Linear(config.d_model, 128, bias=False), nn.SiLU(),
                                    Linear(128, config.n_experts, bias=False))

    @staticmethod
    def _balanced_topk_assignment(probs: torch.Tensor, top_k: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Greedy per-slot assignment under a global per-expert capacity of ``(T * k) // E`` (reference:
        moe.py:353-421).  The indices come from ``ops.balanced_assign`` (one kernel per slot on CUDA, no host
        synchronisation); the weights are gathered from ``probs`` here so they stay differentiable."""
        idx = ops.balanced_assign(probs, top_k)
        w = probs.gather(1, idx)
        return w / (w.sum(dim=-1, keepdim=True) + 1e-9), idx

    def forward(self, hidden_states: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        B, S, _ = hidden_states.shape
        logits = self.router(hidden_states)
        if self.balanced_routing:
            probs = F.softmax(logits, dim=-1).reshape(-1, self.n_experts)
            w, idx = self._balanced_topk_assignment(probs, self.top_k)
            return w.view(B, S, self.top_k), idx.view(B, S, self.top_k), logits
        # one pass: softmax -> top-k -> renormalise, plus the auxiliary-loss sums and expert counts
        w_lb, w_z = self.aux_weights if self.training else (0.0, 0.0)
        w, idx, self.last_aux, self.last_counts = ops.route_topk(logits, self.top_k, w_lb, w_z)
        return w, idx, logits


class ExpertChoiceRouter(nn.Module):
    """Each expert picks its ``ceil(S * cf / E)`` best tokens of every sequence from a
    softmax over tokens (reference: moe.py:465-530)."""

    def __init__(self, config):
        super().__init__()
        self.d_model, self.n_experts = config.d_model, config.n_experts
        self.capacity_factor = config.moe_capacity_factor
        self.router = nn.Sequential(Linear(config.d_model, 128, bias=False), nn.SiLU(),
                                    Linear(128, config.n_experts, bias=False))

    def forward(self, hidden_states: torch.Tensor):
        S = hidden_states.shape[1]
        capacity = min(S, int(math.ceil(S * self.capacity_factor / self.n_experts)))
        logits = self.router(hidden_states)
        w, tok = ops.expert_choice_route(logits, capacity)            # (B, E, C) each
        return w, tok, logits, capacity


class GroupedExperts(nn.Module):
    """Stacked SwiGLU (or 2-matrix SiLU) experts for token-choice routing."""

    def __init__(self, n_experts: int, d_model: int, d_ff: int, activation: str = "swiglu",
                 moe_dtype: str = "bf16"):
        super().__init__()
        self.n_experts, self.d_model, self.d_ff, self.activation = n_experts, d_model, d_ff, activation
        self.moe_dtype = moe_dtype
        self.w1 = nn.Parameter(torch.empty(n_experts, d_model, d_ff))
        if activation == "swiglu":
            self.w2 = nn.Parameter(torch.empty(n_experts, d_model, d_ff))
            self.w3 = nn.Parameter(torch.empty(n_experts, d_ff, d_model))
        else:
            self.w2 = nn.Parameter(torch.empty(n_experts, d_ff, d_model))
            self.w3 = None
        for w in (self.w1, self.w2, self.w3):
            if w is not None:
                _init_stacked(w)

    def forward(self, x: torch.Tensor, expert_indices: torch.Tensor, expert_weights: torch.Tensor,
                keep: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.activation == "swiglu":
            return ops.grouped_swiglu(x, self.w1, self.w2, self.w3, expert_indices, expert_weights,
                                      keep, self.moe_dtype)
        out = torch.zeros_like(x)
        for e in range(self.n_experts):
            sel = expert_indices == e
            if keep is not None:
                sel = sel & keep
            tok, slot = sel.nonzero(as_tuple=True)
            ye = F.silu(x[tok] @ self.w1[e]) @ self.w2[e]
            out.index_add_(0, tok, ye * expert_weights[tok, slot].unsqueeze(1).to(x.dtype))
        return out


class GroupedExpertsExpertChoice(nn.Module):
    """Experts for expert-choice routing: gather (B, E, C, d), batched SwiGLU with the
    stacked weights broadcast over the batch (no ``repeat`` copy, unlike the
    reference's moe.py:609-613), weighted scatter-add back."""

    def __init__(self, n_experts: int, d_model: int, d_ff: int, activation: str = "swiglu"):
        super().__init__()
        self.n_experts, self.d_model, self.d_ff, self.activation = n_experts, d_model, d_ff, activation
        self.w1 = nn.Parameter(torch.empty(n_experts, d_model, d_ff))
        if activation == "swiglu":
            self.w2 = nn.Parameter(torch.empty(n_experts, d_model, d_ff))
            self.w3 = nn.Parameter(torch.empty(n_experts, d_ff, d_model))
        else:
            self.w2 = nn.Parameter(torch.empty(n_experts, d_ff, d_model))
            self.w3 = None
        for w in (self.w1, self.w2, self.w3):
            if w is not None:
                _init_stacked(w)

    def forward(self, x: torch.Tensor, expert_weights: torch.Tensor, token_indices: torch.Tensor) -> torch.Tensor:
        B, S, d = x.shape
        _, E, C = token_indices.shape
        if self.activation == "swiglu":
            # grouped kernels: gather, batched SwiGLU GEMMs over the experts, deterministic weighted combine
            return ops.expert_choice_swiglu(x, self.w1, self.w2, self.w3, expert_weights, token_indices)
        flat_idx = token_indices.reshape(B, E * C)
        xin = torch.gather(x, 1, flat_idx.unsqueeze(-1).expand(-1, -1, d)).view(B, E, C, d)
        y = torch.matmul(F.silu(torch.matmul(xin, self.w1)), self.w2)
        y = (y * expert_weights.unsqueeze(-1).to(y.dtype)).view(B, E * C, d)
        out = torch.zeros_like(x)
        return out.scatter_add(1, flat_idx.unsqueeze(-1).expand(-1, -1, d), y)


class MoELayer(nn.Module):
    """MoE FFN with token-choice or expert-choice routing and the ``batched``,
    ``sparse`` or ``expert_parallel`` execution choices of the reference config.

    ``batched`` and ``sparse`` share one grouped kernel here (they are numerically
    the same function; the reference's split is an implementation detail), and
    keep their distinct parameter containers so checkpoints load.  Auxiliary loss
    (training only): ``w_lb * E * sum f_i P_i + w_z * mean(logsumexp^2)`` for token
    choice, z-loss only for expert choice.
    """

    def __init__(self, config, layer_idx: int, process_group=None):
        super().__init__()
        self.config, self.layer_idx = config, layer_idx
        self.n_experts, self.top_k = config.n_experts, config.moe_top_k
        self.capacity_factor = config.moe_capacity_factor
        self.routing_type = getattr(config, "moe_routing", "token_choice")
        self.implementation = getattr(config, "moe_implementation", "batched")
        self.drop_tokens = getattr(config, "moe_drop_tokens", False)
        self.router = None
        self.grouped_experts = None
        self.grouped_experts_ec = None
        self.expert_parallel_layer = None
        self._use_expert_parallel = self.implementation == "expert_parallel"
        if self._use_expert_parallel:
            from .sparse_moe import ExpertParallelMoE
            self.expert_parallel_layer = ExpertParallelMoE(config, layer_idx, process_group)
        elif self.routing_type == "expert_choice":
            self.router = ExpertChoiceRouter(config)
            self.grouped_experts_ec = GroupedExpertsExpertChoice(
                config.n_experts, config.d_model, config.d_ff_expert, config.ffn_activation)
        else:
            self.router = Router(config)
            if self.implementation == "sparse":
                from .sparse_moe import SparseGroupedExpertsPyTorch
                self.grouped_experts = SparseGroupedExpertsPyTorch(
                    config.n_experts, config.d_model, config.d_ff_expert,
                    moe_dtype=getattr(config, "moe_dtype", "bf16"))
            else:
                self.grouped_experts = GroupedExperts(
                    config.n_experts, config.d_model, config.d_ff_expert, config.ffn_activation,
                    moe_dtype=getattr(config, "moe_dtype", "bf16"))
        self.experts = None
        self.load_balance_loss_weight = config.moe_load_balance_loss_weight
        self.router_z_loss_weight = config.moe_router_z_loss_weight
        self.aux_loss = 0.0
        # device-side routing statistics of the last forward (no host sync to collect)
        self.last_expert_counts: Optional[torch.Tensor] = None
        self.last_drop_count: Optional[torch.Tensor] = None

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        if self._use_expert_parallel:
            out = self.expert_parallel_layer(hidden_states)
            self.aux_loss = self.expert_parallel_layer.aux_loss
            self.last_expert_counts = self.expert_parallel_layer.last_expert_counts
            return out
        if self.routing_type == "expert_choice":
            return self._forward_expert_choice(hidden_states)
        return self._forward_token_choice(hidden_states)

    def _forward_token_choice(self, hidden_states: torch.Tensor) -> torch.Tensor:
        B, S, d = hidden_states.shape
        w, idx, logits = self.router(hidden_states)
        idx_f, w_f = idx.reshape(-1, self.top_k), w.reshape(-1, self.top_k)
        keep = None
        if self.drop_tokens:
            cap = int(math.ceil(self.capacity_factor * idx_f.numel() / self.n_experts))
            keep = ops.capacity_keep_mask(idx_f, self.n_experts, cap)
            self.last_drop_count = (~keep).sum()
        out = self.grouped_experts(hidden_states.reshape(-1, d), idx_f, w_f, keep).view(B, S, d)
        if self.router.last_counts is not None:
            self.last_expert_counts = self.router.last_counts.detach()
            self.aux_loss = self.router.last_aux if self.training else 0.0
            self.router.last_aux = self.router.last_counts = None
        else:                                   # balanced assignment: separate passes
            with torch.no_grad():
                self.last_expert_counts = torch.bincount(idx_f.reshape(-1), minlength=self.n_experts)
            self.aux_loss = ops.moe_aux_loss(logits, idx, self.n_experts, self.load_balance_loss_weight,
                                             self.router_z_loss_weight) if self.training else 0.0
        return out

    def _forward_expert_choice(self, hidden_states: torch.Tensor) -> torch.Tensor:
        w, tok, logits, _cap = self.router(hidden_states)
        out = self.grouped_experts_ec(hidden_states, w, tok)
        if self.training and self.router_z_loss_weight > 0:
            self.aux_loss = self.router_z_loss_weight * self._compute_router_z_loss(logits)
        else:
            self.aux_loss = 0.0
        return out

    def _compute_router_z_loss(self, router_logits: torch.Tensor) -> torch.Tensor:
        return (torch.logsumexp(router_logits, dim=-1) ** 2).mean()

    def _compute_load_balance_loss(self, router_logits: torch.Tensor, selected: torch.Tensor) -> torch.Tensor:
        return ops.moe_aux_loss(router_logits, selected, self.n_experts, 1.0, 0.0)

    def get_expert_utilization(self) -> Dict[str, float]:
        """Utilisation of the last forward (the reference's method is an empty stub,
        moe.py:941-950).  Reads the device counters, so it synchronises; call it at
        logging time only."""
        if self.last_expert_counts is None:
            return {}
        c = self.last_expert_counts.float()
        frac = c / c.sum().clamp(min=1)
        ent = -(frac * (frac + 1e-10).log()).sum() / math.log(self.n_experts)
        out = {"entropy": float(ent), "max_usage": float(frac.max()), "min_usage": float(frac.min())}
        if self.last_drop_count is not None:
            out["dropped"] = float(self.last_drop_count)
        return out


class Expert(nn.Module):
    """One expert as a module of its own: ``ExpertFFN(d_model, d_ff_expert)`` on (n_tokens, d_model) rows
    (reference: moe_arch/model/moe.py:297-324).  The layers of this framework keep their experts stacked in
    ``GroupedExperts``; this class is for code that builds or inspects a single expert."""

    def __init__(self, config):
        super().__init__()
        from .ffn import ExpertFFN
        self.expert_ffn = ExpertFFN(config.d_model, config.d_ff_expert, config.ffn_activation, config.dropout)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.expert_ffn(x)

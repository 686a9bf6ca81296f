"""Mamba sequence mixers: ``MambaBlock``, ``MambaExpert`` and ``RoutingMamba``.

The reference delegates the block to the external ``mamba_ssm`` package and, when
that is missing, silently substitutes a gated depthwise convolution with no
state-space scan (reference: moe_arch/model/mamba.py:22-98).  Here the selective
scan block is implemented natively (``Mamba``), with the parameter names and
shapes the ``mamba_ssm`` module uses, so checkpoints trained with the reference
plus ``mamba_ssm`` load directly; the convolution-only variant (``SimpleSSM``) is
kept for checkpoints trained without it (``config.mamba_impl = "simple"``).
"""
from __future__ import annotations

import math
from typing import Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .linear import Linear


class Mamba(nn.Module):
    """Selective state-space block: in_proj -> causal depthwise conv + SiLU ->
    x_proj (dt, B, C) -> dt_proj -> selective scan (A = -exp(A_log), skip D, gate
    silu(z)) -> out_proj.  All activations stay channels-last (B, S, C)."""

    def __init__(self, d_model: int, d_state: int = 16, d_conv: int = 4, expand: int = 2,
                 dt_min: float = 0.001, dt_max: float = 0.1, dt_init_floor: float = 1e-4):
        super().__init__()
        self.d_model, self.d_state, self.d_conv, self.expand = d_model, d_state, d_conv, expand
        self.d_inner = expand * d_model
        self.dt_rank = math.ceil(d_model / 16)
        self.in_proj = Linear(d_model, 2 * self.d_inner, bias=False)
        self.conv1d = nn.Conv1d(self.d_inner, self.d_inner, kernel_size=d_conv, groups=self.d_inner,
                                padding=d_conv - 1, bias=True)
        self.x_proj = Linear(self.d_inner, self.dt_rank + 2 * d_state, bias=False)
        self.dt_proj = Linear(self.dt_rank, self.d_inner, bias=True)
        std = self.dt_rank ** -0.5
        nn.init.uniform_(self.dt_proj.weight, -std, std)
        dt = torch.exp(torch.rand(self.d_inner) * (math.log(dt_max) - math.log(dt_min))
                       + math.log(dt_min)).clamp(min=dt_init_floor)
        with torch.no_grad():
            self.dt_proj.bias.copy_(dt + torch.log(-torch.expm1(-dt)))
        A = torch.arange(1, d_state + 1, dtype=torch.float32).repeat(self.d_inner, 1)
        self.A_log = nn.Parameter(torch.log(A))
        self.D = nn.Parameter(torch.ones(self.d_inner))
        self.out_proj = Linear(self.d_inner, d_model, bias=False)

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        xz = self.in_proj(hidden_states)
        x, z = xz.chunk(2, dim=-1)
        x = ops.causal_conv1d(x, self.conv1d.weight.squeeze(1), self.conv1d.bias, activation=True)
        x_dbl = self.x_proj(x)
        dt, Bm, Cm = torch.split(x_dbl, [self.dt_rank, self.d_state, self.d_state], dim=-1)
        delta = ops.linear(dt, self.dt_proj.weight)          # bias is added inside the scan
        A = -torch.exp(self.A_log.float())
        y = ops.selective_scan(x, delta, A, Bm, Cm, self.D.float(), z,
                               self.dt_proj.bias.float(), delta_softplus=True)
        return self.out_proj(y)


class SimpleSSM(nn.Module):
    """The scan-free fallback block of the reference (mamba.py:54-86): in_proj to
    (z, x), depthwise causal conv k=4 on x, silu(x) * silu(z), out_proj."""

    def __init__(self, d_model: int, d_inner: int):
        super().__init__()
        self.in_proj = Linear(d_model, d_inner * 2, bias=False)
        self.conv1d = nn.Conv1d(d_inner, d_inner, kernel_size=4, padding=3, groups=d_inner)
        self.out_proj = Linear(d_inner, d_model, bias=False)
        self.act = nn.SiLU()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        z, x = self.in_proj(x).chunk(2, dim=-1)
        x = ops.causal_conv1d(x, self.conv1d.weight.squeeze(1), self.conv1d.bias, activation=True)
        return self.out_proj(ops.swiglu(z, x))


def mamba_forward_batched(mixers, hidden_states: torch.Tensor) -> torch.Tensor:
    """All of ``mixers`` (``Mamba`` modules of equal shape) on the same (B, S, d) input in one pass:
    returns (U, B, S, d).  The projections are batched GEMMs over the stacked weights; convolution and
    scan run once on the (U * B, S, C) stack, each slice of B batch entries with its own mixer's
    parameters (the ops take (U, C, ...) parameter sets).  Same arithmetic as calling the mixers one by one."""
    m0 = mixers[0]
    U = len(mixers)
    B, S, d = hidden_states.shape
    C, N, R = m0.d_inner, m0.d_state, m0.dt_rank
    st = lambda f: torch.stack([f(m) for m in mixers])
    x2 = hidden_states.reshape(1, B * S, d)
    xz = torch.matmul(x2, st(lambda m: m.in_proj.weight).transpose(1, 2)).reshape(U * B, S, 2 * C)
    x, z = xz[..., :C], xz[..., C:]
    x = ops.causal_conv1d(x, st(lambda m: m.conv1d.weight.squeeze(1)), st(lambda m: m.conv1d.bias), activation=True)
    x_dbl = torch.bmm(x.reshape(U, B * S, C), st(lambda m: m.x_proj.weight).transpose(1, 2))
    dt, Bm, Cm = torch.split(x_dbl, [R, N, N], dim=-1)
    delta = torch.bmm(dt, st(lambda m: m.dt_proj.weight).transpose(1, 2)).reshape(U * B, S, C)
    A = -torch.exp(st(lambda m: m.A_log).float())
    y = ops.selective_scan(x, delta, A, Bm.reshape(U * B, S, N), Cm.reshape(U * B, S, N),
                           st(lambda m: m.D).float(), z, st(lambda m: m.dt_proj.bias).float(), delta_softplus=True)
    out = torch.bmm(y.reshape(U, B * S, C), st(lambda m: m.out_proj.weight).transpose(1, 2))
    return out.reshape(U, B, S, d)


class MambaBlock(nn.Module):
    """Holds the mixer under the attribute ``mamba`` (state-dict prefix ``mamba.``)."""

    def __init__(self, config):
        super().__init__()
        self.config = config
        self.d_model, self.d_state = config.d_model, config.ssm_state_dim
        self.d_conv, self.expand = 4, config.ssm_expansion
        if getattr(config, "mamba_impl", "mamba") == "simple":
            self.mamba = SimpleSSM(self.d_model, self.expand * self.d_model)
            self.using_mamba_ssm = False
        else:
            self.mamba = Mamba(self.d_model, self.d_state, self.d_conv, self.expand)
            self.using_mamba_ssm = True

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        return self.mamba(hidden_states)


class MambaExpert(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.mamba = MambaBlock(config)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.mamba(x)


class RoutingMamba(nn.Module):
    """MoE over whole Mamba blocks (reference: mamba.py:126-361).

    A 2-layer MLP router scores experts per token (softmax, top-k, renormalise).
    Every expert that any token selected processes the full (B, S, d) sequence;
    outputs are mixed per token with the routing weights.  The per-token mixing
    weight of expert e is ``sum_k w[t,k] * [idx[t,k] == e]``, computed for all
    experts at once with a scatter instead of the reference's Python loops over
    ``unique(experts)`` x ``top_k`` (mamba.py:266-304).  With selective-scan experts all
    experts run in one stacked pass (one convolution and one scan launch for the layer, no
    host read); the per-expert loop remains for the ``SimpleSSM`` experts, where experts
    nobody selected are skipped by reading the usage mask once.
    """

    def __init__(self, config, layer_idx: int):
        super().__init__()
        self.config, self.layer_idx = config, layer_idx
        self.n_experts, self.top_k, self.d_model = config.n_experts, config.moe_top_k, config.d_model
        self.experts = nn.ModuleList([MambaExpert(config) for _ in range(config.n_experts)])
        self.router = nn.Sequential(Linear(config.d_model, 128, bias=False), nn.SiLU(),
                                    Linear(128, config.n_experts, bias=False))
        self.load_balance_loss_weight = config.moe_load_balance_loss_weight
        self.router_z_loss_weight = config.moe_router_z_loss_weight
        self.aux_loss = 0.0
        # one batched pass over the selected experts instead of one pass per expert
        import os
        self.batched = os.environ.get("KMOE_ROM_BATCHED", "1") != "0"

    def _route(self, hidden_states: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        logits = self.router(hidden_states)
        w_lb, w_z = (self.load_balance_loss_weight, self.router_z_loss_weight) if self.training else (0.0, 0.0)
        w, idx, self._aux, self._counts = ops.route_topk(logits, self.top_k, w_lb, w_z)
        return w, idx, logits

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        w, idx, logits = self._route(hidden_states)
        mix = torch.zeros(*hidden_states.shape[:2], self.n_experts, dtype=w.dtype, device=w.device)
        mix = mix.scatter_add(-1, idx, w)                       # (B, S, E), differentiable in w
        mixers = [ex.mamba.mamba for ex in self.experts]
        if self.batched and all(isinstance(m, Mamba) for m in mixers):
            # every expert runs (an expert nobody selected is mixed in with weight 0, the value the
            # reference's skip gives), so no usage mask has to reach the host
            ys = mamba_forward_batched(mixers, hidden_states)                       # (E, B, S, d)
            out = (mix.permute(2, 0, 1).unsqueeze(-1).to(hidden_states.dtype) * ys).sum(0)
        else:
            used = (self._counts > 0).tolist()                  # one host read for all experts
            sel = [e for e in range(self.n_experts) if used[e]]
            out = torch.zeros_like(hidden_states)
            for e in sel:
                out = out + mix[..., e:e + 1].to(hidden_states.dtype) * self.experts[e](hidden_states)
        self.aux_loss = self._aux if self.training else 0.0
        return out

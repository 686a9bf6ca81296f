"""Pre-norm residual block (reference: moe_arch/model/layers.py:22-209).

    x = x + drop(mixer(norm(x)))                      mixer: GQA | Mamba | RoutingMamba
    x = x + drop(ffn(norm(x)))                        ffn:   dense | MoE

Mixture-of-Depths applies to the FFN half only, and only in training mode: the
router keeps k tokens per sequence, the FFN runs on those, the result is scaled
by the router weight and scattered back; unselected tokens keep the residual.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .attention import GroupedQueryAttention
from .embeddings import get_norm_layer
from .ffn import get_ffn_module
from .. import ops
from .mamba import MambaBlock, RoutingMamba
from .mod import MoDRouter
from .moe import MoELayer


class TransformerBlock(nn.Module):
    def __init__(self, config, layer_idx: int):
        super().__init__()
        self.config, self.layer_idx = config, layer_idx
        mixer, ffn = config.layer_plan(layer_idx)
        self.mixer_kind, self.ffn_kind = mixer, ffn
        self.use_mamba = mixer in ("mamba", "routing_mamba")
        self.use_moe = layer_idx in config.moe_layers
        self.use_mod = config.mod_enabled
        self.seq_norm = get_norm_layer(config)
        if mixer == "routing_mamba":
            self.seq_layer = RoutingMamba(config, layer_idx)
        elif mixer == "mamba":
            self.seq_layer = MambaBlock(config)
        else:
            self.seq_layer = GroupedQueryAttention(config)
        self.ffn_norm = get_norm_layer(config)
        if ffn == "moe":
            self.ffn = MoELayer(config, layer_idx)
        else:
            self.ffn = get_ffn_module(config.d_model, config.d_ff, config.ffn_activation, config.dropout)
        self.ffn_mod_router = MoDRouter(config) if self.use_mod else None
        self.residual_dropout = nn.Dropout(config.residual_dropout)
        self.aux_loss = 0.0
        from .embeddings import RMSNorm
        self._rms = isinstance(self.seq_norm, RMSNorm) and isinstance(self.ffn_norm, RMSNorm)

    def _ffn_with_mod(self, h: torch.Tensor, residual: torch.Tensor):
        """Kept tokens go through the FFN; their weighted outputs are added onto the residual stream
        (gather -> FFN -> residual + scatter(w * out), each a single pass)."""
        picked, sorted_idx, weights = self.ffn_mod_router.route_and_gather(h)
        out = ops.mod_combine(residual, self.ffn(picked), weights, sorted_idx)
        return out, self.ffn_mod_router.aux_loss

    def forward(self, hidden_states: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                position_ids: Optional[torch.Tensor] = None, return_aux_loss: bool = False):
        aux = 0.0
        fused_norms = self._rms and hidden_states.is_cuda
        if fused_norms:
            # the residual stream passes through the norm op, which sums its two gradient paths in one kernel
            hidden_states, h = ops.residual_rmsnorm(hidden_states, None, self.seq_norm.weight, self.seq_norm.eps)
        else:
            h = self.seq_norm(hidden_states)
        if self.use_mamba:
            mixed = self.seq_layer(h)
        else:
            mixed = self.seq_layer(h, attention_mask=attention_mask, position_ids=position_ids)
        if self.mixer_kind == "routing_mamba" and self.training:
            aux = aux + self.seq_layer.aux_loss

        if fused_norms and self.residual_dropout.p == 0.0:
            # residual add + pre-FFN norm in one pass
            hidden_states, h = ops.residual_rmsnorm(hidden_states, mixed, self.ffn_norm.weight, self.ffn_norm.eps)
        else:
            hidden_states = hidden_states + self.residual_dropout(mixed)
            h = self.ffn_norm(hidden_states)
        if self.use_mod and self.training and self.residual_dropout.p == 0.0:
            hidden_states, mod_aux = self._ffn_with_mod(h, hidden_states)
            aux = aux + mod_aux
        elif self.use_mod and self.training:
            delta, mod_aux = self._ffn_with_mod(h, torch.zeros_like(hidden_states))
            aux = aux + mod_aux
            hidden_states = hidden_states + self.residual_dropout(delta)
        else:
            hidden_states = hidden_states + self.residual_dropout(self.ffn(h))
        if self.ffn_kind == "moe" and self.training:
            aux = aux + self.ffn.aux_loss

        self.aux_loss = aux if self.training else 0.0
        if return_aux_loss and self.training:
            if not torch.is_tensor(aux):
                aux = torch.tensor(aux, device=hidden_states.device, dtype=hidden_states.dtype)
            return hidden_states, aux
        return hidden_states

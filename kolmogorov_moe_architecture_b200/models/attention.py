"""Grouped-query attention (reference: moe_arch/model/attention.py:21-249).

Differences that do not change results: K/V are never expanded to ``n_heads``
(the kernel and the eager oracle both index the shared KV head), and the causal
kernel is used whenever no additive mask is given.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from .linear import Linear
from .embeddings import RotaryPositionalEmbedding


class GroupedQueryAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.d_model = config.d_model
        self.n_heads, self.n_kv_heads, self.head_dim = config.n_heads, config.n_kv_heads, config.head_dim
        self.n_groups = self.n_heads // self.n_kv_heads
        assert self.d_model == self.n_heads * self.head_dim, "d_model must equal n_heads * head_dim"
        self.q_proj = Linear(self.d_model, self.n_heads * self.head_dim, bias=False)
        self.k_proj = Linear(self.d_model, self.n_kv_heads * self.head_dim, bias=False)
        self.v_proj = Linear(self.d_model, self.n_kv_heads * self.head_dim, bias=False)
        self.o_proj = Linear(self.n_heads * self.head_dim, self.d_model, bias=False)
        self.rope = RotaryPositionalEmbedding(self.head_dim, config.max_seq_len, config.rope_theta,
                                              config.rope_scaling)
        self.attention_dropout = config.attention_dropout
        self.use_flash_attention = config.use_flash_attention

    def forward(self, hidden_states: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                position_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        B, S, _ = hidden_states.shape
        if self.q_proj.bias is None and self.k_proj.bias is None and self.v_proj.bias is None:
            # the three projections of the same input as one autograd node: dx is accumulated inside the GEMMs
            q, k, v = ops.linear_multi(hidden_states, [self.q_proj.weight, self.k_proj.weight, self.v_proj.weight])
        else:
            q, k, v = self.q_proj(hidden_states), self.k_proj(hidden_states), self.v_proj(hidden_states)
        q = q.view(B, S, self.n_heads, self.head_dim)
        k = k.view(B, S, self.n_kv_heads, self.head_dim)
        v = v.view(B, S, self.n_kv_heads, self.head_dim)
        q, k = self.rope(q, k, position_ids)
        if hasattr(attention_mask, "doc_start"):            # packed documents: boundaries, not a dense mask
            out = ops.attention(q, k, v, causal=True, dropout_p=self.attention_dropout, training=self.training,
                                doc_start=attention_mask.doc_start)
            return self.o_proj(out.reshape(B, S, self.n_heads * self.head_dim))
        if attention_mask is not None and attention_mask.dim() == 2:
            m = attention_mask[:, None, None, :].to(q.dtype)
            attention_mask = (1.0 - m) * torch.finfo(q.dtype).min
        out = ops.attention(q, k, v, causal=True, attn_mask=attention_mask,
                            dropout_p=self.attention_dropout, training=self.training)
        return self.o_proj(out.reshape(B, S, self.n_heads * self.head_dim))

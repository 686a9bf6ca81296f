"""Token embedding, rotary position tables and normalisation layers.

Parameter names match the reference so state dicts interchange
(reference: moe_arch/model/embeddings.py:13-213).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

from .. import ops


class TokenEmbedding(nn.Module):
    """``token_embedding.embedding.weight`` of shape (vocab, d_model)."""

    def __init__(self, config):
        super().__init__()
        self.embedding = nn.Embedding(config.vocab_size, config.d_model)

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        return self.embedding(input_ids)


class RotaryPositionalEmbedding(nn.Module):
    """Rotate-half RoPE with tables precomputed to ``max_seq_len``.

    The tables are non-persistent buffers (not part of the checkpoint), as in
    the reference (embeddings.py:69,79-80).  ``scaling`` is accepted and kept
    but, like the reference (embeddings.py:53), not applied.
    """

    def __init__(self, dim: int, max_seq_len: int = 2048, theta: float = 10000.0,
                 scaling: Optional[dict] = None):
        super().__init__()
        self.dim, self.max_seq_len, self.theta, self.scaling = dim, max_seq_len, theta, scaling
        cos, sin = ops.rope_tables(dim, max_seq_len, theta)
        inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2).float() / dim))
        self.register_buffer("inv_freq", inv_freq, persistent=False)
        self.register_buffer("cos_cached", cos, persistent=False)
        self.register_buffer("sin_cached", sin, persistent=False)

    def tables(self, seq_len: int, position_ids: Optional[torch.Tensor]):
        if position_ids is None:
            if self.cos_cached.is_cuda:
                # the kernel reads fp32 tables: convert the (possibly bf16-cast) buffers once, not on every call
                key = (self.cos_cached.data_ptr(), self.cos_cached.dtype, seq_len)
                hit = getattr(self, "_f32_tables", None)
                if hit is None or hit[0] != key:
                    hit = (key, self.cos_cached[:seq_len].float().contiguous(),
                           self.sin_cached[:seq_len].float().contiguous())
                    self._f32_tables = hit
                return hit[1], hit[2]
            return self.cos_cached[:seq_len], self.sin_cached[:seq_len]
        return self.cos_cached[position_ids], self.sin_cached[position_ids]

    def forward(self, q: torch.Tensor, k: torch.Tensor,
                position_ids: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        cos, sin = self.tables(q.shape[1], position_ids)
        return ops.rope_apply(q, cos, sin), ops.rope_apply(k, cos, sin)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps)


def get_norm_layer(config) -> nn.Module:
    if config.norm_type == "rmsnorm":
        return RMSNorm(config.d_model, config.norm_eps)
    if config.norm_type == "layernorm":
        return nn.LayerNorm(config.d_model, eps=config.norm_eps)
    raise ValueError(f"Unknown norm_type: {config.norm_type}")

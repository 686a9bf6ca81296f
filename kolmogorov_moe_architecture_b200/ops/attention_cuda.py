"""Causal GQA attention on CUDA tensors."""
from __future__ import annotations

import torch
import torch.nn.functional as F


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True) -> torch.Tensor:
    """q (B,S,H,D); k, v (B,S,Hkv,D) -> (B,S,H,D)."""
    out = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                         is_causal=causal, enable_gqa=True)
    return out.transpose(1, 2).contiguous()

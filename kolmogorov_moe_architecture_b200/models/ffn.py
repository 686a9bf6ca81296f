"""Dense feed-forward blocks (reference: moe_arch/model/ffn.py:17-162)."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .linear import Linear


class SwiGLU(nn.Module):
    """w3(silu(w1 x) * w2 x); weights in nn.Linear (out, in) layout."""

    def __init__(self, d_model: int, d_ff: int, dropout: float = 0.0):
        super().__init__()
        self.w1 = Linear(d_model, d_ff, bias=False)
        self.w2 = Linear(d_model, d_ff, bias=False)
        self.w3 = Linear(d_ff, d_model, bias=False)
        self.dropout = nn.Dropout(dropout)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.dropout(ops.dense_swiglu(x, self.w1.weight, self.w2.weight, self.w3.weight))


class StandardFFN(nn.Module):
    def __init__(self, d_model: int, d_ff: int, activation: str = "gelu", dropout: float = 0.0):
        super().__init__()
        self.w1 = Linear(d_model, d_ff, bias=False)
        self.w2 = Linear(d_ff, d_model, bias=False)
        self.act = {"gelu": F.gelu, "silu": F.silu, "relu": F.relu}[activation]
        self.dropout = nn.Dropout(dropout)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.dropout(self.w2(self.act(self.w1(x))))


def get_ffn_module(d_model: int, d_ff: int, activation: str = "swiglu", dropout: float = 0.0) -> nn.Module:
    if activation == "swiglu":
        return SwiGLU(d_model, d_ff, dropout)
    if activation in ("gelu", "silu", "relu"):
        return StandardFFN(d_model, d_ff, activation, dropout)
    raise ValueError(f"Unknown activation: {activation}")


class ExpertFFN(nn.Module):
    """A single stand-alone expert (kept for API parity, ffn.py:136-162)."""

    def __init__(self, d_model: int, d_ff: int = None, activation: str = "swiglu", dropout: float = 0.0,
                 d_ff_expert: int = None):
        super().__init__()
        width = d_ff_expert if d_ff is None else d_ff          # ``d_ff_expert``: the reference's keyword
        assert width is not None, "the expert width is required"
        self.ffn = get_ffn_module(d_model, width, activation, dropout)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.ffn(x)

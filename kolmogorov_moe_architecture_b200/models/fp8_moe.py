"""FP8 layers (API of the reference's ``moe_arch/model/fp8_moe.py``): ``FP8Linear``,
``FP8GroupedExperts``, ``FP8MoELayer``, ``is_fp8_available``.

The reference simulates FP8 (per-tensor delayed scaling, clamp to +-448, bf16 multiply).  Here the
number format is real block-scaled MXFP8 (e4m3 values, 1x32 power-of-two scales, see
``ops/mxfp8.py``); unlike the reference the experts are also selectable from the model config
(``moe_dtype: mxfp8``).  State-dict names (``weight``, ``w1/w2/w3`` and the scale / amax-history
buffers) are kept so reference checkpoints load.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..ops import eager
from ..ops.mxfp8 import grouped_swiglu_mxfp8, linear_mx
from .linear import Linear

FP8_E4M3 = torch.float8_e4m3fn
FP8_E5M2 = torch.float8_e5m2


def is_fp8_available() -> bool:
    """True on GPUs with fp8 tensor cores (sm_89, sm_90, sm_100 and later)."""
    if not torch.cuda.is_available():
        return False
    p = torch.cuda.get_device_properties(0)
    return p.major >= 9 or (p.major == 8 and p.minor >= 9)


class FP8Linear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = False, device=None, dtype=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, device=device, dtype=dtype or torch.bfloat16))
        self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype or torch.bfloat16)) if bias else None
        for n in ("input_scale", "weight_scale", "output_scale"):
            self.register_buffer(n, torch.tensor(1.0))
        self.register_buffer("input_amax_history", torch.zeros(16))
        self.register_buffer("weight_amax_history", torch.zeros(16))
        self.history_idx = 0
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return linear_mx(x, self.weight, self.bias)


class FP8GroupedExperts(nn.Module):
    def __init__(self, n_experts: int, d_model: int, d_ff: int):
        super().__init__()
        self.n_experts, self.d_model, self.d_ff = n_experts, d_model, d_ff
        self.w1 = nn.Parameter(torch.empty(n_experts, d_model, d_ff, dtype=torch.bfloat16))
        self.w2 = nn.Parameter(torch.empty(n_experts, d_model, d_ff, dtype=torch.bfloat16))
        self.w3 = nn.Parameter(torch.empty(n_experts, d_ff, d_model, dtype=torch.bfloat16))
        for n in ("w1_scale", "w2_scale", "w3_scale"):
            self.register_buffer(n, torch.ones(n_experts))
        self.register_buffer("input_scale", torch.tensor(1.0))
        for w in (self.w1, self.w2, self.w3):
            nn.init.uniform_(w, -1.0 / math.sqrt(w.shape[1]), 1.0 / math.sqrt(w.shape[1]))

    def forward(self, x: torch.Tensor, expert_indices: torch.Tensor, expert_weights: torch.Tensor) -> torch.Tensor:
        return grouped_swiglu_mxfp8(x, self.w1, self.w2, self.w3, expert_indices, expert_weights)


class FP8MoELayer(nn.Module):
    """Router ``Linear(d, E)`` (softmax, top-k, renormalise) + MXFP8 experts; aux = E * sum f_i P_i * 0.01."""

    def __init__(self, d_model: int, d_ff: int, n_experts: int, top_k: int = 2):
        super().__init__()
        self.d_model, self.d_ff, self.n_experts, self.top_k = d_model, d_ff, n_experts, top_k
        self.router = Linear(d_model, n_experts, bias=False)
        self.experts = FP8GroupedExperts(n_experts, d_model, d_ff)
        self.aux_loss = 0.0

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        flat = x.reshape(-1, self.d_model)
        logits = self.router(flat.to(self.router.weight.dtype))
        w, idx = eager.topk_softmax_route(logits, self.top_k)
        if self.training:
            self.aux_loss = eager.moe_aux_loss(logits, idx, self.n_experts, 0.01, 0.0)
        return self.experts(flat, idx, w.to(flat.dtype)).view(shape)
